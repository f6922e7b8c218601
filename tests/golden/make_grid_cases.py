"""Exports the GEOMETRY of the reference's correctness grid as a small JSON fixture.

    REFERENCE=/path/to/pth-flash-attn python tests/golden/make_grid_cases.py

The reference describes its GPU correctness grid as data (tests/gpu/grid_cases.py:
``all_cases()``: paging, rows, batches, splits, long contexts, scales, dtypes, stride fuzz,
windows).  This script imports that module from a reference checkout and writes, for every
case, the fields that define its shape - query and sequence lengths, head geometry, page
size and layout, padding, split count, window, dtypes - to ``grid_cases.json``.  The test
that reads the fixture (tests/test_gpu_9_reference_grid.py) builds each case with this
repository's own oracle and data, so no reference code or data travels with the fixture.
"""
from __future__ import annotations

import json
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
# the reference checkout: $REFERENCE, else a directory `reference` next to this repository
REFERENCE = Path(os.environ.get("REFERENCE", HERE.parents[2] / "reference"))
sys.path.insert(0, str(REFERENCE / "python"))
sys.path.insert(0, str(REFERENCE / "tests" / "gpu"))

import grid_cases  # noqa: E402

FIELDS = ("name", "family", "q_lens", "seq_lens", "G", "Hkv", "D", "block_size", "layout", "pad_page_bytes",
          "storage_offset_bytes", "high_block_ids", "q_dtype", "out_dtype", "num_splits", "pad_rows", "strided_io",
          "window", "causal", "tier")


def main() -> None:
    cases = []
    for c in grid_cases.all_cases():
        d = {k: getattr(c, k) for k in FIELDS}
        d["q_lens"], d["seq_lens"] = list(c.q_lens), list(c.seq_lens)
        d["bq"] = c.bq
        cases.append(d)
    out = HERE / "grid_cases.json"
    out.write_text(json.dumps({"source": "tests/gpu/grid_cases.py all_cases()", "cases": cases}, separators=(",", ":")))
    print(f"{len(cases)} cases -> {out} ({out.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
