"""Shared helpers of the test-suite: golden fixtures and tolerance checks."""
from __future__ import annotations

from pathlib import Path

import numpy as np

from oracle import paged_int8_attention as orc

GOLDEN = Path(__file__).resolve().parent / "golden"

# Parity gate against the fp64 oracle: bf16 output max |d| <= 2e-2 and mean |d| <= 2e-3,
# fp32 natural-log LSE |d| <= 1e-3.
OUT_MAX_TOL = 2e-2
OUT_MEAN_TOL = 2e-3
LSE_TOL = 1e-3


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / f"{name}.npz", allow_pickle=False) as z:
        return {k: z[k] for k in z.files}


def golden_dense(g: dict) -> list[orc.DenseKV]:
    n = len(g["seq_lens"])
    return [orc.DenseKV(g[f"k_int{r}"], g[f"k_scale{r}"], g[f"v_int{r}"], g[f"v_scale{r}"])
            for r in range(n)]


def check_out(out, ref_out, valid=None, *, max_tol=OUT_MAX_TOL, mean_tol=OUT_MEAN_TOL, what="",
              relative=False):
    """The parity gate.  ``relative`` divides each error by max(1, |ref|): the gate is stated for
    unit-scale data, and a bf16 output at magnitude 16 rounds by up to 0.06 on its own."""
    out = np.asarray(out, dtype=np.float64)
    ref_out = np.asarray(ref_out, dtype=np.float64)
    if valid is not None:
        out, ref_out = out[valid], ref_out[valid]
    if out.size == 0:
        return 0.0, 0.0
    d = np.abs(out - ref_out)
    if relative:
        d = d / np.maximum(1.0, np.abs(ref_out))
    assert np.isfinite(out).all(), f"{what}: non-finite output"
    mx, mean = float(d.max()), float(d.mean())
    assert mx <= max_tol, f"{what}: max |d| {mx:.3e} > {max_tol}"
    assert mean <= mean_tol, f"{what}: mean |d| {mean:.3e} > {mean_tol}"
    return mx, mean


def check_lse(lse, ref_lse, valid=None, *, tol=LSE_TOL, what=""):
    lse = np.asarray(lse, dtype=np.float64)
    ref_lse = np.asarray(ref_lse, dtype=np.float64)
    if valid is not None:
        lse, ref_lse = lse[valid], ref_lse[valid]
    inf_ref = np.isneginf(ref_lse)
    assert np.array_equal(np.isneginf(lse), inf_ref), f"{what}: -inf rows differ"
    if (~inf_ref).any():
        d = np.abs(lse[~inf_ref] - ref_lse[~inf_ref])
        assert float(d.max()) <= tol, f"{what}: LSE max |d| {float(d.max()):.3e} > {tol}"
        return float(d.max())
    return 0.0
