#!/usr/bin/env python
"""Benchmark of the paged int8 attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config NAME] [--impl reference]

One "pass" is one call of the op over one synthetic batch (the attention launch and, when
the key range is split, the combine launch, for every launch of the workload).  A "step" is
`passes_per_step` passes, chosen at start-up so that the K timed steps take about one
second whatever K is; every number is reported per pass (= per layer of a model).

The headline workload is the long-context split-KV decode configuration: one launch of
batch 1 at context 131072 plus one launch of batch 64 at context 8192 (Hq = 32, Hkv = 8,
D = 128, block size 16, one query token per request).  The metric is the achieved cache
read bandwidth: the algorithmic KV bytes of a pass (every visible (token, KV head) cell
once, 2 D + 8 bytes each) divided by the device time of the pass.  The line's `per_config`
block holds the same measurement for every other configuration (decode, verification,
windowed drafter in GB/s; chunked prefill in TFLOP/s; the mixed batch in both), each with
the roofline that bounds it and a sampled check of its output against the CPU oracle.

With N > 1 (one process per GPU, started by torch.distributed.run) the KV heads are
sharded: rank g owns Hkv / N KV heads, the matching query heads and its own cache; there is
no collective on the data path.  Total work is fixed, so the line says "strong" scaling;
`value` is the whole job's bytes over the slowest rank's time.

Inputs are synthetic: K and V are N(0, 1) values quantised per (token, KV head) to int8 with
scale absmax / 127, written in vLLM's int8_per_token_head page layout on the device; bf16
N(0, 1) queries; seeded random block tables.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

HQ, HKV, D, BS = 32, 8, 128, 16
CELL = 2 * D + 8
HEADLINE = "long_decode"
# the six shapes the reference quotes its numbers on, then the reference's production shape (256 dims, 12 / 2
# heads, HND pages of 816 slots) in decode and chunked prefill, and decode and chunked prefill at 64 dims
PER_CONFIG = ("decode_small", "long_decode", "verify4", "drafter16", "chunked_prefill", "mixed", "decode_d256",
              "prefill_d256", "decode_d64", "prefill_d64")
TENSOR_BOUND = ("chunked_prefill", "chunked_prefill_hnd", "prefill_d256", "prefill_d256_nhd", "prefill_d64")


# --------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------
def workload_launches(name: str, seed: int = 1001):
    """The launches of a workload: dict(seq_lens, q_lens, Hq, Hkv[, window, prefill])."""
    rng = np.random.default_rng(seed)
    if name == "decode_small":  # batch 8, contexts uniform in [1, 4096]
        return [dict(seq_lens=rng.integers(1, 4097, size=8).tolist(), q_lens=[1] * 8, Hq=32, Hkv=8)]
    if name == "long_decode":  # the headline: 1 x 131072, then 64 x 8192
        return [dict(seq_lens=[131072], q_lens=[1], Hq=32, Hkv=8),
                dict(seq_lens=[8192] * 64, q_lens=[1] * 64, Hq=32, Hkv=8)]
    if name == "long_decode_b1":  # the first launch of the headline alone
        return [dict(seq_lens=[131072], q_lens=[1], Hq=32, Hkv=8)]
    if name == "long_decode_b64":  # the second launch of the headline alone
        return [dict(seq_lens=[8192] * 64, q_lens=[1] * 64, Hq=32, Hkv=8)]
    if name == "decode_d256":  # the reference's production shape: 256 dims, 6 query heads per KV head, HND pages of 816 slots
        return [dict(seq_lens=[8192] * 64, q_lens=[1] * 64, Hq=12, Hkv=2, D=256, block_size=816, layout="HND")]
    if name == "prefill_d256":  # chunked prefill at the production shape (the row-major kernel for 256 dims)
        return [dict(seq_lens=[32768] * 4, q_lens=[2048] * 4, Hq=12, Hkv=2, D=256, block_size=816, layout="HND",
                     prefill=True)]
    if name == "prefill_d256_nhd":  # the same chunks over NHD pages of 16 slots
        return [dict(seq_lens=[32768] * 4, q_lens=[2048] * 4, Hq=12, Hkv=2, D=256, prefill=True)]
    if name == "prefill_d64":  # chunked prefill at 64 dims
        return [dict(seq_lens=[32768] * 4, q_lens=[2048] * 4, Hq=32, Hkv=8, D=64, prefill=True)]
    if name == "decode_d64":  # 64 dims
        return [dict(seq_lens=[8192] * 64, q_lens=[1] * 64, Hq=32, Hkv=8, D=64)]
    if name == "verify4":  # speculative verification, 4 draft tokens
        return [dict(seq_lens=rng.integers(16384, 32769, size=32).tolist(), q_lens=[4] * 32, Hq=32, Hkv=8)]
    if name == "drafter16":  # windowed drafter, 16 tokens, window 4096
        return [dict(seq_lens=rng.integers(16384, 32769, size=32).tolist(), q_lens=[16] * 32, Hq=32,
                     Hkv=8, window=4096)]
    if name == "chunked_prefill":  # 4 chunks of 2048 tokens over 30720 cached tokens
        return [dict(seq_lens=[32768] * 4, q_lens=[2048] * 4, Hq=64, Hkv=8, prefill=True)]
    if name == "chunked_prefill_hnd":  # the same chunks over HND pages (the slots of a head together)
        return [dict(seq_lens=[32768] * 4, q_lens=[2048] * 4, Hq=64, Hkv=8, prefill=True, layout="HND")]
    if name == "mixed":  # 48 decode + 8 verify + 2 prefill requests in one launch
        dec = rng.integers(4096, 131073, size=48).tolist()
        return [dict(seq_lens=dec + [32768] * 8 + [17408] * 2, q_lens=[1] * 48 + [4] * 8 + [1024] * 2,
                     Hq=64, Hkv=8, prefill=True)]
    raise SystemExit(f"unknown --config {name}")


def kv_bytes(launch, hkv_local):
    total = 0
    w = launch.get("window", 0)
    for L, ql in zip(launch["seq_lens"], launch["q_lens"]):
        vis = L if w <= 0 else min(L, w + ql - 1)
        total += vis * hkv_local * (2 * launch.get("D", D) + 8)
    return total


def attn_flops(launch, hq_local):
    total = 0
    w = launch.get("window", 0)
    for L, ql in zip(launch["seq_lens"], launch["q_lens"]):
        if w <= 0:
            pairs = ql * (L - ql) + ql * (ql + 1) // 2
        else:
            pairs = sum(min(L - ql + i + 1, w) for i in range(ql))
        total += 4 * launch.get("D", D) * hq_local * pairs
    return total


# --------------------------------------------------------------------------
# one launch, resident on the device
# --------------------------------------------------------------------------
def _align(n, a=256):
    return (n + a - 1) // a * a


class DeviceLaunch:
    """One launch of a workload for one rank: its KV-head shard of the cache, generated on
    the device, the op's per-call inputs as views of ONE device staging buffer with a pinned
    host twin (the end-to-end leg copies it with a single transfer), and the plan."""

    def __init__(self, torch, launch, rank, world, device, seed, num_sms, sets=1):
        from pth_flash_attn_b200 import capi, host, planner, sharding

        self.torch, self.launch_spec = torch, launch
        shard = sharding.head_shard(rank, world, launch["Hq"], launch["Hkv"])
        hkv, hq = shard.num_kv_heads, shard.num_q_heads
        self.hkv, self.hq, self.G = hkv, hq, hq // hkv
        D = self.D = int(launch.get("D", globals()["D"]))
        CELL = self.cell = 2 * D + 8
        BS = self.block_size = int(launch.get("block_size", globals()["BS"]))
        self.layout = launch.get("layout", "NHD")   # HND: the slots of a head together (vLLM's packed page)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        lens, qlens = launch["seq_lens"], launch["q_lens"]
        R, T = len(lens), int(sum(qlens))
        self.R, self.T = R, T
        self.window, self.causal = launch.get("window", 0), launch.get("causal", True)
        nblk = [-(-L // BS) for L in lens]
        need, width = sum(nblk), max(nblk)
        q_max = max(qlens)
        is_prefill = bool(launch.get("prefill", False))
        if not is_prefill:
            w_ts = planner.workspace_token_splits(max_num_seqs=R, q_dec_max=q_max, Hkv=hkv, D=D, num_sms=num_sms)
        elif min(qlens) < max(qlens):
            # a mixed batch in ONE launch: its decode requests only balance if they may be cut, so
            # this caller reserves partials for the whole launch (8 pieces x T tokens)
            w_ts = 8 * T
        else:
            w_ts = 0  # prefill chunks alone are never cut
        plan = planner.plan_launch(num_tokens=T, num_reqs=R, max_query_len=q_max, G=self.G, Hkv=hkv, D=D,
                                   num_sms=num_sms, is_prefill=is_prefill, ws_token_splits=w_ts,
                                   window=self.window)
        self.plan, self.S = plan, plan.num_splits
        self.bq = plan.bq if is_prefill else min(plan.bq, q_max)
        # as the torch op does: max_query_len within one row tile = one row tile per request
        self.flags = capi.FLAG_ONE_TILE_PER_REQUEST if q_max <= self.bq else 0

        # staging layout: q | block_table | seq_lens | query_start_loc
        off_q = 0
        off_bt = _align(off_q + T * hq * D * 2)
        off_len = _align(off_bt + R * width * 4)
        off_qsl = _align(off_len + R * 4)
        self.h2d = _align(off_qsl + (R + 1) * 4)
        qsl = torch.zeros(R + 1, dtype=torch.int32)
        qsl[1:] = torch.tensor(qlens, dtype=torch.int64).cumsum(0).to(torch.int32)
        q_host = torch.randn((T, hq, D), generator=gen).to(torch.bfloat16)

        def carve(buf):
            return (buf[off_q:off_q + T * hq * D * 2].view(torch.bfloat16).view(T, hq, D),
                    buf[off_bt:off_bt + R * width * 4].view(torch.int32).view(R, width),
                    buf[off_len:off_len + R * 4].view(torch.int32),
                    buf[off_qsl:off_qsl + (R + 1) * 4].view(torch.int32))

        page = BS * hkv * CELL
        self.sets = []
        for s in range(sets):
            storage = self._quantised_cache(torch, need, hkv, device, seed + 7 * s, D, BS)
            perm = torch.randperm(need, generator=gen).to(torch.int32)
            bt = torch.zeros((R, width), dtype=torch.int32)
            k = 0
            for r, nb in enumerate(nblk):
                bt[r, :nb] = perm[k:k + nb]
                k += nb
            stage_host = torch.zeros(self.h2d, dtype=torch.uint8).pin_memory()
            hq_, hbt, hlen, hqsl = carve(stage_host)
            hq_.copy_(q_host)
            hbt.copy_(bt)
            hlen.copy_(torch.tensor(lens, dtype=torch.int32))
            hqsl.copy_(qsl)
            stage_dev = stage_host.to(device)
            dq, dbt, dlen, dqsl = carve(stage_dev)
            base = storage.data_ptr()
            slot, head = (hkv * CELL, CELL) if self.layout == "NHD" else (CELL, BS * CELL)
            views = host.CacheViews((base, page, slot, head), (base + D + 4, page, slot, head),
                                    (base + D, page, slot, head), (base + 2 * D + 4, page, slot, head),
                                    need, BS, hkv, D)
            self.sets.append(dict(storage=storage, views=views, stage_host=stage_host, stage_dev=stage_dev,
                                  q=dq, bt=dbt, lens=dlen, qsl=dqsl))
        self.out = torch.zeros((T, hq, D), dtype=torch.bfloat16, device=device)
        self.out_host = torch.empty((T, hq, D), dtype=torch.bfloat16).pin_memory()
        self.d2h = self.out_host.numel() * 2
        self.ws_o = self.ws_lse = None
        if self.S > 1:
            self.ws_o = torch.empty((self.S, T, hq, D), dtype=torch.float32, device=device)
            self.ws_lse = torch.empty((self.S, T, hq), dtype=torch.float32, device=device)
        a = self._args(0)
        self.attention_kernels, self.combine_kernels = capi.load_library().launch_count(a)
        self.kernels = self.attention_kernels + self.combine_kernels

    @staticmethod
    def _quantised_cache(torch, num_blocks, hkv, device, seed, D, BS):
        """N(0, 1) K and V quantised per (token, KV head) like the cache writer does (scale =
        max(absmax / 127, 1e-6), round half away from zero), one packed cell per (block, slot,
        head); the cells are independent random rows, so the same bytes serve as an NHD or an
        HND page (the views decide which cell is which slot and head)."""
        CELL = 2 * D + 8
        gen = torch.Generator(device=device).manual_seed(seed)
        storage = torch.empty(num_blocks * BS * hkv * CELL, dtype=torch.uint8, device=device)
        cells = storage.view(num_blocks, BS, hkv, CELL)
        step = max(1, (64 << 20) // (BS * hkv * D))  # 256 MB of fp32 at a time
        for b0 in range(0, num_blocks, step):
            b1 = min(num_blocks, b0 + step)
            for off in (0, D + 4):  # K half, V half of the cell
                x = torch.randn((b1 - b0, BS, hkv, D), device=device, generator=gen)
                scale = (x.abs().amax(-1) / 127.0).clamp_min(1e-6)
                v = x * (1.0 / scale).unsqueeze(-1)
                v = torch.where(v >= 0, v + 0.5, v - 0.5).clamp(-128.0, 127.0).trunc().to(torch.int8)
                cells[b0:b1, :, :, off:off + D] = v.view(torch.uint8)
                cells[b0:b1, :, :, off + D:off + D + 4] = scale.contiguous().view(torch.uint8).view(b1 - b0, BS, hkv, 4)
        return storage

    def _args(self, which, out=None):
        from pth_flash_attn_b200 import host

        s = self.sets[which % len(self.sets)]
        return host.fill_attn_args(s["q"], self.out if out is None else out, s["views"], s["bt"], s["lens"], s["qsl"],
                                   bq=self.bq, num_splits=self.S, softmax_scale=self.D ** -0.5, ws_o=self.ws_o,
                                   ws_lse=self.ws_lse, window=self.window, causal=self.causal)

    def launch(self, which=0, lse_out=None):
        from pth_flash_attn_b200 import host

        s = self.sets[which % len(self.sets)]
        host.attention_forward(s["q"], self.out, s["views"], s["bt"], s["lens"], s["qsl"], bq=self.bq,
                               num_splits=self.S, softmax_scale=self.D ** -0.5, ws_o=self.ws_o, ws_lse=self.ws_lse,
                               window=self.window, causal=self.causal, flags=self.flags, lse_out=lse_out)

    def launch_attention_only(self, which=0):
        """Only the attention kernel(s) of the launch (for the per-kernel roofline timing)."""
        from pth_flash_attn_b200 import capi

        lib = capi.load_library()
        rc = lib.attention(self._args(which), options=capi.make_options(capi.KERNEL_AUTO, self.flags),
                           stream=self.torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(lib.last_error())

    def launch_copy_ceiling(self, which=0):
        """The paged-copy ceiling of this launch (same bytes, same copies, no compute)."""
        from pth_flash_attn_b200 import capi

        lib = capi.load_library()
        rc = lib.copy_ceiling(self._args(which), stream=self.torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(lib.last_error())

    def e2e_pass(self, which=0):
        """Host buffers in, host buffer out: ONE pinned H2D copy of the call's inputs (queries,
        block table, lengths), the launch, D2H of out."""
        s = self.sets[which % len(self.sets)]
        s["stage_dev"].copy_(s["stage_host"], non_blocking=True)
        self.launch(which)
        self.out_host.copy_(self.out, non_blocking=True)

    def parity(self, which=0, picks_per_launch=12, seed=0):
        """Runs the launch once more, with the log-sum-exp output, on the buffers that were
        timed, and compares sampled (token, head) rows with the fp64 CPU oracle reading the
        same cache bytes.  Returns (max |d out|, mean |d out|, max |d lse|, rows)."""
        from oracle import paged_int8_attention as orc

        torch = self.torch
        s = self.sets[which % len(self.sets)]
        lse = torch.full((self.T, self.hq), float("nan"), dtype=torch.float32, device=self.out.device)
        self.out.fill_(float("nan"))
        self.launch(which, lse_out=lse)
        torch.cuda.synchronize()
        storage = s["storage"].cpu().numpy()
        D, CELL, BS = self.D, self.cell, self.block_size
        page = BS * self.hkv * CELL
        k, v, ks, vs = orc.stream_views(D, self.hkv, BS, self.layout, page, 0)
        lens = np.asarray(self.launch_spec["seq_lens"], dtype=np.int32)
        cache = orc.PagedInt8Cache(storage=storage, k=k, v=v, ks=ks, vs=vs, block_table=s["bt"].cpu().numpy(),
                                   seq_lens=lens, num_blocks=s["views"].num_blocks, block_size=BS, Hkv=self.hkv,
                                   D=D, layout=self.layout, page_bytes=page, storage_offset_bytes=0)
        qsl = s["qsl"].cpu().numpy().astype(np.int64)
        rng = np.random.default_rng(seed)
        reqs = {int(np.argmax(lens)), int(np.argmin(lens)), 0, self.R - 1}
        reqs |= set(rng.integers(0, self.R, size=picks_per_launch).tolist())
        picks = []
        for r in sorted(reqs)[:picks_per_launch]:
            for tok in {int(qsl[r]), int(qsl[r + 1]) - 1, int(rng.integers(qsl[r], qsl[r + 1]))}:
                picks.append((tok, int(rng.integers(0, self.hq))))
        q = s["q"].float().cpu().numpy()
        ref_out, ref_lse = orc.ref_attention_rows(q, cache, qsl, D ** -0.5, picks, window=self.window,
                                                  causal=self.causal)
        out = self.out.float().cpu().numpy()
        lse_h = lse.cpu().numpy()
        got = np.stack([out[t, h] for t, h in picks])
        got_lse = np.array([lse_h[t, h] for t, h in picks])
        whole_finite = bool(np.isfinite(out).all())
        d = np.abs(got - ref_out)
        return dict(max_abs=float(d.max()), mean_abs=float(d.mean()), lse_abs=float(np.abs(got_lse - ref_lse).max()),
                    rows=len(picks), all_rows_written=whole_finite)


class Workload:
    """All launches of a configuration for this rank, with CUDA graphs of a whole pass and of
    the attention kernels alone (one graph per cache set; sets rotate so that a pass never
    finds its cache in L2)."""

    def __init__(self, torch, name, rank, world, device, num_sms, l2_bytes, seed=1234, graphs=True):
        self.torch, self.name, self.world = torch, name, world
        self.launches = workload_launches(name)
        hkv_total = self.launches[0]["Hkv"]
        if hkv_total % world:
            raise SystemExit(f"Hkv={hkv_total} does not shard over {world} GPUs")
        self.bytes_local = sum(kv_bytes(l, l["Hkv"] // world) for l in self.launches)
        self.bytes_total = sum(kv_bytes(l, l["Hkv"]) for l in self.launches)
        self.flops_total = sum(attn_flops(l, l["Hq"]) for l in self.launches)
        self.flops_local = self.flops_total // world
        sets = 1 if self.bytes_local >= 4 * l2_bytes else int(-(-4 * l2_bytes // self.bytes_local))
        self.num_sets = min(sets, 64)
        self.dls = [DeviceLaunch(torch, l, rank, world, device, seed + 100 * i + rank, num_sms, sets=self.num_sets)
                    for i, l in enumerate(self.launches)]
        self.kernels_per_pass = sum(d.kernels for d in self.dls)
        for d in self.dls:  # one eager pass: sets kernel attributes, builds the page maps
            d.launch(0)
        torch.cuda.synchronize()
        # the copy ceiling follows the integer kernel: only where that kernel serves the whole launch
        self.has_copy_ceiling = all(d.attention_kernels == 1 and d.bq * d.G <= 16 and d.D == 128 for d in self.dls)
        if graphs:
            self.graphs = self._capture(lambda d, s: d.launch(s))
            self.attn_graphs = self._capture(lambda d, s: d.launch_attention_only(s))
            if self.has_copy_ceiling:
                for d in self.dls:
                    d.launch_copy_ceiling(0)
                torch.cuda.synchronize()
                self.copy_graphs = self._capture(lambda d, s: d.launch_copy_ceiling(s))

    def _capture(self, fn):
        torch = self.torch
        graphs, side = [], torch.cuda.Stream()
        with torch.cuda.stream(side):
            for s in range(self.num_sets):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for d in self.dls:
                        fn(d, s)
                graphs.append(g)
        torch.cuda.synchronize()
        return graphs

    def run_pass(self, i):
        self.graphs[i % self.num_sets].replay()

    def run_attention(self, i):
        self.attn_graphs[i % self.num_sets].replay()

    def run_copy_ceiling(self, i):
        self.copy_graphs[i % self.num_sets].replay()

    def run_e2e(self, i):
        for d in self.dls:
            d.e2e_pass(i % self.num_sets)

    def describe(self):
        return [{"batch": len(l["seq_lens"]), "context_max": max(l["seq_lens"]), "q_len": max(l["q_lens"]),
                 "window": l.get("window", 0), "num_splits_bound": d.S, "bq": d.bq, "Hq": l["Hq"], "Hkv": l["Hkv"],
                 "D": d.D, "block_size": d.block_size, "layout": d.layout}
                for l, d in zip(self.launches, self.dls)]

    def parity(self):
        worst = dict(max_abs=0.0, mean_abs=0.0, lse_abs=0.0, rows=0, all_rows_written=True)
        for i, d in enumerate(self.dls):
            r = d.parity(which=0, seed=17 + i)
            worst["max_abs"] = max(worst["max_abs"], r["max_abs"])
            worst["mean_abs"] = max(worst["mean_abs"], r["mean_abs"])
            worst["lse_abs"] = max(worst["lse_abs"], r["lse_abs"])
            worst["rows"] += r["rows"]
            worst["all_rows_written"] &= r["all_rows_written"]
        worst["within_tolerance"] = bool(worst["max_abs"] <= 2e-2 and worst["mean_abs"] <= 2e-3 and
                                         worst["lse_abs"] <= 1e-3 and worst["all_rows_written"])
        return worst


# --------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.rows.append((time.monotonic(), parts))

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        """Median SM clock and the throttle reasons seen by the samples taken between the host
        times t0 and t1 (the timed region)."""
        rows = [r for t, r in self.rows if t0 <= t <= t1]
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": "timed region"}


# --------------------------------------------------------------------------
# CPU baselines
# --------------------------------------------------------------------------
def cpu_port_baseline(seconds_target=12.0):
    """The numpy fp64 oracle on a bounded sample of the headline workload: decode requests at
    context 8192 (Hq 32, Hkv 8), as many as fit the time target."""
    from oracle import paged_int8_attention as orc

    rng = np.random.default_rng(5)
    L, reqs, t0, done = 8192, 0, time.perf_counter(), 0.0
    c = orc.make_paged_cache([L], HKV, D, BS, seed=5, poison=False)
    q = orc.round_to_bf16(rng.standard_normal((1, HQ, D), dtype=np.float32))
    t_build = time.perf_counter() - t0
    t0 = time.perf_counter()
    while True:
        orc.ref_attention_paged(q, c, [0, 1], D ** -0.5)
        reqs += 1
        done = time.perf_counter() - t0
        if done > seconds_target or reqs >= 64:
            break
    gbs = reqs * L * HKV * CELL / done / 1e9
    try:
        import threadpoolctl

        threads = max((p["num_threads"] for p in threadpoolctl.threadpool_info()), default=1)
    except Exception:
        threads = os.cpu_count() or 1
    return {"value": gbs, "unit": "GB/s", "cores": int(threads), "kind": "port",
            "sample": f"{reqs} decode requests of the headline workload (context {L}, Hq {HQ}, Hkv {HKV}, D {D}) "
                      f"through the numpy fp64 oracle incl. the paged gather, {done:.1f} s; cache build {t_build:.1f} s"}


def reference_arm(args):
    """Times the reference project's own C++ CPU path (oracle/_ref/libpth_ref_host.so, its
    scalar specification kernel run by 32 lock-step host threads) on a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import ctypes

    from oracle import paged_int8_attention as orc
    from pth_flash_attn_b200 import capi

    lib_path = REPO / "oracle" / "_ref" / "libpth_ref_host.so"
    base = {"impl": "reference", "metric": "kv_read_bandwidth", "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong",
            "dtype": "f32", "data": "synthetic", "vs_baseline": None,
            "config": {"workload": args.config, "Hq": HQ, "Hkv": HKV, "D": D, "block_size": BS}}
    if not lib_path.is_file():
        print(json.dumps({"impl": "reference", "unavailable": f"{lib_path.name} was not built (make -C oracle)"}))
        return
    lib = ctypes.CDLL(str(lib_path))
    lib.pth_ref_attention_host.restype = ctypes.c_int32
    lib.pth_ref_attention_host.argtypes = [ctypes.POINTER(capi.PthAttnArgs)]
    # sample: ONE decode request of the workload's head geometry, truncated to a few keys so that
    # steps + warmup calls end within about two minutes (the library needs ~60 ms per key here)
    L = int(max(1, min(64, 120.0 / (0.06 * max(1, args.steps + args.warmup)))))
    c = orc.make_paged_cache([L], HKV, D, BS, seed=9)
    rng = np.random.default_rng(10)
    q = orc.bf16_bits_from_f32(rng.standard_normal((1, HQ, D), dtype=np.float32))
    out = np.zeros((1, HQ, D), dtype=np.float32)
    qsl = np.asarray([0, 1], dtype=np.int32)
    a = capi.new_attn_args()
    a.q, a.q_dtype, a.q_stride_token, a.q_stride_head = q.ctypes.data, capi.BF16, HQ * D * 2, D * 2
    a.out, a.out_dtype, a.out_stride_token, a.out_stride_head = out.ctypes.data, capi.F32, HQ * D * 4, D * 4
    basep = c.storage.ctypes.data
    for dst, s in ((a.k_cache, c.k), (a.v_cache, c.v), (a.k_scale, c.ks), (a.v_scale, c.vs)):
        dst.data, dst.stride_block, dst.stride_slot, dst.stride_head = (basep + s.offset, s.stride_block,
                                                                       s.stride_slot, s.stride_head)
    a.num_blocks, a.block_size, a.num_kv_heads, a.head_size = c.num_blocks, BS, HKV, D
    a.block_table, a.block_table_row_stride = c.block_table.ctypes.data, c.block_table.shape[1]
    a.seq_lens, a.query_start_loc = c.seq_lens.ctypes.data, qsl.ctypes.data
    a.num_reqs, a.num_tokens, a.num_q_heads, a.bq, a.num_splits = 1, 1, HQ, 1, 1
    a.softmax_scale, a.window, a.causal = D ** -0.5, 0, 1
    for _ in range(args.warmup):
        assert lib.pth_ref_attention_host(ctypes.byref(a)) == 0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        assert lib.pth_ref_attention_host(ctypes.byref(a)) == 0
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    ref = orc.ref_attention_paged(orc.f32_from_bf16_bits(q), c, [0, 1], D ** -0.5)
    assert np.abs(out - ref.out).max() < 1e-3, "reference library disagrees with the oracle"
    gbs = L * HKV * CELL / dt / 1e9
    base.update({"value": gbs, "ms_per_step": dt * 1e3, "gpu_launches": 0, "same_config": False,
                 "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": 32, "kind": "reference",
                                  "sample": f"one decode request truncated to {L} keys (Hq {HQ}, Hkv {HKV}, D {D}) per "
                                            "step through pth_ref_attention_host; the library always runs 32 lock-step "
                                            f"host threads ({os.cpu_count()} cores present)"},
                 "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(base))


# --------------------------------------------------------------------------
# timing
# --------------------------------------------------------------------------
# DRAM bytes the attention kernel moves per algorithmic byte, from the ncu capture of the
# batch-64 decode launch (dram__bytes_read 1.1105 GB + dram__bytes_write 6.2 MB over 1.1073 GB of KV).
DRAM_BYTES_PER_ALGORITHMIC_BYTE = 1.0085


class Timer:
    def __init__(self, torch, dist, device, world):
        self.torch, self.dist, self.device, self.world = torch, dist, device, world

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, ms):
        if self.world > 1:
            t = self.torch.tensor([ms], device=self.device, dtype=self.torch.float64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def passes_per_step(self, fn, steps, target_s):
        """Passes per step so that `steps` steps last about target_s (the same on every rank)."""
        torch = self.torch
        for i in range(3):
            fn(i)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(10):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        pass_ms = self.max_over_ranks(e0.elapsed_time(e1) / 10)
        return max(1, int(round(target_s * 1e3 / max(steps, 1) / max(pass_ms, 1e-3))))

    def timed(self, fn, steps, warmup, pps):
        """Exactly `steps` steps of `pps` passes between two barriers; device time by CUDA events
        on the launching stream, maximum over ranks.  Returns ms per pass and the spread of the
        steps on this rank."""
        torch = self.torch
        c = 0
        for _ in range(warmup):
            for _ in range(pps):
                fn(c)
                c += 1
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        self.barrier()
        t0 = time.monotonic()
        evs[0].record()
        for k in range(steps):
            for _ in range(pps):
                fn(c)
                c += 1
            evs[k + 1].record()
        self.barrier()
        t1 = time.monotonic()
        total = self.max_over_ranks(evs[0].elapsed_time(evs[-1]))
        per = sorted(evs[k].elapsed_time(evs[k + 1]) / pps for k in range(steps))
        return dict(ms_per_pass=total / (steps * pps), ms_per_step=total / steps, t0=t0, t1=t1,
                    spread={"min": per[0], "median": per[len(per) // 2], "max": per[-1]})


def copy_ceiling_of(wl, timer, attn_ms):
    """Time of the paged-copy ceiling of the workload and eta_mem = T_copy / T_attention."""
    if not wl.has_copy_ceiling:
        return None
    pps = timer.passes_per_step(wl.run_copy_ceiling, 5, 0.2)
    ms = timer.timed(wl.run_copy_ceiling, 5, 3, pps)["ms_per_pass"]
    return {"ms_per_pass": ms, "gbs": wl.bytes_local / (ms * 1e-3) / 1e9, "eta_mem": ms / attn_ms,
            "what": "same bytes, same persistent CTAs, schedule and TMA page copies as the attention kernel, no compute"}


def roofline_of(wl, world, attn_ms, pass_ms, hbm_peak, tc_peak, tc_sustained, peak_src):
    """The roofline block of a workload on this rank: achieved = algorithmic bytes (flops) of
    the rank's shard over the time of its attention kernels alone."""
    t_bytes = wl.bytes_local / (hbm_peak * 1e9) * 1e3       # ms at the HBM peak
    t_flops = wl.flops_local / (tc_peak * 1e12) * 1e3       # ms at the tensor peak
    gbs = wl.bytes_local / (attn_ms * 1e-3) / 1e9
    tfs = wl.flops_local / (attn_ms * 1e-3) / 1e12
    if wl.name in TENSOR_BOUND:
        roof = {"bound": "tensor", "achieved": tfs, "peak": tc_peak, "unit": "TFLOP/s", "frac": tfs / tc_peak,
                "frac_of_sustained_peak": tfs / tc_sustained if tc_sustained else None, "traffic": None,
                "kernel": "umma_rows256_attention_kernel" if wl.dls[0].D == 256 else "umma_rows2_attention_kernel"}
    elif wl.name == "mixed":
        # two kernels one after the other: the integer kernel reads the decode and verify requests'
        # cache (HBM-bound), the row-major kernel computes the prefill chunks (tensor-bound); the
        # launch can be no faster than the larger of its two bounds
        bound_ms = max(t_bytes, t_flops)
        roof = {"bound": "hbm" if t_bytes >= t_flops else "tensor", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s",
                "frac": bound_ms / attn_ms, "tflops": tfs, "bound_ms": bound_ms, "traffic": None,
                "kernel": "umma_i8_attention_kernel + umma_rows2_attention_kernel"}
    else:
        # tall row tiles whose requests are all tall run on the one-tile row-major kernel (alone
        # when the launch is uniform, else behind an integer kernel that finds nothing to do)
        rows_kernel = all(d.bq * d.G > 16 and min(d.launch_spec["q_lens"]) * d.G > 16 for d in wl.dls)
        roof = {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                "traffic": (DRAM_BYTES_PER_ALGORITHMIC_BYTE * wl.bytes_local
                            if not rows_kernel and all(d.D == 128 for d in wl.dls) else None),
                "kernel": "umma_rows_attention_kernel" if rows_kernel else "umma_i8_attention_kernel"}
        if roof["traffic"] is not None:
            roof["traffic_source"] = "ncu capture of long_decode_b64, scaled by bytes"
    roof.update({"peak_source": peak_src, "kernel_ms_per_pass": attn_ms, "pass_ms": pass_ms,
                 "algorithmic_bytes_per_pass": wl.bytes_local, "flops_per_pass": wl.flops_local,
                 "frac_of_nominal_8TBs": gbs / 8000.0 if roof["bound"] == "hbm" else None})
    return roof


# --------------------------------------------------------------------------
# main
# --------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default=HEADLINE, help="workload of the headline numbers")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-per-config", action="store_true", help="only the headline workload")
    ap.add_argument("--profile", action="store_true",
                    help="three eager passes over the workload and exit (the command to run under ncu)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from pth_flash_attn_b200 import capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU fallback")
    capi.load_library()  # fails loudly if the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: start N > 1 with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    props = torch.cuda.get_device_properties(device)
    num_sms = props.multi_processor_count
    l2_bytes = getattr(props, "L2_cache_size", 126 * 2 ** 20)
    timer = Timer(torch, dist, device, world)
    steps, warmup = max(args.steps, 1), max(args.warmup, 3)

    peaks_path = REPO / "MEASURED_PEAKS.json"
    if peaks_path.is_file():
        peaks, peak_src = json.loads(peaks_path.read_text()), "measured"
        hbm_peak, tc_peak = float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"])
        tc_sustained = float(peaks.get("bf16_tflops_sustained", 0.0))
    else:
        hbm_peak, tc_peak, tc_sustained, peak_src = 6650.0, 1590.0, 1400.0, "fallback"

    wl = Workload(torch, args.config, rank, world, device, num_sms, l2_bytes, graphs=not args.profile)
    if args.profile:
        for i in range(2):
            for d in wl.dls:
                d.launch(i)
        torch.cuda.synchronize()
        print(json.dumps({"profile": args.config, "launches_per_pass": wl.kernels_per_pass, "passes": 3}))
        return

    clk = ClockSampler(local_rank)
    clk.__enter__()
    pps = timer.passes_per_step(wl.run_pass, steps, 1.0)
    main_t = timer.timed(wl.run_pass, steps, warmup, pps)
    clocks = clk.summary(main_t["t0"], main_t["t1"])
    clk.__exit__()
    ms_pass = main_t["ms_per_pass"]
    value = wl.bytes_total / (ms_pass * 1e-3) / 1e9

    # the attention kernels alone, in graphs of their own (for the roofline of the dominant kernel)
    pps_a = timer.passes_per_step(wl.run_attention, steps, 0.3)
    attn_ms = timer.timed(wl.run_attention, steps, 3, pps_a)["ms_per_pass"]
    # a graph of fewer kernels cannot take longer than the whole pass; jitter of two runs aside
    attn_ms = min(attn_ms, ms_pass)

    # end to end through the host-buffer call: pipelined (no synchronisation between passes)...
    pps_e = timer.passes_per_step(wl.run_e2e, steps, 0.5)
    e2e_t = timer.timed(wl.run_e2e, steps, 3, pps_e)
    e2e_value = wl.bytes_total / (e2e_t["ms_per_pass"] * 1e-3) / 1e9
    # ... and one call at a time: host clock from the copy-in to the result on the host
    lat = []
    for i in range(40):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        wl.run_e2e(i)
        torch.cuda.synchronize()
        lat.append((time.perf_counter() - t0) * 1e3)
    lat_ms = timer.max_over_ranks(float(np.median(lat[5:])))

    roof = roofline_of(wl, world, attn_ms, ms_pass, hbm_peak, tc_peak, tc_sustained, peak_src)
    roof["copy_ceiling"] = copy_ceiling_of(wl, timer, attn_ms)
    parity = wl.parity()
    tensor_headline = args.config in TENSOR_BOUND
    line = {
        "metric": "attention_tflops" if tensor_headline else "kv_read_bandwidth",
        "value": wl.flops_total / (ms_pass * 1e-3) / 1e12 if tensor_headline else value,
        "unit": "TFLOP/s" if tensor_headline else "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "passes_per_step": pps, "ms_per_step": main_t["ms_per_step"], "ms_per_pass": ms_pass,
        "us_per_layer": ms_pass * 1e3, "ms_per_pass_spread": main_t["spread"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8" if roof["kernel"].startswith("umma_i8") else "bf16", "data": "synthetic",
        "config": {"workload": args.config, "launches": wl.describe(), "Hq": wl.launches[0]["Hq"],
                   "Hkv": wl.launches[0]["Hkv"], "D": wl.launches[0].get("D", D), "block_size": wl.launches[0].get("block_size", BS), "sharding": f"kv_heads/{world}",
                   "l2_policy": ("inputs larger than L2" if wl.num_sets == 1 else
                                 f"rotation over {wl.num_sets} cache sets (>= 4x L2)"),
                   "cuda_graph": True,
                   "arithmetic": "int8 cache bytes and int8 digits of Q / P on tcgen05 kind::i8 with int32 accumulators "
                                 "(short row tiles); int8 cache widened exactly to bf16, tcgen05 kind::f16 with fp32 "
                                 "accumulators (tall row tiles); fp32 softmax",
                   "kv_bytes_per_pass": wl.bytes_total, "flops_per_pass": wl.flops_total},
        "tflops": wl.flops_total / (ms_pass * 1e-3) / 1e12,
        "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_pass": e2e_t["ms_per_pass"],
                "h2d_bytes_per_step": sum(d.h2d for d in wl.dls) * pps_e,
                "d2h_bytes_per_step": sum(d.d2h for d in wl.dls) * pps_e, "passes_per_step": pps_e,
                "h2d_bytes_per_pass": sum(d.h2d for d in wl.dls), "d2h_bytes_per_pass": sum(d.d2h for d in wl.dls),
                "mode": "pipelined throughput: passes are enqueued back to back, no synchronisation between them",
                "sync_latency_ms_per_pass": lat_ms,
                "sync_latency_note": "one pass at a time: copy-in, launches, copy-out, stream synchronised (host clock, median)"},
        "gpu_launches": wl.kernels_per_pass * pps * steps,
        "gpu_launches_per_pass": wl.kernels_per_pass,
        "clocks": clocks, "roofline": roof,
        "parity_checked": parity["within_tolerance"], "parity": parity,
    }
    del wl
    torch.cuda.empty_cache()

    if not args.no_per_config:
        per = {}
        for name in PER_CONFIG:
            if name == args.config:
                per[name] = {"ms_per_pass": ms_pass, "kv_gbs": value, "tflops": line["tflops"],
                             "roofline_frac": roof["frac"], "bound": roof["bound"], "kernel_ms_per_pass": attn_ms,
                             "parity_checked": parity["within_tolerance"]}
                continue
            if any(l["Hkv"] % world for l in workload_launches(name)):
                per[name] = {"skipped": f"its KV heads do not divide over {world} ranks"}
                continue
            w = Workload(torch, name, rank, world, device, num_sms, l2_bytes)
            p1 = timer.passes_per_step(w.run_pass, 5, 0.4)
            t = timer.timed(w.run_pass, 5, 3, p1)
            p2 = timer.passes_per_step(w.run_attention, 5, 0.2)
            a_ms = min(timer.timed(w.run_attention, 5, 3, p2)["ms_per_pass"], t["ms_per_pass"])
            r = roofline_of(w, world, a_ms, t["ms_per_pass"], hbm_peak, tc_peak, tc_sustained, peak_src)
            ceiling = copy_ceiling_of(w, timer, a_ms)
            par = w.parity()
            per[name] = {"ms_per_pass": t["ms_per_pass"], "us_per_layer": t["ms_per_pass"] * 1e3,
                         "kv_gbs": w.bytes_total / (t["ms_per_pass"] * 1e-3) / 1e9,
                         "tflops": w.flops_total / (t["ms_per_pass"] * 1e-3) / 1e12,
                         "roofline_frac": r["frac"], "bound": r["bound"], "unit": r["unit"], "achieved": r["achieved"],
                         "peak": r["peak"], "kernel": r["kernel"], "kernel_ms_per_pass": a_ms,
                         "eta_mem": ceiling["eta_mem"] if ceiling else None,
                         "copy_ceiling_gbs": ceiling["gbs"] if ceiling else None,
                         "launches": w.describe(), "l2_sets": w.num_sets, "gpu_launches_per_pass": w.kernels_per_pass,
                         "parity_checked": par["within_tolerance"], "parity": par}
            del w
            torch.cuda.empty_cache()
        line["per_config"] = per

    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_port_baseline()
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
