#!/usr/bin/env python
"""Benchmark of the paged int8 attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config NAME] [--impl reference]

A "step" is one pass of the hot path over one synthetic batch.  The default
workload is the long-context split-KV decode configuration: one launch of
batch 1 at context 131072 plus one launch of batch 64 at context 8192
(Hq = 32, Hkv = 8, D = 128, block size 16, one query token per request), each
launch being the attention kernel and, when the planner splits the KV range,
the combine kernel.  The metric is the achieved cache read bandwidth: the
algorithmic KV bytes of a step (every visible (token, KV head) cell once,
2 D + 8 bytes each) divided by the device time of the step.

With N > 1 (one process per GPU, started by torch.distributed.run) the KV heads
are sharded: rank g owns Hkv / N KV heads, the matching query heads and its own
cache; there is no collective on the data path.  Total work is fixed, so the
line says "strong" scaling; `value` is the whole job's bytes over the slowest
rank's time.

Inputs are synthetic: random int8 cells with plausible fp32 scales written
directly in vLLM's int8_per_token_head page layout on the device, bf16 N(0,1)
queries, seeded random block tables.  Values do not change the memory traffic.
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


# --------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------
def workload_launches(name: str, seed: int = 1001):
    """Returns a list of launches: dict(seq_lens, q_lens, window, causal, Hq, Hkv)."""
    rng = np.random.default_rng(seed)
    if name == "decode_small":  # BASELINE config 0
        return [dict(seq_lens=rng.integers(1, 4097, size=8).tolist(), q_lens=[1] * 8, Hq=32, Hkv=8)]
    if name == "long_decode":  # BASELINE config 1 (default)
        return [dict(seq_lens=[131072], q_lens=[1], Hq=32, Hkv=8),
                dict(seq_lens=[8192] * 64, q_lens=[1] * 64, Hq=32, Hkv=8)]
    if name == "long_decode_b1":
        return [dict(seq_lens=[131072], q_lens=[1], Hq=32, Hkv=8)]
    if name == "long_decode_b64":
        return [dict(seq_lens=[8192] * 64, q_lens=[1] * 64, Hq=32, Hkv=8)]
    if name == "decode_h1":  # one KV head per GPU (the 8-GPU shard shape), same bytes as long_decode_b64
        return [dict(seq_lens=[8192] * 512, q_lens=[1] * 512, Hq=4, Hkv=1)]
    if name == "shard8_b1":  # what one of 8 GPUs sees of long_decode's first launch
        return [dict(seq_lens=[131072], q_lens=[1], Hq=4, Hkv=1)]
    if name == "shard8_b64":  # ... and of its second launch
        return [dict(seq_lens=[8192] * 64, q_lens=[1] * 64, Hq=4, Hkv=1)]
    if name == "verify4":  # BASELINE config 2a
        return [dict(seq_lens=rng.integers(16384, 32769, size=32).tolist(), q_lens=[4] * 32, Hq=32, Hkv=8)]
    if name == "drafter16":  # BASELINE config 2b
        return [dict(seq_lens=rng.integers(16384, 32769, size=32).tolist(), q_lens=[16] * 32, Hq=32,
                     Hkv=8, window=4096)]
    if name == "chunked_prefill":  # BASELINE config 3
        return [dict(seq_lens=[32768] * 4, q_lens=[2048] * 4, Hq=64, Hkv=8, prefill=True)]
    if name == "mixed":  # BASELINE config 4, one launch
        dec = rng.integers(4096, 131073, size=48).tolist()
        return [dict(seq_lens=dec + [32768] * 8 + [17408] * 2, q_lens=[1] * 48 + [4] * 8 + [1024] * 2,
                     Hq=64, Hkv=8, prefill=True)]
    raise SystemExit(f"unknown --config {name}")


def kv_bytes(launch, hkv_local):
    total = 0
    w = launch.get("window", 0)
    for L, ql in zip(launch["seq_lens"], launch["q_lens"]):
        vis = L if w <= 0 else min(L, w + ql - 1)
        total += vis * hkv_local * CELL
    return total


def attn_flops(launch, hq_local):
    total = 0
    w = launch.get("window", 0)
    for L, ql in zip(launch["seq_lens"], launch["q_lens"]):
        if w <= 0:
            pairs = ql * (L - ql) + ql * (ql + 1) // 2
        else:
            pairs = sum(min(L - ql + i + 1, w) for i in range(ql))
        total += 4 * D * hq_local * pairs
    return total


# --------------------------------------------------------------------------
# device-side synthetic cache
# --------------------------------------------------------------------------
class DeviceLaunch:
    """One launch with everything resident on the device, plus pinned host copies of the
    per-step inputs for the end-to-end leg."""

    def __init__(self, torch, launch, hkv_local, hq_local, device, seed, num_sms, sets=1, splits=None, layout="NHD"):
        from pth_flash_attn_b200 import capi, host, planner

        self.torch = torch
        self.flags = 0
        g = torch.Generator(device="cpu").manual_seed(seed)
        lens, qlens = launch["seq_lens"], launch["q_lens"]
        R, T = len(lens), int(sum(qlens))
        self.R, self.T = R, T
        self.window, self.causal = launch.get("window", 0), launch.get("causal", True)
        G = hq_local // hkv_local
        nblk = [-(-L // BS) for L in lens]
        need = sum(nblk)
        page = BS * hkv_local * CELL
        self.sets = []
        q_max = max(qlens)
        is_prefill = bool(launch.get("prefill", False))
        w_ts = planner.workspace_token_splits(max_num_seqs=max(R, 1), q_dec_max=q_max, Hkv=hkv_local, D=D,
                                              num_sms=num_sms)
        plan = planner.plan_launch(num_tokens=T, num_reqs=R, max_query_len=q_max, G=G, Hkv=hkv_local, D=D,
                                   num_sms=num_sms, is_prefill=is_prefill, ws_token_splits=w_ts,
                                   window=self.window)
        self.S = int(splits) if splits else plan.num_splits
        self.bq = min(plan.bq, q_max) if not is_prefill else plan.bq
        self.plan = plan
        for s in range(sets):
            storage = torch.randint(0, 256, (need * page,), dtype=torch.uint8, device=device,
                                    generator=torch.Generator(device=device).manual_seed(seed + 7 * s))
            words = storage.view(torch.float32).view(need, BS, hkv_local, CELL // 4)
            scale = torch.rand((need, BS, hkv_local), device=device) * 0.02 + 0.01
            words[..., D // 4] = scale
            words[..., CELL // 4 - 1] = scale
            perm = (torch.arange(need) if os.environ.get("BENCH_SEQUENTIAL_BLOCKS") else torch.randperm(need, generator=g)).to(torch.int32)
            bt = torch.zeros((R, max(nblk)), dtype=torch.int32)
            k = 0
            for r, nb in enumerate(nblk):
                bt[r, :nb] = perm[k:k + nb]
                k += nb
            base = storage.data_ptr()
            slot, head = (hkv_local * CELL, CELL) if layout == "NHD" else (CELL, BS * CELL)
            views = host.CacheViews((base, page, slot, head), (base + D + 4, page, slot, head),
                                    (base + D, page, slot, head), (base + 2 * D + 4, page, slot, head),
                                    need, BS, hkv_local, D)
            self.sets.append(dict(storage=storage, views=views, bt_host=bt.pin_memory(), bt=bt.to(device)))
        self.q_host = torch.randn((T, hq_local, D), generator=g).to(torch.bfloat16).pin_memory()
        self.q = self.q_host.to(device)
        qsl = torch.zeros(R + 1, dtype=torch.int32)
        qsl[1:] = torch.tensor(qlens, dtype=torch.int64).cumsum(0).to(torch.int32)
        self.qsl_host, self.lens_host = qsl.pin_memory(), torch.tensor(lens, dtype=torch.int32).pin_memory()
        self.qsl, self.lens = self.qsl_host.to(device), self.lens_host.to(device)
        self.out = torch.zeros((T, hq_local, D), dtype=torch.bfloat16, device=device)
        self.out_host = torch.empty((T, hq_local, D), dtype=torch.bfloat16).pin_memory()
        self.ws_o = self.ws_lse = None
        if self.S > 1:
            self.ws_o = torch.empty((self.S, T, hq_local, D), dtype=torch.float32, device=device)
            self.ws_lse = torch.empty((self.S, T, hq_local), dtype=torch.float32, device=device)
        # as the torch op does: max_query_len within one row tile = one row tile per request
        if q_max <= self.bq:
            self.flags |= capi.FLAG_ONE_TILE_PER_REQUEST
        # tall row tiles: the automatic choice runs the integer kernel (short requests) and the
        # row-major kernel (the others) one after the other
        pair = KERNEL_CHOICE == capi.KERNEL_AUTO and self.bq * G > 16
        self.kernels = (2 if pair else 1) + (1 if self.S > 1 else 0)
        self.h2d = self.q_host.numel() * 2 + self.sets[0]["bt_host"].numel() * 4 + (2 * R + 1) * 4
        self.d2h = self.out_host.numel() * 2

    def launch(self, which=0):
        from pth_flash_attn_b200 import host

        s = self.sets[which % len(self.sets)]
        host.attention_forward(self.q, self.out, s["views"], s["bt"], self.lens, self.qsl, bq=self.bq,
                               num_splits=self.S, softmax_scale=D ** -0.5, ws_o=self.ws_o, ws_lse=self.ws_lse,
                               window=self.window, causal=self.causal, flags=self.flags, kernel=KERNEL_CHOICE)

    def launch_attention_only(self, which=0):
        """Only the attention kernel (for the per-kernel roofline timing)."""
        from pth_flash_attn_b200 import capi, host

        s = self.sets[which % len(self.sets)]
        a = host.fill_attn_args(self.q, self.out, s["views"], s["bt"], self.lens, self.qsl, bq=self.bq,
                                num_splits=self.S, softmax_scale=D ** -0.5, ws_o=self.ws_o, ws_lse=self.ws_lse,
                                window=self.window, causal=self.causal)
        lib = capi.load_library()
        rc = lib.attention(a, options=capi.make_options(KERNEL_CHOICE, self.flags),
                           stream=self.torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(lib.last_error())

    def e2e_step(self, which=0):
        """Host buffers in, host buffer out: pinned H2D of the step's inputs, the launch, D2H of out."""
        s = self.sets[which % len(self.sets)]
        self.q.copy_(self.q_host, non_blocking=True)
        s["bt"].copy_(s["bt_host"], non_blocking=True)
        self.lens.copy_(self.lens_host, non_blocking=True)
        self.qsl.copy_(self.qsl_host, non_blocking=True)
        self.launch(which)
        self.out_host.copy_(self.out, non_blocking=True)


# --------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------
# Kernel family of the C ABI options (0 = the library's own choice); --kernel overrides it for exploration.
KERNEL_CHOICE = 0

# Measured with ncu on the batch-64 decode launch (see profiles/).
DRAM_BYTES_PER_ALGORITHMIC_BYTE = 1.22


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

    def summary(self, t0=None, t1=None):
        """Median SM clock and the throttle reasons seen.  With (t0, t1) only the samples
        taken inside that host-time window count, if there are at least three of them; a
        shorter timed region falls back to every sample taken while the GPU was under the
        benchmark's load (warm-up, timed steps, end-to-end and per-kernel passes)."""
        rows, window = [r for _, r in self.rows], "whole load phase"
        if t0 is not None:
            inside = [r for t, r in self.rows if t0 <= t <= t1]
            if len(inside) >= 3:
                rows, window = inside, "timed region"
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
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


# --------------------------------------------------------------------------
# CPU baselines
# --------------------------------------------------------------------------
def cpu_port_baseline(seconds_target=12.0):
    """The numpy fp64 oracle on a bounded sample of the default workload: decode requests at
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
            "sample": f"{reqs} decode requests of the default workload (context {L}, Hq {HQ}, Hkv {HKV}, D {D}) "
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
    base.update({"value": gbs, "ms_per_step": dt * 1e3, "gpu_launches": 0,
                 "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": 32, "kind": "reference",
                                  "sample": f"one decode request truncated to {L} keys (Hq {HQ}, Hkv {HKV}, D {D}) per "
                                            "step through pth_ref_attention_host; the library always runs 32 lock-step "
                                            f"host threads ({os.cpu_count()} cores present)"},
                 "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(base))


# --------------------------------------------------------------------------
# main
# --------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--config", default="long_decode")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--splits", type=int, default=0, help="override the planner's split count (exploration)")
    ap.add_argument("--kernel", type=int, default=0, help="kernel family of the C ABI (exploration; 0 = automatic)")
    ap.add_argument("--layout", default="NHD", choices=["NHD", "HND"], help="physical order inside a page")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="three eager passes over the workload and exit (the command to run under ncu)")
    args = ap.parse_args()
    global KERNEL_CHOICE
    KERNEL_CHOICE = args.kernel
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

    launches = workload_launches(args.config)
    hkv_total = launches[0]["Hkv"]
    if hkv_total % world:
        raise SystemExit(f"Hkv={hkv_total} does not shard over {world} GPUs")
    step_bytes_local = sum(kv_bytes(l, l["Hkv"] // world) for l in launches)
    sets = 1 if step_bytes_local >= 4 * l2_bytes else int(-(-4 * l2_bytes // step_bytes_local))
    sets = min(sets, 64)
    dls = [DeviceLaunch(torch, l, l["Hkv"] // world, l["Hq"] // world, device, 1234 + 100 * i + rank, num_sms,
                        sets=sets, splits=args.splits, layout=args.layout) for i, l in enumerate(launches)]
    step_bytes_total = sum(kv_bytes(l, l["Hkv"]) for l in launches)
    step_flops_total = sum(attn_flops(l, l["Hq"]) for l in launches)
    kernels_per_step = sum(d.kernels for d in dls)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # one eager pass (also sets kernel attributes), then one CUDA graph per cache set
    for d in dls:
        d.launch(0)
    torch.cuda.synchronize()
    if args.profile:
        for i in range(2):
            for d in dls:
                d.launch(i)
        torch.cuda.synchronize()
        print(json.dumps({"profile": args.config, "launches_per_pass": kernels_per_step, "passes": 3}))
        return
    graphs = []
    if not args.no_graph:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for s in range(sets):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for d in dls:
                        d.launch(s)
                graphs.append(g)
        torch.cuda.synchronize()

    def run_step(i):
        if graphs:
            graphs[i % sets].replay()
        else:
            for d in dls:
                d.launch(i % sets)

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    clk = ClockSampler(local_rank)
    clk.__enter__()
    for i in range(max(args.warmup, 3)):
        run_step(i)
    t_begin = time.monotonic()
    ms_total = timed(run_step, args.steps)
    t_end = time.monotonic()
    ms_per_step = ms_total / args.steps
    value = step_bytes_total / (ms_per_step * 1e-3) / 1e9

    # end to end through the host-buffer call
    def e2e(i):
        for d in dls:
            d.e2e_step(i % sets)

    for i in range(3):
        e2e(i)
    ms_e2e = timed(e2e, args.steps) / args.steps
    e2e_value = step_bytes_total / (ms_e2e * 1e-3) / 1e9

    # per-kernel timing of the dominant kernel (attention) for the roofline line
    attn_ms = 0.0
    reps = max(10, min(args.steps, 50))
    evs = []
    torch.cuda.synchronize()
    for i in range(reps):
        for d in dls:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            d.launch_attention_only(i % sets)
            b.record()
            evs.append((a, b))
    torch.cuda.synchronize()
    attn_ms = sum(a.elapsed_time(b) for a, b in evs) / reps  # all attention launches of one step
    clk.__exit__()
    clocks = clk.summary(t_begin, t_end)
    peaks_path = REPO / "MEASURED_PEAKS.json"
    if peaks_path.is_file():
        peaks, peak_src = json.loads(peaks_path.read_text()), "measured"
        hbm_peak, tc_peak = float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"])
    else:
        hbm_peak, tc_peak, peak_src = 6650.0, 1590.0, "fallback"
    tensor_bound = args.config in ("chunked_prefill",)
    if tensor_bound:
        achieved = (step_flops_total / world) / (attn_ms * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": tc_peak, "unit": "TFLOP/s",
                "frac": achieved / tc_peak, "traffic": None}
    else:
        achieved = step_bytes_local / (attn_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "traffic": None}
    roof["peak_source"] = peak_src
    # the library sends row tiles of more than 16 rows to the row-major bf16 kernel
    rows_kernel = any(d.bq * (l["Hq"] // l["Hkv"]) > 16 for l, d in zip(launches, dls))
    roof["kernel"] = "umma_rows_attention_kernel" if rows_kernel else "umma_i8_attention_kernel"
    roof["kernel_ms_per_step"] = attn_ms
    roof["algorithmic_bytes_per_step"] = step_bytes_local
    if not tensor_bound:
        # DRAM bytes per algorithmic byte of the attention kernel, from the ncu capture of the
        # batch-64 decode launch summarised under profiles/ (dram__bytes_read + write over
        # 1.107 GB of KV); traffic grows in proportion to the keys read, so the ratio scales to
        # the workload's bytes.
        roof["traffic"] = DRAM_BYTES_PER_ALGORITHMIC_BYTE * step_bytes_local
        roof["traffic_source"] = "ncu capture of long_decode_b64, scaled by bytes"

    if rank == 0:
        line = {
            "metric": "kv_read_bandwidth", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "us_per_layer": ms_per_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if rows_kernel else "int8",
            "data": "synthetic",
            "config": {"workload": args.config, "launches": [
                {"batch": len(l["seq_lens"]), "context_max": max(l["seq_lens"]), "q_len": max(l["q_lens"]),
                 "window": l.get("window", 0), "num_splits": d.S, "bq": d.bq} for l, d in zip(launches, dls)],
                "Hq": launches[0]["Hq"], "Hkv": hkv_total, "D": D, "block_size": BS, "sharding": f"kv_heads/{world}",
                "l2_policy": ("inputs larger than L2" if sets == 1 else f"rotation over {sets} cache sets (>= 4x L2)"),
                "cuda_graph": bool(graphs),
                "arithmetic": ("int8 cache widened exactly to bf16 in shared memory, tcgen05 kind::f16 with fp32 "
                               "accumulators in TMEM, fp32 softmax" if rows_kernel else
                               "int8 cache bytes and int8 digits of Q / P on tcgen05 kind::i8, int32 accumulators, "
                               "fp32 softmax and output accumulation"),
                "kv_bytes_per_step": step_bytes_total, "flops_per_step": step_flops_total},
            "tflops": step_flops_total / (ms_per_step * 1e-3) / 1e12,
            "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": sum(d.h2d for d in dls), "d2h_bytes_per_step": sum(d.d2h for d in dls)},
            "gpu_launches": kernels_per_step * args.steps,
            "clocks": clocks, "roofline": roof,
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_port_baseline()
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
