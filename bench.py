#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One JSON line on stdout (rank 0).  Headline metric: prefill attention TFLOP/s on configuration 2
(FlashAttention-2 + RoPE, causal, batch 4, 32 heads, seq 2048, head_dim 128, bf16 tensor-core
path); the decode configuration 3 (GQA decode, batch 32, 32/8 heads, KV 4096 -> 4352, 256 steps)
is measured in the same run and reported under "decode".  Synthetic N(0,1) inputs from a seed.

A step is one pass of the hot path over one batch.  `value` times the kernel with inputs resident
in HBM (CUDA events on the library's stream); `e2e` times the public Python op
(grilly_core.flash_attention2 / decode_step) with pinned HOST buffers, copies inside the timed
region.  With N > 1 (torchrun, one process per GPU) every rank runs the same per-GPU workload on
its own GPU (weak scaling, no data-path collective); times are the max over ranks.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "grilly-next_b200", "python"))

CFG2 = dict(B=4, H=32, S=2048, D=128, theta=10000.0, seed=1002)
CFG4 = dict(Hq=32, Hkv=8, D=128, T=131072, seed=1004)
CFG3 = dict(B=32, Hq=32, Hkv=8, D=128, T0=4096, steps=256, theta=10000.0, seed=1003, page=64)


def prefill_flops(c):
    return 4 * c["D"] * c["B"] * c["H"] * (c["S"] * (c["S"] + 1) // 2)


def decode_bytes(c):
    """Algorithmic bytes of the 256-step run: K+V rows attended (bf16) + q read + O write + append write."""
    per_pos = 2 * c["B"] * c["Hkv"] * c["D"] * 2
    kv = sum(per_pos * (c["T0"] + t + 1) for t in range(c["steps"]))
    other = c["steps"] * (c["B"] * c["Hq"] * c["D"] * (4 + 4) + 2 * c["B"] * c["Hkv"] * c["D"] * 2)
    return kv + other


# dram__bytes_read.sum + dram__bytes_write.sum of one flash_fwd_sm100_kernel launch on cfg2 (ncu, see profiles/)
PREFILL_TRAFFIC_BYTES = 208.9e6 + 103.1e6
DECODE_TRAFFIC_BYTES = 546.1e6 + 11.0e6     # one decode_mma_kernel launch at cache length ~4117 (ncu, see profiles/)


def prefill_roofline(tflops_gpu, timed_ms, pk):
    """The prefill kernel against the measured cuBLAS bf16 rate: the burst figure when the timed region is
    short (clocks still at boost), the sustained one when it runs long enough to sit under the power cap."""
    long_run = timed_ms > 100.0 and pk["tf_sustained"]
    peak = pk["tf_sustained"] if long_run else pk["tf"]
    return {"bound": "tensor", "achieved": tflops_gpu, "peak": peak, "unit": "TFLOP/s", "frac": tflops_gpu / peak,
            "traffic": PREFILL_TRAFFIC_BYTES, "peak_source": pk["src"] + (" (sustained: timed region > 100 ms)" if long_run else " (burst)"),
            "frac_of_burst": tflops_gpu / pk["tf"],
            "frac_of_sustained": tflops_gpu / pk["tf_sustained"] if pk["tf_sustained"] else None,
            "frac_of_nominal_2250": tflops_gpu / 2250.0, "kernel": "flash_fwd_sm100_kernel"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tf=d["bf16_tflops"], tf_sustained=d.get("bf16_tflops_sustained"), src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, src="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.t0 = self.t1 = None

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([time.time()] + [x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.t.join(timeout=2)
        # samples taken while the timed region ran (20 ms of slack for the sampler's own latency)
        rows = [r[1:] for r in self.rows if len(r) >= 7 and self.t0 is not None and self.t0 <= r[0] <= self.t1 + 0.02]
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[2].replace(".", "").isdigit() for r in [r[1:]]]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------- reference arm
def run_reference(args):
    """The reference's CPU implementation of the path: its Vulkan shaders cannot run here (no
    graphics stack) and its C++ library does not build without the Vulkan SDK, so this arm times
    the C restatement of its CPU attention (oracle/attn_oracle.c, OpenMP, all host threads)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())   # torchrun pins it to 1; this arm may use every host thread
    from oracle import c_oracle
    c = CFG2
    heads = 32                                   # bounded sample: 32 of the 128 (batch, head) pairs per step
    rng = np.random.default_rng(c["seed"])
    Q, K, V = (rng.standard_normal((1, heads, c["S"], c["D"]), dtype=np.float32) for _ in range(3))
    from oracle import attention_oracle as orc
    pos = np.arange(c["S"])
    fl = 4 * c["D"] * heads * (c["S"] * (c["S"] + 1) // 2)
    for _ in range(max(1, min(args.warmup, 2))):
        c_oracle.attention(Q, K, V, causal=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        q = orc.rope_interleaved(Q, pos, c["theta"])   # RoPE is part of the path
        k = orc.rope_interleaved(K, pos, c["theta"])
        c_oracle.attention(q, k, V, causal=True)
    dt = time.perf_counter() - t0
    val = fl * args.steps / dt / 1e12
    line = {
        "impl": "reference", "metric": "prefill_attn_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg2: FlashAttention-2+RoPE causal prefill, B4 H32 S2048 D128", "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": c_oracle.num_threads(), "kind": "port",
                         "sample": f"{heads} of 128 (batch, head) slices of cfg2 per step, RoPE + causal attention, C/OpenMP"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------- our arm
def pinned_array(L, shape, dtype):
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    p = C.c_void_p()
    rc = L.grl_host_alloc(n, C.byref(p))
    if rc != 0:
        raise RuntimeError(L.grl_last_error().decode())
    buf = (C.c_char * n).from_address(p.value)
    return np.frombuffer(buf, dtype=dtype).reshape(shape), p


def bench_prefill(dev, cabi, args, dist):
    c = CFG2
    B, H, S, D = c["B"], c["H"], c["S"], c["D"]
    rng = np.random.default_rng(c["seed"] + dist["rank"])
    n = B * H * S * D
    q = dev.upload_bf16(rng.standard_normal((B, H, S, D), dtype=np.float32))
    k = dev.upload_bf16(rng.standard_normal((B, H, S, D), dtype=np.float32))
    v = dev.upload_bf16(rng.standard_normal((B, H, S, D), dtype=np.float32))
    o = dev.malloc(n * 4)
    p = cabi.FlashParams()
    p.q, p.k, p.v, p.o = q, k, v, o
    p.in_dtype, p.out_dtype = cabi.BF16, cabi.F32
    p.batch, p.heads, p.seq_len, p.head_dim = B, H, S, D
    p.causal, p.rope_mode, p.rope_theta, p.rope_scaling = 1, cabi.ROPE_INTERLEAVED, c["theta"], 1.0
    if args.variant == "norope":          # profiling aids: not the benchmark configuration
        p.rope_mode = cabi.ROPE_NONE
    elif args.variant == "noncausal":
        p.causal = 0
    p.kernel = cabi.KERNEL_TCGEN05
    L = dev.L

    def step():
        cabi.check(L.grl_flash_fwd(dev.h, C.byref(p)))

    sampler = ClockSampler(dist["local_rank"])
    sampler.start()
    for _ in range(args.warmup):
        step()
    dev.sync()
    e0, e1 = dev.event(), dev.event()
    dist["barrier"]()
    launches0 = L.grl_launch_count()
    sampler.mark_start()
    dev.record(e0)
    for _ in range(args.steps):
        step()
    dev.record(e1)
    dev.sync()
    sampler.mark_end()
    ms = dev.elapsed_ms(e0, e1)
    launches = L.grl_launch_count() - launches0
    ms = dist["max"](ms)
    dist["barrier"]()
    clocks = sampler.stop()
    for x in (q, k, v, o):
        dev.free(x)
    return ms, launches, clocks


def bench_prefill_e2e(args, L, steps, dist):
    """grilly_core.flash_attention2(dtype='bf16') with pinned host arrays: upload, cast, kernel, download."""
    import grilly_core
    c = CFG2
    shape = (c["B"], c["H"], c["S"], c["D"])
    rng = np.random.default_rng(c["seed"])
    arrs, ptrs = [], []
    for _ in range(3):
        a, pp = pinned_array(L, shape, np.float32)
        a[...] = rng.standard_normal(shape, dtype=np.float32)
        arrs.append(a)
        ptrs.append(pp)
    ctx = grilly_core.Device()
    out_arr, out_ptr = pinned_array(L, shape, np.float32)
    ptrs.append(out_ptr)
    kw = dict(causal=True, rope_theta=c["theta"], dtype="bf16", out=out_arr)
    for _ in range(2):
        out = grilly_core.flash_attention2(ctx, *arrs, **kw)
    dist["barrier"]()
    t0 = time.perf_counter()
    for _ in range(steps):
        out = grilly_core.flash_attention2(ctx, *arrs, **kw)   # synchronous: returns with the result on the host
    dt = dist["max"]((time.perf_counter() - t0) / steps)
    assert np.isfinite(out[0, 0, -1]).all()
    del ctx
    for pp in ptrs:
        L.grl_host_free(pp)
    nbytes = int(np.prod(shape)) * 4
    # what crosses the link: the op's host threads round a share of every chunk to bf16 before the upload
    # (all of it with one process per node, 50 %/N with N), the rest goes up as float32
    lws = int(os.environ.get("LOCAL_WORLD_SIZE", "1"))
    pct = int(os.environ.get("GRILLY_PIPELINE_HOST_CAST_PCT", 100 if lws <= 1 else 50 // lws))
    h2d = 3 * (nbytes // 2 * pct + nbytes * (100 - pct)) // 100
    return dt, h2d, nbytes


def bench_decode(dev, cabi, dist, repeats=3, use_graph=True, force_splits=0):
    """cfg3: 256 decode steps (RoPE + append + split-KV attention + merge), graph-replayed."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle import attention_oracle as orc
    c = CFG3
    B, Hq, Hkv, D, T0, steps, P = c["B"], c["Hq"], c["Hkv"], c["D"], c["T0"], c["steps"], c["page"]
    L = dev.L
    rng = np.random.default_rng(c["seed"] + dist["rank"])
    max_tokens = T0 + steps
    max_pages = (max_tokens + P - 1) // P
    n_pages = max_pages * B
    page_elems = Hkv * P * D
    kp, vp = dev.malloc(n_pages * page_elems * 2), dev.malloc(n_pages * page_elems * 2)
    # iid N(0,1) bf16 in every page (the prefix is "already rotated" keys; layout does not matter for iid data)
    chunk = rng.standard_normal(32 * page_elems, dtype=np.float32)
    bits = orc.to_bf16_bits(chunk)
    for dst in (kp, vp):
        off = 0
        total = n_pages * page_elems
        while off < total:
            m = min(bits.size, total - off)
            rolled = np.roll(bits, int(rng.integers(0, bits.size)))[:m]
            cabi.check(L.grl_memcpy_h2d(dev.h, C.c_void_p(dst.value + off * 2), rolled.ctypes.data_as(C.c_void_p), m * 2))
            dev.sync()
            off += m
    table = dev.upload(np.arange(n_pages, dtype=np.int32).reshape(B, max_pages))
    lens0 = np.full(B, T0, np.int32)
    seq_lens = dev.upload(lens0)
    qs = dev.upload(rng.standard_normal((steps, B, 1, Hq, D), dtype=np.float32))
    ks = dev.upload(rng.standard_normal((steps, B, 1, Hkv, D), dtype=np.float32))
    vs = dev.upload(rng.standard_normal((steps, B, 1, Hkv, D), dtype=np.float32))
    q_rot = dev.malloc(B * Hq * D * 4)
    out = dev.malloc(steps * B * Hq * D * 4)

    lay = cabi.KVLayout()
    lay.k_pages, lay.v_pages, lay.cache_dtype = kp, vp, cabi.BF16
    lay.block_table, lay.seq_lens = table, seq_lens
    lay.batch, lay.num_kv_heads, lay.head_dim, lay.page_tokens, lay.max_pages = B, Hkv, D, P, max_pages
    lay.num_pages = n_pages
    dp = cabi.DecodeParams()
    dp.kv, dp.num_q_heads, dp.max_seq_len = lay, Hq, max_tokens
    dp.n_splits = force_splits
    ns = C.c_int()
    cabi.check(L.grl_decode_pick_splits(dev.h, C.byref(dp), C.byref(ns)))
    wb = C.c_size_t()
    cabi.check(L.grl_decode_workspace_bytes(C.byref(dp), ns.value, C.byref(wb)))
    ws = dev.malloc(wb.value)
    dp.n_splits, dp.workspace, dp.workspace_bytes = ns.value, ws, wb.value

    def record_steps():
        for t in range(steps):
            ap = cabi.AppendParams()
            ap.kv = lay
            ap.k_new = C.c_void_p(ks.value + t * B * Hkv * D * 4)
            ap.v_new = C.c_void_p(vs.value + t * B * Hkv * D * 4)
            ap.q_in = C.c_void_p(qs.value + t * B * Hq * D * 4)
            ap.q_out = q_rot
            ap.n_new, ap.num_q_heads = 1, Hq
            ap.rope_mode, ap.rope_theta, ap.rope_scaling, ap.pos_base, ap.update_lens = cabi.ROPE_INTERLEAVED, c["theta"], 1.0, 0, 1
            cabi.check(L.grl_kv_append(dev.h, C.byref(ap)))
            dp.q = q_rot
            dp.out = C.c_void_p(out.value + t * B * Hq * D * 4)
            cabi.check(L.grl_gqa_decode(dev.h, C.byref(dp)))

    def reset():
        cabi.check(L.grl_memcpy_h2d(dev.h, seq_lens, lens0.ctypes.data_as(C.c_void_p), lens0.nbytes))

    launches0 = L.grl_launch_count()
    g = C.c_void_p()
    if use_graph:
        cabi.check(L.grl_graph_begin(dev.h))
        record_steps()
        cabi.check(L.grl_graph_end(dev.h, C.byref(g)))
        run = lambda: cabi.check(L.grl_graph_launch(dev.h, g))
    else:
        run = record_steps
        record_steps()
    launches_per_run = L.grl_launch_count() - launches0
    reset()
    run()                                       # warm-up run
    dev.sync()
    best = None
    e0, e1 = dev.event(), dev.event()
    for _ in range(repeats):
        reset()
        dev.sync()
        dist["barrier"]()
        dev.record(e0)
        run()
        dev.record(e1)
        dev.sync()
        ms = dist["max"](dev.elapsed_ms(e0, e1))
        best = ms if best is None else min(best, ms)
    o_last = dev.download(C.c_void_p(out.value + (steps - 1) * B * Hq * D * 4), (B, Hq, D), np.float32)
    assert np.isfinite(o_last).all()
    if use_graph:
        L.grl_graph_destroy(g)
    for x in (kp, vp, table, seq_lens, qs, ks, vs, q_rot, out, ws):
        dev.free(x)
    return best, launches_per_run, ns.value


def bench_evict(dev, cabi, repeats=3):
    """Eviction on a cfg3-sized cache (B32, Hkv8, D128, 4096 tokens, bf16): H2O selection of a quarter of every
    sequence, then compaction.  Returns (select_us, compact_us, bytes moved by one compaction)."""
    from oracle import attention_oracle as orc
    c = CFG3
    B, Hkv, D, T, P = c["B"], c["Hkv"], c["D"], c["T0"], c["page"]
    L = dev.L
    rng = np.random.default_rng(7)
    max_pages = T // P
    n_pages, page_elems = max_pages * B, Hkv * P * D
    kp, vp = dev.malloc(n_pages * page_elems * 2), dev.malloc(n_pages * page_elems * 2)
    for p_ in (kp, vp):
        cabi.check(L.grl_memset(dev.h, p_, 0x3c, n_pages * page_elems * 2))
    table = dev.upload(np.arange(n_pages, dtype=np.int32).reshape(B, max_pages))
    lens_host = np.full(B, T, np.int32)
    seq_lens = dev.upload(lens_host)
    lay = cabi.KVLayout()
    lay.k_pages, lay.v_pages, lay.cache_dtype = kp, vp, cabi.BF16
    lay.block_table, lay.seq_lens = table, seq_lens
    lay.batch, lay.num_kv_heads, lay.head_dim, lay.page_tokens, lay.max_pages, lay.num_pages = B, Hkv, D, P, max_pages, n_pages
    cap = max_pages * P
    scores = rng.random((B, cap), dtype=np.float32)
    cum, tomb, evicted = dev.malloc(B * cap * 4), dev.malloc(B * cap), dev.malloc(B * 4)
    m = cabi.KVMeta()
    m.cum_score, m.tombstone, m.relevance, m.evicted, m.capacity = cum, tomb, None, evicted, cap
    nb = C.c_size_t()
    cabi.check(L.grl_kv_compact_scratch_bytes(C.byref(lay), C.byref(m), C.byref(nb)))
    scratch = dev.malloc(nb.value)
    e0, e1, e2 = dev.event(), dev.event(), dev.event()
    best_sel = best_cmp = None
    for _ in range(repeats + 1):
        cabi.check(L.grl_memcpy_h2d(dev.h, seq_lens, lens_host.ctypes.data_as(C.c_void_p), lens_host.nbytes))
        cabi.check(L.grl_memcpy_h2d(dev.h, cum, scores.ctypes.data_as(C.c_void_p), scores.nbytes))
        cabi.check(L.grl_memset(dev.h, tomb, 0, B * cap))
        cabi.check(L.grl_memset(dev.h, evicted, 0, B * 4))
        dev.sync()
        dev.record(e0)
        cabi.check(L.grl_kv_evict_lowest(dev.h, C.byref(lay), C.byref(m), T // 4))
        dev.record(e1)
        cabi.check(L.grl_kv_compact(dev.h, C.byref(lay), C.byref(m), scratch, nb.value))
        dev.record(e2)
        dev.sync()
        sel, cmp_ = dev.elapsed_ms(e0, e1) * 1e3, dev.elapsed_ms(e1, e2) * 1e3
        best_sel = sel if best_sel is None else min(best_sel, sel)
        best_cmp = cmp_ if best_cmp is None else min(best_cmp, cmp_)
    left = dev.download(seq_lens, (B,), np.int32)
    assert (left == T - T // 4).all(), left
    moved = 2 * 2 * B * (T - T // 4) * Hkv * D * 2          # K and V, survivors read and written, bf16
    for x in (kp, vp, table, seq_lens, cum, tomb, evicted, scratch):
        dev.free(x)
    return best_sel, best_cmp, moved


def bench_decode_e2e(dist, steps=32):
    """grilly_core.decode_step with host arrays per step (upload q/k/v, append, attend, download)."""
    import grilly_core
    c = CFG3
    B, Hq, Hkv, D, T0 = c["B"], c["Hq"], c["Hkv"], c["D"], c["T0"]
    rng = np.random.default_rng(c["seed"])
    ctx = grilly_core.Device()
    kv = grilly_core.create_kv_cache(ctx, num_heads=Hkv, head_dim=D, compression_ratio=1, max_cache_tokens=T0 + steps + 8,
                                     use_h2o=False, batch_size=B, page_tokens=c["page"], dtype="bf16")
    blk = 512
    for _ in range(T0 // blk):
        k0 = rng.standard_normal((B, blk, Hkv, D), dtype=np.float32)
        grilly_core.kv_cache_append(ctx, kv, k0, k0)
    from grilly_next import cabi
    L = cabi.lib()
    q, qp = pinned_array(L, (B, 1, Hq, D), np.float32)
    k1, kp = pinned_array(L, (B, 1, Hkv, D), np.float32)
    o, op = pinned_array(L, (B, 1, Hq, D), np.float32)
    q[...] = rng.standard_normal(q.shape, dtype=np.float32)
    k1[...] = rng.standard_normal(k1.shape, dtype=np.float32)
    for _ in range(4):
        grilly_core.decode_step(ctx, kv, q, k1, k1, rope_theta=c["theta"], out=o)
    dist["barrier"]()
    t0 = time.perf_counter()
    for _ in range(steps):
        grilly_core.decode_step(ctx, kv, q, k1, k1, rope_theta=c["theta"], out=o)
    dt = dist["max"]((time.perf_counter() - t0) / steps)
    assert np.isfinite(o).all()
    grilly_core.destroy_kv_cache(ctx, kv)
    nb = (q.nbytes + 2 * k1.nbytes, o.nbytes)
    del q, k1, o
    for pp in (qp, kp, op):
        L.grl_host_free(pp)
    return dt, nb[0], nb[1]


def bench_long_decode(dev, cabi, dist, steps=50, repeats=3, n_splits=0):
    """cfg4: B=1, Hq32/Hkv8, D128, KV length 131072 split in contiguous shards over the ranks; per step
    every rank decodes its shard to one partial, the partials cross NVLink (peer stores, or NCCL all-gather
    with GRILLY_EXCHANGE=nccl) and every rank merges."""
    import torch
    import torch.distributed as td
    from grilly_next.parallel import CudaShardOps, ShardedDecoder, shard_range, torch_stream_handle
    from oracle import attention_oracle as orc
    c = CFG4
    B, Hq, Hkv, D, T, P = 1, c["Hq"], c["Hkv"], c["D"], c["T"], 64
    world, rank = dist["world"], dist["rank"]
    lo, hi = shard_range(T, world, rank)
    Tg = hi - lo
    L = dev.L
    cabi.check(L.grl_device_use_stream(dev.h, torch_stream_handle(torch)))
    n_pages = (Tg + P - 1) // P
    page_elems = Hkv * P * D
    shard_bytes = 2 * n_pages * page_elems * 2
    nbuf = max(1, -(-(512 << 20) // shard_bytes))        # rotate buffers so that a shard never sits in L2
    rng = np.random.default_rng(c["seed"] + rank)
    bits = orc.to_bf16_bits(rng.standard_normal(32 * page_elems, dtype=np.float32))
    pools = []
    for _ in range(nbuf):
        pair = []
        for _kv in range(2):
            t = torch.empty(n_pages * page_elems, dtype=torch.int16, device="cuda")
            src = torch.from_numpy(np.roll(bits, int(rng.integers(0, bits.size))).view(np.int16)).cuda()
            reps = -(-t.numel() // src.numel())
            t.copy_(src.repeat(reps)[: t.numel()])
            pair.append(t)
        pools.append(pair)
    table = torch.arange(n_pages, dtype=torch.int32, device="cuda").reshape(B, n_pages)
    lens = torch.full((B,), Tg, dtype=torch.int32, device="cuda")
    q = torch.from_numpy(rng.standard_normal((B, 1, Hq, D), dtype=np.float32)).cuda()
    if world > 1:
        td.broadcast(q, src=0)

    def layout(i):
        l = cabi.KVLayout()
        l.k_pages, l.v_pages, l.cache_dtype = pools[i][0].data_ptr(), pools[i][1].data_ptr(), cabi.BF16
        l.block_table, l.seq_lens = table.data_ptr(), lens.data_ptr()
        l.batch, l.num_kv_heads, l.head_dim, l.page_tokens, l.max_pages, l.num_pages = B, Hkv, D, P, n_pages, n_pages
        return l

    ops = CudaShardOps(cabi, dev, layout(0), Hq, Tg, torch, n_splits=n_splits)
    fused = ""
    mode = os.environ.get("GRILLY_EXCHANGE", "decode")     # profiling aid: "nccl" | "merge" | "decode"
    if world > 1 and mode != "nccl":
        # peers' inboxes over CUDA IPC; NCCL all-gather is the fallback
        if ops.setup_p2p(td, one_launch=(mode == "decode"), low_latency=(mode != "merge")):
            fused = "decode" if ops.one_launch else ("ll" if mode == "ll" else "merge")
    dec = ShardedDecoder(td if world > 1 else _NoDist(), ops, lambda n, m: torch.empty((n, m), dtype=torch.float32, device="cuda"))
    layouts = [layout(i) for i in range(nbuf)]
    for i in range(5):
        ops.set_layout(layouts[i % nbuf]); out = dec.step(q)
    torch.cuda.synchronize()

    def run_steps():
        o = None
        for i in range(steps):
            ops.set_layout(layouts[i % nbuf]); o = dec.step(q)
        return o

    # The step is one to three small launches: replay `steps` of them from one CUDA graph so that launch
    # latency does not hide the kernels.  The library's launches are captured like any
    # other work on the capturing stream (grl_device_use_stream).
    graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            cabi.check(L.grl_device_use_stream(dev.h, torch_stream_handle(torch)))
            out = run_steps()
        cabi.check(L.grl_device_use_stream(dev.h, torch_stream_handle(torch)))
        graph.replay()
        torch.cuda.synchronize()
    except Exception as e:          # fall back to plain launches, and say so
        graph = None
        cabi.check(L.grl_device_use_stream(dev.h, torch_stream_handle(torch)))
        sys.stderr.write(f"long decode: graph capture unavailable ({e}); timing plain launches\n")
    best = None
    e0, e1 = dev.event(), dev.event()
    launches0 = L.grl_launch_count()
    for _ in range(repeats):
        dist["barrier"]()
        dev.record(e0)
        if graph is not None:
            graph.replay()
        else:
            out = run_steps()
        dev.record(e1)
        torch.cuda.synchronize()
        ms = dist["max"](dev.elapsed_ms(e0, e1))
        best = ms if best is None else min(best, ms)
    # this library's launches per step: the decode kernel merges its own splits; NCCL mode adds the final merge
    # (the all-gather is NCCL's kernel), "merge" mode the step-counter bump and the exchange+merge kernel
    launches = {"": 1 if world == 1 else 2, "merge": 3, "ll": 3, "decode": 1}[fused]
    assert bool(torch.isfinite(out).all())
    cabi.check(L.grl_device_use_stream(dev.h, None))
    return best / steps, launches, ops.p.n_splits, nbuf, graph is not None, fused


class _NoDist:
    def is_initialized(self):
        return False


def cpu_baseline():
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())
    from oracle import attention_oracle as orc
    from oracle import c_oracle
    c = CFG2
    heads = 32
    rng = np.random.default_rng(c["seed"])
    Q, K, V = (rng.standard_normal((1, heads, c["S"], c["D"]), dtype=np.float32) for _ in range(3))
    pos = np.arange(c["S"])
    c_oracle.attention(Q[:, :2], K[:, :2], V[:, :2], causal=True)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 10.0 and reps < 8:
        c_oracle.attention(orc.rope_interleaved(Q, pos, c["theta"]), orc.rope_interleaved(K, pos, c["theta"]), V, causal=True)
        reps += 1
    dt = time.perf_counter() - t0
    fl = 4 * c["D"] * heads * (c["S"] * (c["S"] + 1) // 2) * reps
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": c_oracle.num_threads(), "kind": "port",
            "sample": f"{reps} passes over {heads} of 128 (batch, head) slices of cfg2 (RoPE + causal attention), C/OpenMP oracle"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-decode", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true", help="profiling aid: run the decode workload only")
    ap.add_argument("--no-graph", action="store_true", help="profiling aid: plain launches instead of graph replay")
    ap.add_argument("--decode-repeats", type=int, default=3)
    ap.add_argument("--decode-splits", type=int, default=0, help="profiling aid: force the split-KV count (0 = library choice)")
    ap.add_argument("--variant", default="cfg2", choices=["cfg2", "norope", "noncausal"],
                    help="profiling aid: drop RoPE or the causal mask from the prefill workload")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-long", action="store_true", help="skip the long-context (cfg4) decode leg")
    ap.add_argument("--skip-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        return run_reference(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = {"rank": rank, "world": world, "local_rank": local_rank, "barrier": lambda: None, "max": lambda x: x}
    if world > 1:
        import torch
        import torch.distributed as td
        torch.cuda.set_device(local_rank)
        td.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

        def _barrier():
            td.barrier()
            torch.cuda.synchronize()

        def _max(x):
            t = torch.tensor([x], dtype=torch.float64, device="cuda")
            td.all_reduce(t, op=td.ReduceOp.MAX)
            return float(t.item())

        dist["barrier"], dist["max"] = _barrier, _max

    if world == 1 and not (args.skip_decode or args.skip_long):
        import torch
        torch.cuda.set_device(local_rank)
    from grilly_next import cabi
    if os.environ.get("GRL_LIB_OVERRIDE"):      # profiling aid: try an experimental build of the library
        cabi.LIB_PATH = os.environ["GRL_LIB_OVERRIDE"]
    dev = cabi.Device(local_rank)          # raises if the CUDA library or the GPU is missing: no fallback
    L = dev.L
    pk = peaks()

    if args.skip_prefill:
        dms, dl, nsplit = bench_decode(dev, cabi, dist, args.decode_repeats, not args.no_graph, args.decode_splits)
        print(json.dumps({"decode_ms": dms, "launches": int(dl), "n_splits": nsplit}), flush=True)
        dev.close()
        return
    ms, launches, clocks = bench_prefill(dev, cabi, args, dist)
    fl = prefill_flops(CFG2)
    if args.variant == "noncausal":
        fl = 4 * CFG2["D"] * CFG2["B"] * CFG2["H"] * CFG2["S"] * CFG2["S"]
    tflops_gpu = fl * args.steps / (ms * 1e-3) / 1e12
    value = tflops_gpu * world
    line = {
        "metric": "prefill_attn_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "cfg2: FlashAttention-2+RoPE causal prefill, B4 H32 S2048 D128, bf16 in / fp32 out, per GPU"
                   + ("" if args.variant == "cfg2" else f" [variant {args.variant}: NOT the benchmark configuration]"),
                   "flops_per_step_per_gpu": fl, "l2": "inputs larger than L2 (320 MiB per step)",
                   "parallelism": f"replica per GPU x{world}, no collective"},
        "clocks": clocks, "gpu_launches": int(launches),
        "roofline": prefill_roofline(tflops_gpu, ms, pk),
    }

    if not args.skip_decode:
        dms, dl, nsplit = bench_decode(dev, cabi, dist, args.decode_repeats, not args.no_graph, args.decode_splits)
        c = CFG3
        toks = c["B"] * c["steps"] / (dms * 1e-3)
        gbs = decode_bytes(c) / (dms * 1e-3) / 1e9
        line["decode"] = {"metric": "decode_tokens_per_s", "value": toks * world, "unit": "tokens/s",
                          "ms_per_step": dms / c["steps"], "workload": "cfg3: GQA decode B32 Hq32/Hkv8 D128 KV 4096->4352, 256 steps, bf16 paged cache, CUDA-graph replay, per GPU",
                          "gpu_launches": int(dl), "n_splits": nsplit,
                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s", "frac": gbs / pk["hbm"],
                                       "traffic": DECODE_TRAFFIC_BYTES, "peak_source": pk["src"], "frac_of_nominal_8000": gbs / 8000.0,
                                       "note": "achieved = algorithmic bytes of the 256-step run / its time (append + decode + merge per step)",
                                       "kernel": "decode_mma_kernel"}}

    if not args.skip_decode and world == 1:
        sel_us, cmp_us, moved = bench_evict(dev, cabi)
        gbs = moved / (cmp_us * 1e-6) / 1e9
        line["evict"] = {"workload": "cfg3-sized cache (B32 Hkv8 D128 4096 tokens bf16): H2O selection of a quarter of every sequence, "
                                     "then compaction", "select_us": sel_us, "compact_us": cmp_us,
                         "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s", "frac": gbs / pk["hbm"],
                                      "peak_source": pk["src"], "note": "surviving K/V rows read once and written once; rows that stay in place are skipped, so this is an upper bound on the traffic"}}
    if not args.skip_decode and not args.skip_long:
        lms, ll, lsplit, nbuf, graphed, fused = bench_long_decode(dev, cabi, dist)
        kv_bytes = 2 * CFG4["Hkv"] * CFG4["D"] * 2 * CFG4["T"]
        gbs = kv_bytes / (lms * 1e-3) / 1e9
        line["decode_long"] = {"metric": "decode_long_tokens_per_s", "value": 1.0 / (lms * 1e-3), "unit": "tokens/s",
                               "ms_per_step": lms, "scaling": "strong",
                               "workload": f"cfg4: GQA decode B1 Hq32/Hkv8 D128 KV 131072 bf16 split over {world} GPU(s); "
                                           + ("18 splits merged inside the decode kernel" if world == 1 else "per-GPU partial (16,640 B/rank) + ")
                                           + {"decode": "exchange over NVLink peer stores and LSE merge inside the decode kernel (one launch per step)",
                                              "merge": "exchange over NVLink peer stores fused with the LSE merge",
                                              "ll": "exchange over NVLink peer stores ({value, step} pairs, no flag) fused with the LSE merge",
                                              "": "NCCL all-gather + LSE merge" if world > 1 else ""}[fused]
                                           + f"; {nbuf} rotating KV buffers (L2); "
                                           + ("CUDA-graph replay" if graphed else "plain launches"),
                               "gpu_launches_per_step": int(ll), "n_splits": lsplit,
                               "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"] * world, "unit": "GB/s",
                                            "frac": gbs / (pk["hbm"] * world), "peak_source": pk["src"] + f" x{world}"}}
    if not args.skip_e2e:
        os.environ["GRILLY_GPU_INDEX"] = str(local_rank)     # the op layer's device selector
        dt, h2d, d2h = bench_prefill_e2e(args, L, min(args.steps, 5), dist)
        line["e2e"] = {"value": fl / dt / 1e12 * world, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "ms_per_step": dt * 1e3, "api": "grilly_core.flash_attention2(dtype='bf16', out=pinned), pinned fp32 host arrays in and out; "
                              "h2d bytes are what crosses the link (the op rounds inputs to bf16 on host threads; 402,653,184 B of fp32 are read)"}
        if not args.skip_decode:
            ddt, dh2d, dd2h = bench_decode_e2e(dist)
            line["decode"]["e2e"] = {"value": CFG3["B"] / ddt * world, "unit": "tokens/s", "h2d_bytes_per_step": dh2d,
                                     "d2h_bytes_per_step": dd2h, "ms_per_step": ddt * 1e3, "api": "grilly_core.decode_step(out=pinned), pinned fp32 host arrays in and out"}
    if rank == 0 and world == 1 and not args.skip_cpu:
        line["cpu_baseline"] = cpu_baseline()

    dev.close()
    if world > 1:
        import torch.distributed as td
        td.barrier()
        td.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
