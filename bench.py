#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--legs a,b,...]

One JSON line on stdout (rank 0).  Headline metric: prefill attention TFLOP/s on configuration 2
(FlashAttention-2 + RoPE, causal, batch 4, 32 heads, seq 2048, head_dim 128, bf16 tensor-core
path).  The other configurations are measured in the same run and reported as objects of the same
line: "cfg1" (fp32 exact path, absolute time), "cfg5" (padded batch of ragged lengths), "decode"
(configuration 3: GQA decode, batch 32, 32/8 heads, KV 4096 -> 4352, 256 steps), "decode_long"
(configuration 4: KV length 131072 sharded over the GPUs), "evict" (H2O selection + compaction).
Synthetic N(0,1) inputs from a seed.

A step is one pass of the hot path over one batch.  `value` times the kernel with inputs resident
in HBM (CUDA events on the library's stream); `e2e` times the public Python op
(grilly_core.flash_attention2 / decode_step) with pinned HOST buffers, copies inside the timed
region.  With N > 1 (torchrun, one process per GPU) every rank runs the same per-GPU workload on
its own GPU (weak scaling, no data-path collective) for the headline; "strong_scaling" times ONE
problem whose (batch, head) slices are split over the ranks; configuration 4 is strong scaling by
construction.  Times are the max over ranks.  Every leg checks one sampled result against the CPU
oracle before it is timed ("parity"); a result outside its tolerance ends the run with a non-zero
exit code.

Legs (--legs, default all): prefill, cfg1, cfg5, decode, evict, long, e2e, cpu.
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

CFG1 = dict(B=1, H=4, S=256, D=64, seed=1001)
CFG2 = dict(B=4, H=32, S=2048, D=128, theta=10000.0, seed=1002)
CFG3 = dict(B=32, Hq=32, Hkv=8, D=128, T0=4096, steps=256, theta=10000.0, seed=1003, page=64)
CFG4 = dict(Hq=32, Hkv=8, D=128, T=131072, seed=1004)
CFG5 = dict(B=8, H=32, S=4096, D=128, theta=10000.0, seed=1005)
ALL_LEGS = ("prefill", "cfg1", "cfg5", "decode", "evict", "linear", "long", "e2e", "cpu")
TOL_BF16_PREFILL, TOL_FP32_PREFILL, TOL_DECODE = 2e-2, 1e-4, 5e-3

# dram__bytes_read.sum + dram__bytes_write.sum of one launch (ncu, see profiles/)
PREFILL_TRAFFIC_BYTES = 208.9e6 + 103.1e6   # flash_fwd_sm100_kernel on cfg2
DECODE_TRAFFIC_BYTES = 546.1e6 + 11.0e6     # decode_mma_kernel at cache length ~4117


def causal_flops(D, heads, lens):
    """4*D FLOP per visible (q, k) pair: QK^T and PV, multiply and add."""
    return 4 * D * heads * sum(int(L) * (int(L) + 1) // 2 for L in lens)


def decode_bytes(c):
    """Algorithmic bytes of the 256-step run: K+V rows attended (bf16) + q read + O write + append write."""
    per_pos = 2 * c["B"] * c["Hkv"] * c["D"] * 2
    kv = sum(per_pos * (c["T0"] + t + 1) for t in range(c["steps"]))
    other = c["steps"] * (c["B"] * c["Hq"] * c["D"] * (4 + 4) + 2 * c["B"] * c["Hkv"] * c["D"] * 2)
    return kv + other


def to_bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def round_bf16(x):
    return (to_bf16_bits(x).astype(np.uint32) << np.uint32(16)).view(np.float32).reshape(np.shape(x))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tf=d["bf16_tflops"], tf_sustained=d.get("bf16_tflops_sustained"), src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, src="fallback")


def prefill_roofline(tflops_gpu, timed_ms, pk, traffic=None):
    """The prefill kernel against the measured cuBLAS bf16 rate: the burst figure when the timed region is
    short (clocks still at boost), the sustained one when it runs long enough to sit under the power cap."""
    long_run = timed_ms > 100.0 and pk["tf_sustained"]
    peak = pk["tf_sustained"] if long_run else pk["tf"]
    return {"bound": "tensor", "achieved": tflops_gpu, "peak": peak, "unit": "TFLOP/s", "frac": tflops_gpu / peak,
            "traffic": traffic, "peak_source": pk["src"] + (" (sustained: timed region > 100 ms)" if long_run else " (burst)"),
            "frac_of_burst": tflops_gpu / pk["tf"],
            "frac_of_sustained": tflops_gpu / pk["tf_sustained"] if pk["tf_sustained"] else None,
            "frac_of_nominal_2250": tflops_gpu / 2250.0, "kernel": "flash_fwd_sm100_kernel"}


class ParityError(RuntimeError):
    pass


def parity(name, max_abs, tol, **extra):
    d = {"max_abs": float(max_abs), "tol": tol, **extra}
    if not (max_abs <= tol):
        raise ParityError(f"{name}: max-abs {max_abs:.3e} exceeds {tol:.1e} ({extra})")
    return d


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons from start() to stop(); regions are marked by time."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

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
        if self.proc:
            self.proc.terminate()
            self.t.join(timeout=2)

    def region(self, t0, t1):
        """Median SM clock and the throttle reasons seen between two time.time() stamps."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        rows = [r[1:] for r in self.rows if len(r) >= 7 and t0 <= r[0] <= t1 + 0.02]
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 7 and r[2].replace(".", "").isdigit()]
        reasons = [n for i, n in enumerate(self.NAMES) if any(r[2 + i] == "Active" for r in rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------- reference arm
def run_reference(args):
    """The reference's CPU implementation of the path: its Vulkan shaders cannot run here (no
    graphics stack) and its C++ library does not build without the Vulkan SDK, so this arm times
    the C restatement of its CPU attention (oracle/attn_oracle.c, OpenMP, all host threads), the
    rotation of Q and K included (also C/OpenMP)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())   # torchrun pins it to 1; this arm may use every host thread
    from oracle import c_oracle
    c = CFG2
    heads = 32                                   # bounded sample: 32 of the 128 (batch, head) pairs per step
    rng = np.random.default_rng(c["seed"])
    Q, K, V = (rng.standard_normal((1, heads, c["S"], c["D"]), dtype=np.float32) for _ in range(3))
    fl = causal_flops(c["D"], heads, [c["S"]])

    def step():
        c_oracle.attention(c_oracle.rope_interleaved(Q, c["theta"]), c_oracle.rope_interleaved(K, c["theta"]), V, causal=True)

    for _ in range(max(1, min(args.warmup, 2))):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    t1 = time.perf_counter()
    c_oracle.rope_interleaved(Q, c["theta"]); c_oracle.rope_interleaved(K, c["theta"])
    rope_share = (time.perf_counter() - t1) / (dt / args.steps)
    val = fl * args.steps / dt / 1e12
    line = {
        "impl": "reference", "metric": "prefill_attn_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg2: FlashAttention-2+RoPE causal prefill, B4 H32 S2048 D128", "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": c_oracle.num_threads(), "kind": "port",
                         "sample": f"{heads} of 128 (batch, head) slices of cfg2 per step, RoPE (C/OpenMP, {rope_share:.1%} of the "
                                   "step) + causal attention, C/OpenMP"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------- plumbing
class Dist:
    """One process per GPU.  torch.distributed (NCCL) is plumbing only: barrier, max over ranks, and the
    host channel that carries the NCCL id and the CUDA IPC handles of the library's own exchange."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.td = None
        if self.world > 1:
            import torch
            import torch.distributed as td
            torch.cuda.set_device(self.local_rank)
            td.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.td, self.torch = td, torch

    def barrier(self):
        if self.td:
            self.td.barrier()
            self.torch.cuda.synchronize()

    def max(self, x):
        if not self.td:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.td.all_reduce(t, op=self.td.ReduceOp.MAX)
        return float(t.item())

    def all_gather_bytes(self, payload):
        if not self.td:
            return [bytes(payload)]
        out = [None] * self.world
        self.td.all_gather_object(out, bytes(payload))
        return out

    def close(self):
        if self.td:
            self.td.barrier()
            self.td.destroy_process_group()


def pinned_array(L, shape, dtype):
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    p = C.c_void_p()
    rc = L.grl_host_alloc(n, C.byref(p))
    if rc != 0:
        raise RuntimeError(L.grl_last_error().decode())
    buf = (C.c_char * n).from_address(p.value)
    return np.frombuffer(buf, dtype=dtype).reshape(shape), p


def fill_random_bf16(dev, cabi, dst, n_elems, rng, block_elems=1 << 21):
    """iid N(0,1) bf16 over a large device buffer: one random block from the host, then doubling copies on
    the device.  (The timed kernels read every element once; their time does not depend on the values.)"""
    L = dev.L
    m = min(block_elems, n_elems)
    bits = to_bf16_bits(rng.standard_normal(m, dtype=np.float32))
    cabi.check(L.grl_memcpy_h2d(dev.h, dst, bits.ctypes.data_as(C.c_void_p), m * 2))
    dev.sync()
    filled = m
    while filled < n_elems:
        k = min(filled, n_elems - filled)
        cabi.check(L.grl_memcpy_d2d(dev.h, C.c_void_p(dst.value + filled * 2), dst, k * 2))
        filled += k
    dev.sync()


def time_steps(dev, dist, step, steps):
    """steps launches between two events on the library's stream; max over ranks, in ms."""
    e0, e1 = dev.event(), dev.event()
    dev.sync()
    dist.barrier()
    dev.record(e0)
    for _ in range(steps):
        step()
    dev.record(e1)
    dev.sync()
    ms = dev.elapsed_ms(e0, e1)
    for e in (e0, e1):
        dev.L.grl_event_destroy(e)
    return dist.max(ms)


def flash_params(cabi, q, k, v, o, B, H, S, D, *, bf16, causal=True, theta=0.0, seq_lens=None, kernel=None, scale=0.0):
    p = cabi.FlashParams()
    p.q, p.k, p.v, p.o = q, k, v, o
    p.in_dtype, p.out_dtype = (cabi.BF16 if bf16 else cabi.F32), cabi.F32
    p.batch, p.heads, p.seq_len, p.head_dim = B, H, S, D
    p.causal, p.scale = int(causal), scale
    if theta:
        p.rope_mode, p.rope_theta, p.rope_scaling = cabi.ROPE_INTERLEAVED, theta, 1.0
    if seq_lens is not None:
        p.seq_lens = seq_lens
    p.kernel = kernel if kernel is not None else (cabi.KERNEL_TCGEN05 if bf16 else cabi.KERNEL_SIMT_F32)
    return p


def oracle_head(Qh, Kh, Vh, theta, causal=True, length=None):
    """The checker on one (batch, head) slice: RoPE + causal attention in float32 on the unrounded inputs."""
    from oracle import c_oracle
    q, k = Qh[None, None], Kh[None, None]
    if theta:
        q, k = c_oracle.rope_interleaved(q, theta), c_oracle.rope_interleaved(k, theta)
    sl = None if length is None else np.array([length], np.int32)
    return c_oracle.attention(q, k, Vh[None, None], causal=causal, seq_lens=sl)[0, 0]


# ------------------------------------------------------------------------------------- prefill legs
def bench_prefill(dev, cabi, args, dist, pk, sampler):
    """cfg2 on every GPU (the headline), the same block repeated for a sustained figure, and -- with several
    GPUs -- the ONE problem split by heads over the ranks."""
    c = CFG2
    B, H, S, D = c["B"], c["H"], c["S"], c["D"]
    rng = np.random.default_rng(c["seed"] + dist.rank)
    n = B * H * S * D
    sb, sh = B - 1, 5                                   # the sampled (batch, head) slice of the parity check
    host, dptr = [], []
    for _ in range(3):
        a = rng.standard_normal((B, H, S, D), dtype=np.float32)
        host.append(a[sb, sh].copy())
        dptr.append(dev.upload_bf16(a))
        del a
    q, k, v = dptr
    o = dev.malloc(n * 4)
    L = dev.L
    p = flash_params(cabi, q, k, v, o, B, H, S, D, bf16=True, theta=c["theta"])

    def step():
        cabi.check(L.grl_flash_fwd(dev.h, C.byref(p)))

    for _ in range(args.warmup):
        step()
    dev.sync()
    got = dev.download(C.c_void_p(o.value + (sb * H + sh) * S * D * 4), (S, D), np.float32)
    par = parity("prefill cfg2", np.abs(got - oracle_head(*host, c["theta"])).max(), TOL_BF16_PREFILL,
                 sample=f"(batch, head) = ({sb}, {sh}) of rank {dist.rank}, all {S} rows, against the fp32 oracle on the unrounded inputs")
    launches0 = L.grl_launch_count()
    t0 = time.time()
    ms = time_steps(dev, dist, step, args.steps)
    t1 = time.time()
    launches = L.grl_launch_count() - launches0
    fl = causal_flops(D, B * H, [S])
    tflops_gpu = fl * args.steps / (ms * 1e-3) / 1e12
    # the same block back to back until the timed region is long enough for the clock sampler (and the power cap)
    reps, t2 = max(1, int(np.ceil(0.5 / max(ms * 1e-3, 1e-6)))), time.time()
    ms_long = time_steps(dev, dist, step, args.steps * reps) if reps > 1 else ms
    t3 = time.time()
    tf_long = fl * args.steps * reps / (ms_long * 1e-3) / 1e12
    ck_short, ck_long = sampler.region(t0, t1), sampler.region(t2, t3)
    clocks = dict(ck_short if ck_short["samples"] >= 3 else ck_long)
    clocks["region"] = "headline timed region" if ck_short["samples"] >= 3 else "sustained repeat of the timed block (the headline region is shorter than the sampler's period)"
    clocks["headline_samples"] = ck_short["samples"]
    out = {"ms": ms, "launches": launches, "tflops_gpu": tflops_gpu, "flops": fl, "clocks": clocks, "parity": par,
           "sustained": {"value": tf_long * dist.world, "unit": "TFLOP/s", "ms_per_step": ms_long / (args.steps * reps),
                         "timed_region_ms": ms_long, "steps": args.steps * reps, "clocks": ck_long,
                         "ms_x_mhz": (ms_long / (args.steps * reps)) * ck_long["sm_mhz"] if ck_long["sm_mhz"] else None,
                         "frac_of_sustained_peak": tf_long / pk["tf_sustained"] if pk["tf_sustained"] else None}}
    if dist.world > 1 and H % dist.world == 0:
        # strong scaling: the 128 (batch, head) slices of ONE cfg2 problem, heads split over the ranks
        Hl = H // dist.world
        ps = flash_params(cabi, q, k, v, o, B, Hl, S, D, bf16=True, theta=c["theta"])
        steps = args.steps
        for _ in range(args.warmup):
            cabi.check(L.grl_flash_fwd(dev.h, C.byref(ps)))
        ms_s = time_steps(dev, dist, lambda: cabi.check(L.grl_flash_fwd(dev.h, C.byref(ps))), steps)
        out["strong"] = {"value": fl * steps / (ms_s * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_s / steps,
                         "scaling": "strong", "parallelism": f"one cfg2 problem, {Hl} of {H} heads per GPU (x{B} batch rows), no collective",
                         "ctas_per_gpu": B * Hl * (S // 256)}
    for x in (q, k, v, o):
        dev.free(x)
    return out


def bench_cfg1(dev, cabi, args, dist):
    """cfg1: the exact fp32 path, B1 H4 S256 D64 causal -- 33.7 MFLOP, bounded by launch latency: absolute time."""
    c = CFG1
    B, H, S, D = c["B"], c["H"], c["S"], c["D"]
    rng = np.random.default_rng(c["seed"])
    Q, K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(3))
    L = dev.L
    q, k, v = dev.upload(Q), dev.upload(K), dev.upload(V)
    o = dev.malloc(Q.nbytes)
    p = flash_params(cabi, q, k, v, o, B, H, S, D, bf16=False, scale=0.125)
    cabi.check(L.grl_flash_fwd(dev.h, C.byref(p)))
    dev.sync()
    from oracle import c_oracle
    got = dev.download(o, Q.shape, np.float32)
    par = parity("prefill cfg1", np.abs(got - c_oracle.attention(Q, K, V, causal=True, scale=0.125)).max(), TOL_FP32_PREFILL,
                 sample="all heads and rows")
    # cold: 1 MiB of tensors would sit in L2, so a 256 MiB write flushes it before every timed launch
    flush = dev.malloc(256 << 20)
    e0, e1 = dev.event(), dev.event()
    cold = []
    for _ in range(12):
        cabi.check(L.grl_memset(dev.h, flush, 0, 256 << 20))
        dev.record(e0)
        cabi.check(L.grl_flash_fwd(dev.h, C.byref(p)))
        dev.record(e1)
        dev.sync()
        cold.append(dev.elapsed_ms(e0, e1) * 1e3)
    warm = time_steps(dev, dist, lambda: cabi.check(L.grl_flash_fwd(dev.h, C.byref(p))), 200) / 200 * 1e3
    for x in (q, k, v, o, flush):
        dev.free(x)
    cold_us = float(np.median(cold[2:]))
    fl = causal_flops(D, B * H, [S])
    res = {"workload": "cfg1: flash-attention2 fp32 exact path, B1 H4 S256 D64 causal, scale 1/8 (flash_fwd_f32_kernel)",
           "us_per_call": cold_us, "us_per_call_l2_warm": warm, "flops": fl, "gflops": fl / cold_us / 1e3,
           "l2": "cold figure: L2 flushed by a 256 MiB write before every timed launch; warm: 200 launches back to back",
           "bound": "launch latency and fp32 FMA (no tensor cores on the exact path)", "parity": par}
    return res, (Q, K, V)


def bench_cfg1_e2e(qkv, dist):
    import grilly_core
    ctx = grilly_core.Device()
    Q, K, V = qkv
    for _ in range(3):
        grilly_core.flash_attention2(ctx, Q, K, V, causal=True, scale=0.125)
    t0 = time.perf_counter()
    for _ in range(50):
        out = grilly_core.flash_attention2(ctx, Q, K, V, causal=True, scale=0.125)
    dt = dist.max((time.perf_counter() - t0) / 50)
    assert np.isfinite(out).all()
    return {"us_per_call": dt * 1e6, "h2d_bytes_per_step": 3 * Q.nbytes, "d2h_bytes_per_step": Q.nbytes,
            "api": "grilly_core.flash_attention2(causal=True, scale=0.125) on numpy arrays"}


def bench_cfg5(dev, cabi, args, dist, pk):
    """cfg5: batch of 8 ragged sequences (512..4096 tokens) padded to 4096, causal + length mask, RoPE."""
    c = CFG5
    B, H, S, D = c["B"], c["H"], c["S"], c["D"]
    rng = np.random.default_rng(c["seed"])
    lens = rng.integers(512, 4097, size=B).astype(np.int32)
    n = B * H * S * D
    sb, sh = int(np.argmin(lens)), 3                     # the shortest sequence: padding rows and a ragged last tile
    host, dptr = [], []
    for _ in range(3):
        a = rng.standard_normal((B, H, S, D), dtype=np.float32)
        host.append(a[sb, sh].copy())
        dptr.append(dev.upload_bf16(a))
        del a
    q, k, v = dptr
    o = dev.malloc(n * 4)
    sl = dev.upload(lens)
    L = dev.L
    p = flash_params(cabi, q, k, v, o, B, H, S, D, bf16=True, theta=c["theta"], seq_lens=sl)
    steps = max(3, min(args.steps, 20))
    for _ in range(3):
        cabi.check(L.grl_flash_fwd(dev.h, C.byref(p)))
    dev.sync()
    got = dev.download(C.c_void_p(o.value + (sb * H + sh) * S * D * 4), (S, D), np.float32)
    Lb = int(lens[sb])
    want = oracle_head(*host, c["theta"], length=Lb)
    assert not got[Lb:].any(), "rows at or beyond the sequence length must be zero"
    par = parity("prefill cfg5", np.abs(got[:Lb] - want[:Lb]).max(), TOL_BF16_PREFILL,
                 sample=f"(batch, head) = ({sb}, {sh}), length {Lb}: valid rows against the fp32 oracle, padded rows exactly zero")
    ms = time_steps(dev, dist, lambda: cabi.check(L.grl_flash_fwd(dev.h, C.byref(p))), steps)
    fl = causal_flops(D, H, lens)
    tf = fl * steps / (ms * 1e-3) / 1e12
    res = {"metric": "prefill_attn_tflops", "value": tf * dist.world, "unit": "TFLOP/s", "ms_per_step": ms / steps, "steps": steps,
           "workload": f"cfg5: FlashAttention-2+RoPE, B8 H32 D128, lengths {lens.tolist()} padded to {S}, causal and length mask, "
                       "bf16 in / fp32 out, per GPU", "flops_per_step_per_gpu": fl, "scaling": "weak",
           "roofline": prefill_roofline(tf, ms, pk), "parity": par}
    if dist.world > 1 and H % dist.world == 0:
        Hl = H // dist.world
        ps = flash_params(cabi, q, k, v, o, B, Hl, S, D, bf16=True, theta=c["theta"], seq_lens=sl)
        for _ in range(3):
            cabi.check(L.grl_flash_fwd(dev.h, C.byref(ps)))
        ms_s = time_steps(dev, dist, lambda: cabi.check(L.grl_flash_fwd(dev.h, C.byref(ps))), steps)
        res["strong"] = {"value": fl * steps / (ms_s * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_s / steps, "scaling": "strong",
                         "parallelism": f"one cfg5 problem, {Hl} of {H} heads per GPU, all 8 sequences on every GPU, no collective"}
    for x in (q, k, v, o, sl):
        dev.free(x)
    return res


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
    sb, sh = 2, 11
    par = parity("prefill e2e", np.abs(out[sb, sh] - oracle_head(arrs[0][sb, sh], arrs[1][sb, sh], arrs[2][sb, sh], c["theta"])).max(),
                 TOL_BF16_PREFILL, sample=f"(batch, head) = ({sb}, {sh}) of the op's host result")
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        out = grilly_core.flash_attention2(ctx, *arrs, **kw)   # synchronous: returns with the result on the host
    dt = dist.max((time.perf_counter() - t0) / steps)
    info = grilly_core.last_pipeline_info()            # of the last timed call: what crossed the link
    h2d, d2h = int(info["h2d_bytes"]), int(info["d2h_bytes"])
    # one more call, untimed, with per-stage event timing on: which stage is the limiter
    grilly_core.set_pipeline_timing(True)
    grilly_core.flash_attention2(ctx, *arrs, **kw)
    stages = grilly_core.last_pipeline_info()
    grilly_core.set_pipeline_timing(False)
    busy = {k: stages[k] for k in ("host_round_ms", "h2d_busy_ms", "kernel_busy_ms", "d2h_busy_ms")}
    stages["limiter"] = max(busy, key=busy.get)
    stages["note"] = ("busy time per stage of one call (the stages overlap across chunks); host_round = the op's host threads "
                      "rounding float32 to bf16 into pinned staging, h2d / d2h = copy queues, kernel = device cast + attention")
    del ctx
    for pp in ptrs:
        L.grl_host_free(pp)
    info = stages
    return dt, h2d, d2h, par, info


# ------------------------------------------------------------------------------------- decode legs
def kv_layout(cabi, kp, vp, table, seq_lens, B, Hkv, D, P, max_pages, n_pages):
    lay = cabi.KVLayout()
    lay.k_pages, lay.v_pages, lay.cache_dtype = kp, vp, cabi.BF16
    lay.block_table, lay.seq_lens = table, seq_lens
    lay.batch, lay.num_kv_heads, lay.head_dim, lay.page_tokens, lay.max_pages, lay.num_pages = B, Hkv, D, P, max_pages, n_pages
    return lay


def bench_decode(dev, cabi, dist, repeats=3, use_graph=True, quant=False, simt=False):
    """cfg3: 256 decode steps (RoPE + append + split-KV attention + merge), graph-replayed.  quant: the same run over
    the FP8 / INT4 cache (the prefix is appended through the quantiser, so every stored byte is a real code).  simt: the
    generic decode_split_kernel (+ lse_merge_kernel) instead of the tensor-core kernel, for shapes that one does not take."""
    from oracle import c_oracle
    c = CFG3
    B, Hq, Hkv, D, T0, steps, P = c["B"], c["Hq"], c["Hkv"], c["D"], c["T0"], c["steps"], c["page"]
    L = dev.L
    rng = np.random.default_rng(c["seed"] + dist.rank)
    max_tokens = T0 + steps
    max_pages = (max_tokens + P - 1) // P
    n_pages = max_pages * B
    page_elems = Hkv * P * D
    table = dev.upload(np.arange(n_pages, dtype=np.int32).reshape(B, max_pages))
    lens0 = np.full(B, T0, np.int32)
    scales = None
    if quant:
        kp, vp = dev.malloc(n_pages * page_elems), dev.malloc(n_pages * page_elems // 2)
        scales = dev.malloc(n_pages * page_elems // 32 * 2)
        seq_lens = dev.upload(np.zeros(B, np.int32))
        lay0 = kv_layout(cabi, kp, vp, table, seq_lens, B, Hkv, D, P, max_pages, n_pages)
        lay0.cache_dtype, lay0.scales = cabi.FP8_INT4, scales
        blk = 512
        for _ in range(T0 // blk):          # the prefix goes in through the quantiser
            kd = dev.upload(rng.standard_normal((B, blk, Hkv, D), dtype=np.float32))
            vd = dev.upload(rng.standard_normal((B, blk, Hkv, D), dtype=np.float32))
            ap0 = cabi.AppendParams()
            ap0.kv, ap0.k_new, ap0.v_new, ap0.n_new, ap0.update_lens = lay0, kd, vd, blk, 1
            cabi.check(L.grl_kv_append(dev.h, C.byref(ap0)))
            dev.sync()
            dev.free(kd); dev.free(vd)
    else:
        kp, vp = dev.malloc(n_pages * page_elems * 2), dev.malloc(n_pages * page_elems * 2)
        for dst in (kp, vp):      # the prefix is "already rotated" keys: iid N(0,1) bf16
            fill_random_bf16(dev, cabi, dst, n_pages * page_elems, rng)
        seq_lens = dev.upload(lens0)
    q_host = rng.standard_normal((steps, B, 1, Hq, D), dtype=np.float32)
    k_host = rng.standard_normal((steps, B, 1, Hkv, D), dtype=np.float32)
    qs, ks = dev.upload(q_host), dev.upload(k_host)
    vs = dev.upload(rng.standard_normal((steps, B, 1, Hkv, D), dtype=np.float32))
    q_rot = dev.malloc(B * Hq * D * 4)
    out = dev.malloc(steps * B * Hq * D * 4)
    lay = kv_layout(cabi, kp, vp, table, seq_lens, B, Hkv, D, P, max_pages, n_pages)
    if quant:
        lay.cache_dtype, lay.scales = cabi.FP8_INT4, scales
    dp = cabi.DecodeParams()
    dp.kv, dp.num_q_heads, dp.max_seq_len = lay, Hq, max_tokens
    dp.force_simt = int(simt)
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

    dev.sync()
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
    # parity of the last step of sequence 0: its cache read back through grl_kv_gather (bf16 values, exact in
    # float32), the rotated q of that step, and the checker's decode over them; the appended key of that step
    # against the rotation of the new key at its position
    sb = 0
    T = T0 + steps
    gk, gv = dev.malloc(T * Hkv * D * 4), dev.malloc(T * Hkv * D * 4)
    cabi.check(L.grl_kv_gather(dev.h, C.byref(lay), sb, T, gk, gv))
    dev.sync()
    Kc, Vc = dev.download(gk, (1, T, Hkv, D), np.float32), dev.download(gv, (1, T, Hkv, D), np.float32)
    q_last = dev.download(q_rot, (B, 1, Hq, D), np.float32)[sb:sb + 1]
    o_last = dev.download(C.c_void_p(out.value + (steps - 1) * B * Hq * D * 4), (B, 1, Hq, D), np.float32)[sb:sb + 1]
    par = parity("decode cfg3" + (" (quantised cache)" if quant else ""), np.abs(o_last - c_oracle.gqa_decode(q_last, Kc, Vc)).max(),
                 TOL_DECODE, sample=f"sequence {sb}, step {steps}: all 32 query heads over its {T} cached tokens"
                                    + (" as the cache dequantises them" if quant else ""))
    k_rot = c_oracle.rope_interleaved(np.concatenate([np.zeros((Hkv, T - 1, D), np.float32),
                                                      k_host[steps - 1, sb, 0][:, None, :]], axis=1), c["theta"])[:, -1]
    if quant:     # the stored key is the quantiser's image of RoPE(k): compare with the checker's quantiser
        kq_want = c_oracle.kv_dequantize(*c_oracle.kv_quantize(k_rot[None], k_rot[None]))[0][0]
        par["appended_key_codes_differing"] = float(np.mean(Kc[0, T - 1] != kq_want))
        if par["appended_key_codes_differing"] > 0.02:
            raise ParityError("decode cfg3 (quantised): appended key differs from quantise(RoPE(k))")
    else:
        par["appended_key_max_abs"] = float(np.abs(Kc[0, T - 1] - round_bf16(k_rot)).max())
        if par["appended_key_max_abs"] > 2e-2:
            raise ParityError(f"decode cfg3: appended key differs from RoPE(k) by {par['appended_key_max_abs']}")
    q_want = c_oracle.rope_interleaved(np.concatenate([np.zeros((Hq, T - 1, D), np.float32),
                                                       q_host[steps - 1, sb, 0][:, None, :]], axis=1), c["theta"])[:, -1]
    par["rotated_q_max_abs"] = float(np.abs(q_last[0, 0] - q_want).max())
    if par["rotated_q_max_abs"] > 1e-4:
        raise ParityError(f"decode cfg3: rotated q differs from RoPE(q) by {par['rotated_q_max_abs']}")
    dev.free(gk); dev.free(gv)
    best = None
    e0, e1 = dev.event(), dev.event()
    for _ in range(repeats):
        reset()
        dev.sync()
        dist.barrier()
        dev.record(e0)
        run()
        dev.record(e1)
        dev.sync()
        ms = dist.max(dev.elapsed_ms(e0, e1))
        best = ms if best is None else min(best, ms)
    if use_graph:
        L.grl_graph_destroy(g)
    for x in (kp, vp, table, seq_lens, qs, ks, vs, q_rot, out, ws) + ((scales,) if quant else ()):
        dev.free(x)
    return best, launches_per_run, ns.value, par


def bench_evict(dev, cabi, repeats=3):
    """Eviction on a cfg3-sized cache (B32, Hkv8, D128, 4096 tokens, bf16): H2O selection of a quarter of every
    sequence, then compaction.  Returns (select_us, compact_us, bytes moved by one compaction)."""
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
    lay = kv_layout(cabi, kp, vp, table, seq_lens, B, Hkv, D, P, max_pages, n_pages)
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


def bench_linear(dev, cabi, pk, M=4096, K=4096, N=4096, steps=20):
    """grl_linear on device-resident bf16 operands (the projection on either side of attention): parity of a sampled
    block against numpy on the bf16-rounded operands, then CUDA-event time of `steps` launches."""
    L = dev.L
    rng = np.random.default_rng(21)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = (rng.standard_normal((N, K), dtype=np.float32) / np.sqrt(K)).astype(np.float32)
    bias = rng.standard_normal(N, dtype=np.float32)
    xf, wf, bd = dev.upload(x), dev.upload(w), dev.upload(bias)
    xb, wb, y = dev.malloc(M * K * 2), dev.malloc(N * K * 2), dev.malloc(M * N * 4)
    cabi.check(L.grl_cast(dev.h, xf, cabi.F32, xb, cabi.BF16, M * K))
    cabi.check(L.grl_cast(dev.h, wf, cabi.F32, wb, cabi.BF16, N * K))
    call = lambda: cabi.check(L.grl_linear(dev.h, xb, wb, bd, y, M, K, N, cabi.BF16))
    call()
    dev.sync()
    got = dev.download(y, (M, N), np.float32)
    rows, cols = slice(M - 200, M), slice(N - 136, N)
    want = round_bf16(x[rows]).astype(np.float64) @ round_bf16(w[cols]).astype(np.float64).T + bias[cols]
    par = parity("linear", np.abs(got[rows, cols] - want).max(), 2e-5 * K, sample="last 200 x 136 block against numpy on the bf16-rounded operands")
    for _ in range(3):
        call()
    e0, e1 = dev.event(), dev.event()
    dev.sync()
    dev.record(e0)
    for _ in range(steps):
        call()
    dev.record(e1)
    dev.sync()
    ms = dev.elapsed_ms(e0, e1) / steps
    tf = 2.0 * M * K * N / (ms * 1e-3) / 1e12
    for p_ in (xf, wf, bd, xb, wb, y):
        dev.free(p_)
    return {"workload": f"grl_linear bf16 ({M} x {K}) x ({N} x {K})^T + bias -> fp32, device-resident, L2-warm operands", "ms_per_call": ms,
            "value": tf, "unit": "TFLOP/s", "parity": par,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["tf"], "unit": "TFLOP/s", "frac": tf / pk["tf"],
                         "peak_source": pk["src"] + " (burst)", "kernel": "linear_sm100_kernel"}}


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
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        grilly_core.decode_step(ctx, kv, q, k1, k1, rope_theta=c["theta"], out=o)
    dt = dist.max((time.perf_counter() - t0) / steps)
    assert np.isfinite(o).all()
    grilly_core.destroy_kv_cache(ctx, kv)
    nb = (q.nbytes + 2 * k1.nbytes, o.nbytes)
    del q, k1, o
    for pp in (qp, kp, op):
        L.grl_host_free(pp)
    return dt, nb[0], nb[1]


LONG_MODES = ("decode", "ll", "merge", "nccl")
LONG_MODE_TEXT = {
    "decode": "exchange over NVLink peer stores and LSE merge inside the decode kernel (one launch per step)",
    "ll": "exchange over NVLink peer stores ({value, step} pairs, no flag) fused with the LSE merge",
    "merge": "exchange over NVLink peer stores (fence + flag) fused with the LSE merge",
    "nccl": "NCCL all-gather (grl_group_allgather_merge) + LSE merge",
}


def long_decode_parity(dev, cabi, dist, ops_factory):
    """Every form of the exchange on a small seeded case (T = 1000 per rank) against the checker on the
    bf16-rounded cache, before anything is timed.  Returns {mode: max-abs}."""
    from grilly_next.parallel import ShardedDecoder, shard_range
    from oracle import c_oracle
    c = CFG4
    B, Hq, Hkv, D, P = 1, c["Hq"], c["Hkv"], c["D"], 64
    world, rank = dist.world, dist.rank
    T = 1000 * world
    rng = np.random.default_rng(c["seed"])                    # the same data on every rank
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    lo, hi = shard_range(T, world, rank)
    Tg = hi - lo
    n_pages = (Tg + P - 1) // P
    L = dev.L
    kp, vp = dev.malloc(n_pages * Hkv * P * D * 2), dev.malloc(n_pages * Hkv * P * D * 2)
    table = dev.upload(np.arange(n_pages, dtype=np.int32).reshape(B, n_pages))
    seq_lens = dev.upload(np.zeros(B, np.int32))
    lay = kv_layout(cabi, kp, vp, table, seq_lens, B, Hkv, D, P, n_pages, n_pages)
    kd, vd = dev.upload(k[:, lo:hi]), dev.upload(v[:, lo:hi])
    ap = cabi.AppendParams()
    ap.kv, ap.k_new, ap.v_new, ap.n_new, ap.update_lens = lay, kd, vd, Tg, 1
    cabi.check(L.grl_kv_append(dev.h, C.byref(ap)))
    dev.sync()
    kb, vb = round_bf16(k), round_bf16(v)
    res = {}
    for mode in (LONG_MODES if world > 1 else ("decode",)):
        ops = ops_factory(lay, Tg, mode)
        dec = ShardedDecoder(dist, ops)
        worst = 0.0
        for _ in range(3):                                     # both inbox parities
            q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
            qd = dev.upload(q)
            out_ptr = dec.step(qd)
            dev.sync()
            out = dev.download(out_ptr, (B, 1, Hq, D), np.float32)
            dev.free(qd)
            worst = max(worst, float(np.abs(out - c_oracle.gqa_decode(q, kb, vb)).max()))
        ops.close()
        res[mode if world > 1 else "single_gpu"] = worst
    worst = max(res.values())
    out = parity("decode_long cfg4", worst, TOL_DECODE,
                 sample=f"T = {T} tokens over {world} GPU(s), 3 steps per exchange form, rank {rank}'s output against the checker on the bf16-rounded cache")
    out.update(res)
    for x in (kp, vp, table, seq_lens, kd, vd):
        dev.free(x)
    return out


def bench_long_decode(dev, cabi, dist, steps=50, repeats=3):
    """cfg4: B=1, Hq32/Hkv8, D128, KV length 131072 split in contiguous shards over the ranks; per step
    every rank decodes its shard to one partial, the partials cross NVLink and every rank merges."""
    from grilly_next.parallel import CudaShardOps, ShardedDecoder, shard_range
    c = CFG4
    B, Hq, Hkv, D, T, P = 1, c["Hq"], c["Hkv"], c["D"], c["T"], 64
    world, rank = dist.world, dist.rank
    L = dev.L

    def make_ops(lay, Tg, mode):
        ops = CudaShardOps(cabi, dev, lay, Hq, Tg)
        if world > 1:
            if mode == "nccl":
                ops.setup_nccl(dist)
            elif not ops.setup_p2p(dist, one_launch=(mode == "decode"), low_latency=(mode != "merge")):
                raise RuntimeError("peer inboxes could not be mapped (no peer access between the GPUs?)")
        return ops

    par = long_decode_parity(dev, cabi, dist, make_ops)
    lo, hi = shard_range(T, world, rank)
    Tg = hi - lo
    n_pages = (Tg + P - 1) // P
    page_elems = Hkv * P * D
    shard_bytes = 2 * n_pages * page_elems * 2
    nbuf = max(1, -(-(512 << 20) // shard_bytes))        # rotate buffers so that a shard never sits in L2
    rng = np.random.default_rng(c["seed"] + rank)
    pools = []
    for _ in range(nbuf):
        pair = [dev.malloc(n_pages * page_elems * 2) for _ in range(2)]
        for dst in pair:
            fill_random_bf16(dev, cabi, dst, n_pages * page_elems, rng)
        pools.append(pair)
    table = dev.upload(np.arange(n_pages, dtype=np.int32).reshape(B, n_pages))
    lens = dev.upload(np.full(B, Tg, np.int32))
    q = dev.upload(np.random.default_rng(c["seed"]).standard_normal((B, 1, Hq, D), dtype=np.float32))   # same q on every rank
    layouts = [kv_layout(cabi, pools[i][0], pools[i][1], table, lens, B, Hkv, D, P, n_pages, n_pages) for i in range(nbuf)]
    timings, n_splits, graphed = {}, 0, True
    for mode in (LONG_MODES if world > 1 else ("decode",)):
        ops = make_ops(layouts[0], Tg, mode)
        dec = ShardedDecoder(dist, ops)
        n_splits = ops.p.n_splits
        for i in range(5):
            ops.set_layout(layouts[i % nbuf]); dec.step(q)
        dev.sync()

        def run_steps():
            for i in range(steps):
                ops.set_layout(layouts[i % nbuf]); dec.step(q)

        # a step is one to three small launches: replay `steps` of them from one CUDA graph so that launch
        # latency does not hide the kernels
        g = C.c_void_p()
        dist.barrier()
        cabi.check(L.grl_graph_begin(dev.h))
        run_steps()
        cabi.check(L.grl_graph_end(dev.h, C.byref(g)))
        cabi.check(L.grl_graph_launch(dev.h, g))
        dev.sync()
        best = None
        e0, e1 = dev.event(), dev.event()
        for _ in range(repeats):
            dev.sync()
            dist.barrier()
            dev.record(e0)
            cabi.check(L.grl_graph_launch(dev.h, g))
            dev.record(e1)
            dev.sync()
            ms = dist.max(dev.elapsed_ms(e0, e1))
            best = ms if best is None else min(best, ms)
        L.grl_graph_destroy(g)
        out = dev.download(ops.out, (B, 1, Hq, D), np.float32)
        assert np.isfinite(out).all()
        timings[mode] = best / steps
        dist.barrier()
        ops.close()
    for pair in pools:
        for x in pair:
            dev.free(x)
    for x in (table, lens, q):
        dev.free(x)
    launches = {"decode": 1, "ll": 3, "merge": 3, "nccl": 2}
    return timings, launches, n_splits, nbuf, graphed, par


# ------------------------------------------------------------------------------------- CPU baselines
def cpu_baseline():
    """The checker's C/OpenMP restatement of the reference's CPU attention, RoPE included, on a bounded sample."""
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())
    from oracle import attention_oracle as orc
    from oracle import c_oracle
    c = CFG2
    heads = 32
    rng = np.random.default_rng(c["seed"])
    Q, K, V = (rng.standard_normal((1, heads, c["S"], c["D"]), dtype=np.float32) for _ in range(3))
    c_oracle.attention(Q[:, :2], K[:, :2], V[:, :2], causal=True)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 10.0 and reps < 8:
        c_oracle.attention(c_oracle.rope_interleaved(Q, c["theta"]), c_oracle.rope_interleaved(K, c["theta"]), V, causal=True)
        reps += 1
    dt = time.perf_counter() - t0
    fl = causal_flops(c["D"], heads, [c["S"]]) * reps
    res = {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": c_oracle.num_threads(), "kind": "port",
           "sample": f"{reps} passes over {heads} of 128 (batch, head) slices of cfg2 (RoPE + causal attention), C/OpenMP oracle"}
    # the numpy form the reference's tests define (tests/test_attention.py:20-35), restated in oracle/attention_oracle.py
    nh = 2
    pos = np.arange(c["S"])
    mask = orc.causal_length_mask(1, nh, c["S"], None, True)
    t0 = time.perf_counter()
    orc.attention_4d(orc.rope_interleaved(Q[:, :nh], pos, c["theta"]), orc.rope_interleaved(K[:, :nh], pos, c["theta"]), V[:, :nh], mask=mask)
    dt = time.perf_counter() - t0
    res["numpy"] = {"value": causal_flops(c["D"], nh, [c["S"]]) / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(),
                    "sample": f"one pass over {nh} of 128 (batch, head) slices, numpy restatement of the reference's _ref_attention_4d "
                              "(dense (S,S) scores with a tril mask, so it also computes the masked half)"}
    return res


def cpu_baseline_decode():
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())
    from oracle import c_oracle
    c = CFG3
    Bs, T = 4, c["T0"]
    rng = np.random.default_rng(c["seed"])
    k = rng.standard_normal((Bs, T, c["Hkv"], c["D"]), dtype=np.float32)
    v = rng.standard_normal((Bs, T, c["Hkv"], c["D"]), dtype=np.float32)
    q = rng.standard_normal((Bs, 1, c["Hq"], c["D"]), dtype=np.float32)
    c_oracle.gqa_decode(q, k, v)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 4.0 and reps < 200:
        c_oracle.gqa_decode(q, k, v)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": Bs / dt, "unit": "tokens/s", "cores": c_oracle.num_threads(), "kind": "port",
            "sample": f"{reps} decode steps of {Bs} of the 32 sequences at cache length {T} (fp32 cache, attention only: no RoPE, no append), "
                      "C/OpenMP oracle_gqa_decode_f32"}


def cpu_baseline_long():
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())
    from oracle import c_oracle
    c = CFG4
    Ts = c["T"] // 4
    rng = np.random.default_rng(c["seed"])
    k = rng.standard_normal((1, Ts, c["Hkv"], c["D"]), dtype=np.float32)
    v = rng.standard_normal((1, Ts, c["Hkv"], c["D"]), dtype=np.float32)
    q = rng.standard_normal((1, 1, c["Hq"], c["D"]), dtype=np.float32)
    c_oracle.gqa_decode(q, k, v)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 4.0 and reps < 200:
        c_oracle.gqa_decode(q, k, v)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": 1.0 / (dt * 4), "unit": "tokens/s", "cores": c_oracle.num_threads(), "kind": "port",
            "sample": f"{reps} decode steps over a quarter of the cache ({Ts} of {c['T']} tokens, fp32), time scaled by 4 (the step is linear "
                      "in the cache length), C/OpenMP oracle_gqa_decode_f32"}


# ------------------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--legs", default=",".join(ALL_LEGS), help="comma-separated subset of: " + ", ".join(ALL_LEGS))
    ap.add_argument("--no-graph", action="store_true", help="cfg3 as plain launches instead of graph replay (for a profiler's launch list)")
    ap.add_argument("--decode-repeats", type=int, default=3)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    legs = set(x for x in args.legs.split(",") if x)
    unknown = legs - set(ALL_LEGS)
    if unknown:
        ap.error(f"unknown legs {sorted(unknown)}")

    if args.impl == "reference":
        return run_reference(args)

    dist = Dist()
    rank, world, local_rank = dist.rank, dist.world, dist.local_rank
    os.environ["GRILLY_GPU_INDEX"] = str(local_rank)     # the op layer's device selector
    from grilly_next import cabi
    dev = cabi.Device(local_rank)          # raises if the CUDA library or the GPU is missing: no fallback
    L = dev.L
    pk = peaks()
    line = {"metric": "prefill_attn_tflops", "value": None, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic"}
    try:
        if "prefill" in legs:
            sampler = ClockSampler(local_rank)
            sampler.start()
            r = bench_prefill(dev, cabi, args, dist, pk, sampler)
            sampler.stop()
            line.update({
                "value": r["tflops_gpu"] * world, "ms_per_step": r["ms"] / args.steps,
                "config": {"workload": "cfg2: FlashAttention-2+RoPE causal prefill, B4 H32 S2048 D128, bf16 in / fp32 out, per GPU",
                           "flops_per_step_per_gpu": r["flops"], "l2": "inputs larger than L2 (320 MiB per step)",
                           "parallelism": f"replica per GPU x{world}, no collective",
                           "rope": "rotation of Q and K inside the attention kernel (device-resident bf16 inputs, unrotated)"},
                "clocks": r["clocks"], "gpu_launches": int(r["launches"]),
                "roofline": prefill_roofline(r["tflops_gpu"], r["ms"], pk, PREFILL_TRAFFIC_BYTES),
                "parity": r["parity"], "sustained": r["sustained"]})
            if "strong" in r:
                line["strong_scaling"] = {"cfg2": r["strong"]}
        if "cfg1" in legs:
            line["cfg1"], qkv1 = bench_cfg1(dev, cabi, args, dist)
            if "e2e" in legs:
                line["cfg1"]["e2e"] = bench_cfg1_e2e(qkv1, dist)
        if "cfg5" in legs:
            r5 = bench_cfg5(dev, cabi, args, dist, pk)
            if "strong" in r5:
                line.setdefault("strong_scaling", {})["cfg5"] = r5.pop("strong")
            line["cfg5"] = r5
        if "decode" in legs:
            dms, dl, nsplit, dpar = bench_decode(dev, cabi, dist, args.decode_repeats, not args.no_graph)
            c = CFG3
            toks = c["B"] * c["steps"] / (dms * 1e-3)
            gbs = decode_bytes(c) / (dms * 1e-3) / 1e9
            line["decode"] = {"metric": "decode_tokens_per_s", "value": toks * world, "unit": "tokens/s",
                              "ms_per_step": dms / c["steps"],
                              "workload": "cfg3: GQA decode B32 Hq32/Hkv8 D128 KV 4096->4352, 256 steps, bf16 paged cache, "
                                          + ("CUDA-graph replay" if not args.no_graph else "plain launches") + ", per GPU",
                              "gpu_launches": int(dl), "n_splits": nsplit, "parity": dpar,
                              "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s", "frac": gbs / pk["hbm"],
                                           "traffic": DECODE_TRAFFIC_BYTES, "peak_source": pk["src"], "frac_of_nominal_8000": gbs / 8000.0,
                                           "note": "achieved = algorithmic bytes of the 256-step run / its time (append + decode + merge per step)",
                                           "kernel": "decode_mma_kernel"}}
        if "decode" in legs and world == 1:
            qms, ql, qsplit, qpar = bench_decode(dev, cabi, dist, args.decode_repeats, not args.no_graph, quant=True)
            c = CFG3
            per_pos = c["B"] * c["Hkv"] * (c["D"] + c["D"] // 2 + c["D"] // 32 * 2)      # key bytes + value nibbles + scales
            qbytes = sum(per_pos * (c["T0"] + t + 1) for t in range(c["steps"])) + c["steps"] * c["B"] * c["Hq"] * c["D"] * 8
            qgbs = qbytes / (qms * 1e-3) / 1e9
            line["decode_q"] = {"metric": "decode_tokens_per_s", "value": c["B"] * c["steps"] / (qms * 1e-3), "unit": "tokens/s",
                                "ms_per_step": qms / c["steps"],
                                "workload": "cfg3 geometry over the quantised cache (FP8-E4M3 keys, INT4 values, float16 scale per 32: "
                                            "200 B per cached (token, kv head) against 512 B in bf16), the tensor-core decode kernel dequantising in registers",
                                "gpu_launches": int(ql), "n_splits": qsplit, "parity": qpar,
                                "roofline": {"bound": "hbm", "achieved": qgbs, "peak": pk["hbm"], "unit": "GB/s", "frac": qgbs / pk["hbm"],
                                             "peak_source": pk["src"], "kernel": "decode_mma_kernel<quantised>",
                                             "note": "achieved = bytes of the quantised cache actually read per step / time (append + decode "
                                                     "per step); the kernel is bound by its dequantising arithmetic and its dependent chains, "
                                                     "not by HBM"}}
        if "decode" in legs and world == 1:
            sms_, sl_, ssplit_, spar_ = bench_decode(dev, cabi, dist, 1, not args.no_graph, simt=True)
            c = CFG3
            sgbs = decode_bytes(c) / (sms_ * 1e-3) / 1e9
            line["decode_simt"] = {"metric": "decode_tokens_per_s", "value": c["B"] * c["steps"] / (sms_ * 1e-3), "unit": "tokens/s",
                                   "ms_per_step": sms_ / c["steps"], "gpu_launches": int(sl_), "n_splits": ssplit_, "parity": spar_,
                                   "workload": "cfg3 through the generic kernel (decode_split_kernel + lse_merge_kernel): the path of "
                                               "every geometry the tensor-core kernel does not take (head_dim 32 / 64, other page sizes, fp32 cache)",
                                   "roofline": {"bound": "hbm", "achieved": sgbs, "peak": pk["hbm"], "unit": "GB/s", "frac": sgbs / pk["hbm"],
                                                "peak_source": pk["src"], "kernel": "decode_split_kernel<bf16,128,4>"}}
        if "linear" in legs and world == 1:
            line["linear"] = bench_linear(dev, cabi, pk)
        if "evict" in legs and world == 1:
            sel_us, cmp_us, moved = bench_evict(dev, cabi)
            gbs = moved / (cmp_us * 1e-6) / 1e9
            line["evict"] = {"workload": "cfg3-sized cache (B32 Hkv8 D128 4096 tokens bf16): H2O selection of a quarter of every sequence, "
                                         "then compaction", "select_us": sel_us, "compact_us": cmp_us,
                             "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s", "frac": gbs / pk["hbm"],
                                          "peak_source": pk["src"], "note": "surviving K/V rows read once and written once; rows that stay in place are skipped, so this is an upper bound on the traffic"}}
        if "long" in legs:
            timings, launches, lsplit, nbuf, graphed, lpar = bench_long_decode(dev, cabi, dist)
            kv_bytes = 2 * CFG4["Hkv"] * CFG4["D"] * 2 * CFG4["T"]
            best = min(timings, key=timings.get)    # every form passed its parity check above; the headline is the fastest
            lms = timings[best]
            gbs = kv_bytes / (lms * 1e-3) / 1e9
            line["decode_long"] = {
                "metric": "decode_long_tokens_per_s", "value": 1.0 / (lms * 1e-3), "unit": "tokens/s", "ms_per_step": lms, "scaling": "strong",
                "workload": f"cfg4: GQA decode B1 Hq32/Hkv8 D128 KV 131072 bf16 split over {world} GPU(s); "
                            + (f"{lsplit} splits merged inside the decode kernel" if world == 1 else "per-GPU partial (16,640 B/rank) + " + LONG_MODE_TEXT[best])
                            + f"; {nbuf} rotating KV buffers (L2); CUDA-graph replay",
                "gpu_launches_per_step": launches[best], "n_splits": lsplit, "parity": lpar, "exchange": best,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"] * world, "unit": "GB/s",
                             "frac": gbs / (pk["hbm"] * world), "peak_source": pk["src"] + f" x{world}"}}
            if world > 1:
                line["decode_long"]["ms_per_step_by_exchange"] = {m: {"ms_per_step": t, "launches_per_step": launches[m], "how": LONG_MODE_TEXT[m]}
                                                                  for m, t in timings.items()}
        if "e2e" in legs and "prefill" in legs:
            fl = causal_flops(CFG2["D"], CFG2["B"] * CFG2["H"], [CFG2["S"]])
            dt, h2d, d2h, epar, info = bench_prefill_e2e(args, L, min(args.steps, 5), dist)
            line["e2e"] = {"value": fl / dt / 1e12 * world, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "ms_per_step": dt * 1e3, "parity": epar,
                           "api": "grilly_core.flash_attention2(dtype='bf16', out=pinned), pinned fp32 host arrays in and out; "
                                  "h2d bytes are what crosses the link (the op's host threads round a share of every chunk to bf16 "
                                  "first -- pipeline.host_cast_pct; 402,653,184 B of fp32 are read from the host arrays)"}
            if info:
                line["e2e"]["pipeline"] = info
        if "e2e" in legs and "decode" in legs:
            ddt, dh2d, dd2h = bench_decode_e2e(dist)
            line["decode"]["e2e"] = {"value": CFG3["B"] / ddt * world, "unit": "tokens/s", "h2d_bytes_per_step": dh2d,
                                     "d2h_bytes_per_step": dd2h, "ms_per_step": ddt * 1e3, "api": "grilly_core.decode_step(out=pinned), pinned fp32 host arrays in and out"}
        if "cpu" in legs and rank == 0 and world == 1:
            if "prefill" in legs:
                line["cpu_baseline"] = cpu_baseline()
            if "decode" in legs:
                line["decode"]["cpu_baseline"] = cpu_baseline_decode()
            if "long" in legs:
                line["decode_long"]["cpu_baseline"] = cpu_baseline_long()
    except ParityError as e:
        sys.stderr.write(f"PARITY FAILURE on rank {rank}: {e}\n")
        sys.stderr.flush()
        os._exit(3)

    dev.close()
    dist.close()
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
