"""Seeded inputs shared by the golden generator, the CPU tests and the GPU parity tests."""
import numpy as np

# name -> shape/config.  "seed" follows 1000 + config index for the benchmark configurations.
PREFILL_CASES = {
    # configuration 1 of the benchmark: fp32, causal
    "cfg1": dict(B=1, H=4, S=256, D=64, causal=True, seed=1001),
    # configuration 2 (sampled heads): causal + RoPE theta 10000
    "cfg2": dict(B=4, H=32, S=2048, D=128, causal=True, rope=10000.0, seed=1002, sample=2),
    # reduced forms that the CPU finishes quickly
    "cfg2_small": dict(B=2, H=3, S=384, D=128, causal=True, rope=10000.0, seed=2002),
    "noncausal_d128": dict(B=1, H=2, S=256, D=128, causal=False, seed=2003),
    "ragged_d128": dict(B=3, H=2, S=320, D=128, causal=True, rope=10000.0, seed=2004,
                        lens=[320, 129, 77]),
    "odd_s_d64": dict(B=2, H=2, S=197, D=64, causal=True, seed=2005),
    "tiny_s8_d64": dict(B=1, H=1, S=8, D=64, causal=False, seed=2006),
    "s1_d64": dict(B=1, H=2, S=1, D=64, causal=True, seed=2007),
    "d32": dict(B=1, H=2, S=100, D=32, causal=False, seed=2008),
}

DECODE_CASES = {
    # shapes of the reference's known-answer tests (tests/test_inference_ops.py:352-430)
    # (legacy=True: drawn as those tests draw them, np.random.seed(42) then randn * 0.1)
    "kat_b1": dict(B=1, T=16, Hq=12, Hkv=4, D=64, seed=42, scale=0.1, legacy=True),
    "kat_b3": dict(B=3, T=16, Hq=12, Hkv=4, D=64, seed=42, scale=0.1, legacy=True),
    "kat_group": dict(B=1, T=8, Hq=6, Hkv=2, D=32, seed=42, scale=0.1, legacy=True),
    "kat_len1": dict(B=1, T=1, Hq=8, Hkv=4, D=32, seed=42, scale=0.1, legacy=True),
    "kat_len64": dict(B=1, T=64, Hq=8, Hkv=4, D=32, seed=42, scale=0.1, legacy=True),
    # unit-normal cases at the benchmark's head geometry
    "gqa_t300": dict(B=2, T=300, Hq=32, Hkv=8, D=128, seed=3001, scale=1.0),
    "gqa_t4097": dict(B=2, T=4097, Hq=32, Hkv=8, D=128, seed=3002, scale=1.0),
    "mha_t130": dict(B=2, T=130, Hq=4, Hkv=4, D=64, seed=3003, scale=1.0),
}


def prefill_inputs(c):
    rng = np.random.default_rng(c["seed"])
    shape = (c["B"], c["H"], c["S"], c["D"])
    Q = rng.standard_normal(shape, dtype=np.float32)
    K = rng.standard_normal(shape, dtype=np.float32)
    V = rng.standard_normal(shape, dtype=np.float32)
    return Q, K, V


def seq_lens(c):
    return None if "lens" not in c else np.asarray(c["lens"], dtype=np.int32)


def sampled_heads(c):
    """(b,h) pairs that hold golden vectors: all of them, or a seeded sample for big cases."""
    allp = [(b, h) for b in range(c["B"]) for h in range(c["H"])]
    if "sample" not in c:
        return allp
    rng = np.random.default_rng(c["seed"] + 7)
    idx = rng.choice(len(allp), size=c["sample"], replace=False)
    return [allp[i] for i in sorted(idx)]


def random_dense_mask(c):
    rng = np.random.default_rng(c["seed"] + 11)
    m = (rng.random((c["B"], c["H"], c["S"], c["S"])) > 0.3).astype(np.float32)
    for i in range(c["S"]):
        m[:, :, i, i] = 1.0  # keep at least one key per row
    return m


def decode_inputs(c):
    """query (B,1,Hq,D), k_cache/v_cache (B,T,Hkv,D) float32."""
    s = np.float32(c["scale"])
    if c.get("legacy"):
        rs = np.random.RandomState(c["seed"])
        q = rs.randn(c["B"], 1, c["Hq"], c["D"]).astype(np.float32) * s
        k = rs.randn(c["B"], c["T"], c["Hkv"], c["D"]).astype(np.float32) * s
        v = rs.randn(c["B"], c["T"], c["Hkv"], c["D"]).astype(np.float32) * s
        return q, k, v
    rng = np.random.default_rng(c["seed"])
    q = rng.standard_normal((c["B"], 1, c["Hq"], c["D"]), dtype=np.float32) * s
    k = rng.standard_normal((c["B"], c["T"], c["Hkv"], c["D"]), dtype=np.float32) * s
    v = rng.standard_normal((c["B"], c["T"], c["Hkv"], c["D"]), dtype=np.float32) * s
    return q, k, v
