"""GPU parity of the prefill path against the oracle and the golden vectors.

Tolerances (max-abs on unit-normal inputs): 1e-4 for the fp32 path, 2e-2 for the bf16
tensor-core path measured against the fp32 oracle on the UNROUNDED fp32 inputs.
"""
import os

import numpy as np
import pytest

import cases
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-4
TOL_BF16 = 2e-2
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_golden.npz"))


@pytest.fixture(scope="module")
def dev():
    from grilly_next import cabi
    d = cabi.Device(0)
    yield d
    d.close()


@pytest.fixture(scope="module")
def gpu():
    from grilly_next import Compute
    g = Compute()
    yield g
    g.cleanup()


def _check_case(out, name, c, tol):
    lens = cases.seq_lens(c)
    for (b, h) in cases.sampled_heads(c):
        want = GOLD[f"prefill/{name}/{b}_{h}"]
        err = np.abs(out[b, h] - want).max()
        assert err <= tol, f"{name} head ({b},{h}): max-abs {err:.3e} > {tol}"
    if lens is not None:
        for b in range(c["B"]):
            assert np.all(out[b, :, int(lens[b]):] == 0), "padded query rows must be zero"


@pytest.mark.parametrize("name", [n for n in cases.PREFILL_CASES if n != "cfg2"])
def test_fp32_kernel_matches_golden(dev, name):
    from grilly_next import cabi
    from gpu_helpers import flash_cabi
    c = cases.PREFILL_CASES[name]
    Q, K, V = cases.prefill_inputs(c)
    out = flash_cabi(dev, Q, K, V, causal=c["causal"], seq_lens=cases.seq_lens(c),
                     rope_mode=cabi.ROPE_INTERLEAVED if c.get("rope") else cabi.ROPE_NONE,
                     rope_theta=c.get("rope", 10000.0), kernel=cabi.KERNEL_SIMT_F32)
    assert np.all(np.isfinite(out))
    _check_case(out, name, c, TOL_F32)


@pytest.mark.parametrize("name", ["cfg1", "cfg2_small", "ragged_d128", "tiny_s8_d64", "s1_d64"])
def test_python_op_matches_golden(gpu, name):
    # the numpy drop-in path: Compute().flash_attention2 (host arrays in, host array out)
    c = cases.PREFILL_CASES[name]
    Q, K, V = cases.prefill_inputs(c)
    kw = dict(causal=c["causal"])
    if c.get("rope"):
        kw.update(rope_theta=c["rope"])
    if "lens" in c:
        kw.update(seq_lens=np.asarray(c["lens"], np.int32))
    out = gpu.flash_attention2(Q, K, V, **kw)
    assert out.shape == Q.shape and out.dtype == np.float32
    _check_case(out, name, c, TOL_F32)


def test_reference_mask_argument(gpu):
    # (B,H,S,S) mask as the reference's tests pass it (tril of ones), and an arbitrary dense mask
    c = cases.PREFILL_CASES["cfg1"]
    Q, K, V = cases.prefill_inputs(c)
    tril = np.tril(np.ones((c["B"], c["H"], c["S"], c["S"]), np.float32))
    out = gpu.flash_attention2(Q, K, V, mask=tril)
    _check_case(out, "cfg1", c, TOL_F32)
    c8 = cases.PREFILL_CASES["tiny_s8_d64"]
    Q, K, V = cases.prefill_inputs(c8)
    m = cases.random_dense_mask(c8)
    out = gpu.flash_attention2(Q, K, V, mask=m)
    np.testing.assert_allclose(out, GOLD["prefill_densemask/tiny_s8_d64"], atol=TOL_F32, rtol=0)


def test_mask_conventions_by_shape(gpu):
    rng = np.random.default_rng(77)
    B, H, S, D = 2, 3, 70, 64
    Q, K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(3))
    key = (rng.random((B, S)) > 0.3).astype(np.float32)
    key[:, 0] = 1
    bss = (rng.random((B, S, S)) > 0.3).astype(np.float32)
    bss[:, np.arange(S), np.arange(S)] = 1
    for m in (key, bss, bss[:, None]):
        want = orc.attention_4d(Q, K, V, mask=orc.expand_mask(m, B, H, S))
        got = gpu.flash_attention2(Q, K, V, mask=m)
        assert np.abs(got - want).max() <= TOL_F32
    # a fully masked row follows the reference arithmetic: every score is -1e9 -> uniform average
    full = np.ones((B, H, S, S), np.float32)
    full[0, 1, 5, :] = 0
    got = gpu.flash_attention2(Q, K, V, mask=full)
    np.testing.assert_allclose(got[0, 1, 5], V[0, 1].mean(axis=0), atol=TOL_F32)


def test_rope_pairings_in_the_fused_kernel(gpu):
    rng = np.random.default_rng(78)
    B, H, S, D = 1, 2, 150, 64
    Q, K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(3))
    m = orc.causal_length_mask(B, H, S, None, True)
    pos = np.arange(S)
    want_i = orc.attention_4d(orc.rope_interleaved(Q, pos, 10000.0, 2.0), orc.rope_interleaved(K, pos, 10000.0, 2.0), V, mask=m)
    got_i = gpu.flash_attention2_rope(Q, K, V, rope_base=10000.0, rope_scaling=2.0, causal=True)
    assert np.abs(got_i - want_i).max() <= TOL_F32
    # rotate_half pairing: oracle works on (B,S,H,D)
    qh = orc.rope_half(Q.transpose(0, 2, 1, 3), 500.0).transpose(0, 2, 1, 3)
    kh = orc.rope_half(K.transpose(0, 2, 1, 3), 500.0).transpose(0, 2, 1, 3)
    want_h = orc.attention_4d(qh, kh, V, mask=m)
    got_h = gpu.flash_attention2(Q, K, V, causal=True, rope_theta=500.0, rope_mode="half")
    assert np.abs(got_h - want_h).max() <= TOL_F32
    # use_rope=False is plain attention
    got_n = gpu.flash_attention2_rope(Q, K, V, use_rope=False, causal=True)
    assert np.abs(got_n - orc.attention_4d(Q, K, V, mask=m)).max() <= TOL_F32


def test_structural_properties_like_the_reference_tests(gpu):
    # shape / finite / bounded by V / identical queries -> identical rows / mask changes the result
    np.random.seed(42)
    for (B, H, S, D) in [(1, 1, 16, 64), (1, 1, 8, 64), (1, 4, 8, 64), (1, 1, 1, 64), (1, 1, 4, 64), (1, 1, 32, 64)]:
        Q = np.random.randn(B, H, S, D).astype(np.float32) * 0.1
        K = np.random.randn(B, H, S, D).astype(np.float32) * 0.1
        V = np.random.randn(B, H, S, D).astype(np.float32) * 0.1
        out = gpu.flash_attention2(Q, K, V)
        assert out.shape == (B, H, S, D) and np.all(np.isfinite(out)) and np.abs(out).sum() > 0
        assert np.all(out >= V.min() - 0.01) and np.all(out <= V.max() + 0.01)
    q_vec = np.random.randn(64).astype(np.float32) * 0.1
    Q = np.tile(q_vec, (1, 1, 4, 1))
    K = np.random.randn(1, 1, 4, 64).astype(np.float32) * 0.1
    V = np.random.randn(1, 1, 4, 64).astype(np.float32) * 0.1
    out = gpu.flash_attention2(Q, K, V)
    for i in range(1, 4):
        np.testing.assert_allclose(out[0, 0, 0], out[0, 0, i], atol=1e-4)
    Q = np.random.randn(1, 1, 8, 64).astype(np.float32) * 0.1
    K = np.random.randn(1, 1, 8, 64).astype(np.float32) * 0.1
    V = np.random.randn(1, 1, 8, 64).astype(np.float32) * 0.1
    mask = np.tril(np.ones((1, 1, 8, 8), np.float32))
    assert not np.allclose(gpu.flash_attention2(Q, K, V, mask=mask)[0, 0, 0], gpu.flash_attention2(Q, K, V)[0, 0, 0], atol=1e-6)


def test_error_behaviour(gpu):
    x = np.zeros((2, 8, 64), np.float32)
    with pytest.raises(RuntimeError, match="Q must be 4D"):
        gpu.flash_attention2(x, x, x)
    q = np.zeros((1, 1, 8, 48), np.float32)
    with pytest.raises(RuntimeError, match="head_dim"):
        gpu.flash_attention2(q, q, q)
    q = np.zeros((1, 1, 8, 32), np.float32)
    with pytest.raises(RuntimeError, match="bf16 path"):
        gpu.flash_attention2(q, q, q, dtype="bf16")          # the tensor-core kernel takes head_dim 128 and 64
    stats = gpu.device.pool_stats()
    assert set(stats) == {"hits", "misses", "allocations", "total_acquired", "total_released"}
    assert set(gpu.device.cache_stats()) == {"hits", "misses", "evictions", "cached_sets"}
    assert "B200" in gpu.device.device_name or len(gpu.device.device_name) > 0


# --------------------------------------------------------------------------- bf16 tensor-core path
@pytest.mark.parametrize("name", ["cfg2_small", "ragged_d128", "noncausal_d128", "cfg1", "odd_s_d64", "tiny_s8_d64", "s1_d64"])
def test_tcgen05_kernel_small_cases(dev, name):
    from grilly_next import cabi
    from gpu_helpers import flash_cabi
    c = cases.PREFILL_CASES[name]
    Q, K, V = cases.prefill_inputs(c)
    out = flash_cabi(dev, Q, K, V, causal=c["causal"], seq_lens=cases.seq_lens(c),
                     rope_mode=cabi.ROPE_INTERLEAVED if c.get("rope") else cabi.ROPE_NONE,
                     rope_theta=c.get("rope", 10000.0), bf16=True, kernel=cabi.KERNEL_TCGEN05)
    assert np.all(np.isfinite(out))
    _check_case(out, name, c, TOL_BF16)


def test_tcgen05_kernel_rope_half_and_bf16_out(dev):
    from grilly_next import cabi
    from gpu_helpers import flash_cabi
    rng = np.random.default_rng(79)
    B, H, S, D = 1, 2, 300, 128
    Q, K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(3))
    qh = orc.rope_half(Q.transpose(0, 2, 1, 3), 10000.0).transpose(0, 2, 1, 3)
    kh = orc.rope_half(K.transpose(0, 2, 1, 3), 10000.0).transpose(0, 2, 1, 3)
    want = orc.attention_4d(qh, kh, V, mask=orc.causal_length_mask(B, H, S, None, True))
    got = flash_cabi(dev, Q, K, V, causal=True, rope_mode=cabi.ROPE_HALF, bf16=True, kernel=cabi.KERNEL_TCGEN05)
    assert np.abs(got - want).max() <= TOL_BF16
    got16 = flash_cabi(dev, Q, K, V, causal=True, rope_mode=cabi.ROPE_HALF, bf16=True, kernel=cabi.KERNEL_TCGEN05,
                       out_bf16=True)
    assert np.abs(got16 - want).max() <= 3e-2   # + one bf16 rounding of O


@pytest.mark.parametrize("mode", ["interleaved", "half"])
def test_tcgen05_kernel_head_dim_64_with_rope(dev, mode):
    """head_dim 64 (the shape of the reference's own tests) on the tensor-core kernel: both RoPE pairings, ragged
    lengths, float32 and bf16 output, a sequence long enough for several K tiles."""
    from grilly_next import cabi
    from gpu_helpers import flash_cabi
    rng = np.random.default_rng(80)
    B, H, S, D = 2, 3, 700, 64
    lens = np.array([700, 333], np.int32)
    Q, K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(3))
    pos = np.arange(S)
    if mode == "interleaved":
        q, k = orc.rope_interleaved(Q, pos, 10000.0), orc.rope_interleaved(K, pos, 10000.0)
    else:
        q = orc.rope_half(Q.transpose(0, 2, 1, 3), 10000.0).transpose(0, 2, 1, 3)
        k = orc.rope_half(K.transpose(0, 2, 1, 3), 10000.0).transpose(0, 2, 1, 3)
    want = orc.attention_4d(q, k, V, mask=orc.causal_length_mask(B, H, S, lens, True))
    want[1, :, 333:] = 0.0
    rm = cabi.ROPE_INTERLEAVED if mode == "interleaved" else cabi.ROPE_HALF
    got = flash_cabi(dev, Q, K, V, causal=True, seq_lens=lens, rope_mode=rm, bf16=True, kernel=cabi.KERNEL_TCGEN05)
    assert np.abs(got - want).max() <= TOL_BF16
    got16 = flash_cabi(dev, Q, K, V, causal=True, seq_lens=lens, rope_mode=rm, bf16=True, kernel=cabi.KERNEL_AUTO, out_bf16=True)
    assert np.abs(got16 - want).max() <= 3e-2   # + one bf16 rounding of O


def test_tcgen05_cfg2_full_size(dev):
    """Configuration 2 at full size: sampled heads against the golden vectors, every head against
    the fp32 SIMT kernel fed the same bf16 inputs, and the softmax row-sum property (V = 1 -> O = 1)."""
    from grilly_next import cabi
    from gpu_helpers import flash_cabi
    c = cases.PREFILL_CASES["cfg2"]
    Q, K, V = cases.prefill_inputs(c)
    out = flash_cabi(dev, Q, K, V, causal=True, rope_mode=cabi.ROPE_INTERLEAVED, rope_theta=c["rope"], bf16=True,
                     kernel=cabi.KERNEL_TCGEN05)
    assert np.all(np.isfinite(out))
    _check_case(out, "cfg2", c, TOL_BF16)
    ref = flash_cabi(dev, Q, K, V, causal=True, rope_mode=cabi.ROPE_INTERLEAVED, rope_theta=c["rope"], bf16=True,
                     kernel=cabi.KERNEL_SIMT_F32)
    assert np.abs(out - ref).max() <= TOL_BF16
    ones = flash_cabi(dev, Q, K, np.ones_like(V), causal=True, rope_mode=cabi.ROPE_INTERLEAVED, rope_theta=c["rope"],
                      bf16=True, kernel=cabi.KERNEL_TCGEN05)
    assert np.abs(ones - 1.0).max() <= 1e-2


def test_tcgen05_cfg5_padded_batch_full_size(dev):
    """Configuration 5 at full size: batch 8, 32 heads, max seq 4096, per-sequence lengths uniform in
    [512, 4096] from a seed, causal + padding, RoPE.  Sampled (batch, head) slices against the C oracle
    on the unrounded fp32 inputs; padded query rows must be exactly zero."""
    from grilly_next import cabi
    from gpu_helpers import flash_cabi
    from oracle import c_oracle
    rng = np.random.default_rng(1005)
    B, H, S, D = 8, 32, 4096, 128
    lens = rng.integers(512, 4097, size=B).astype(np.int32)
    Q = rng.standard_normal((B, H, S, D), dtype=np.float32)
    K = rng.standard_normal((B, H, S, D), dtype=np.float32)
    V = rng.standard_normal((B, H, S, D), dtype=np.float32)
    out = flash_cabi(dev, Q, K, V, causal=True, seq_lens=lens, rope_mode=cabi.ROPE_INTERLEAVED, rope_theta=10000.0,
                     bf16=True, kernel=cabi.KERNEL_TCGEN05)
    assert np.all(np.isfinite(out))
    pos = np.arange(S)
    pick = [(int(np.argmin(lens)), 0), (int(np.argmax(lens)), 31), (3, 7), (6, 20)]
    for (b, h) in pick:
        q = orc.rope_interleaved(Q[b:b + 1, h:h + 1], pos)
        k = orc.rope_interleaved(K[b:b + 1, h:h + 1], pos)
        want = c_oracle.attention(q, k, V[b:b + 1, h:h + 1], causal=True, seq_lens=lens[b:b + 1])
        err = np.abs(out[b, h] - want[0, 0]).max()
        assert err <= TOL_BF16, f"cfg5 ({b},{h}) len {lens[b]}: max-abs {err:.3e}"
    for b in range(B):
        assert np.all(out[b, :, lens[b]:] == 0)


def test_python_op_bf16_path(gpu):
    c = cases.PREFILL_CASES["cfg2_small"]
    Q, K, V = cases.prefill_inputs(c)
    out = gpu.flash_attention2(Q, K, V, causal=True, rope_theta=c["rope"], dtype="bf16")
    _check_case(out, "cfg2_small", c, TOL_BF16)
    # out=: the result lands in the caller's array
    buf = np.empty_like(Q)
    ret = gpu.flash_attention2(Q, K, V, causal=True, rope_theta=c["rope"], dtype="bf16", out=buf)
    assert ret is buf or np.shares_memory(ret, buf)
    assert np.array_equal(buf, out)
    with pytest.raises(RuntimeError, match="out must be"):
        gpu.flash_attention2(Q, K, V, out=np.empty((1, 2, 3, 4), np.float32))


def test_python_op_chunked_pipeline_is_bit_identical(dev, gpu):
    # Above 8 MiB per tensor the host op uploads, computes and downloads (batch, head) chunks on three
    # queues at once; the chunks must give exactly what one launch over device-resident tensors gives.
    from grilly_next import cabi
    from gpu_helpers import flash_cabi
    rng = np.random.default_rng(77)
    # bf16 tensor-core kernel, causal + RoPE + ragged lengths: 2 chunks of 8 heads
    B, H, S, D = 2, 8, 1024, 128
    Q, K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(3))
    lens = np.array([1024, 700], np.int32)
    got = gpu.flash_attention2(Q, K, V, causal=True, seq_lens=lens, rope_theta=10000.0, dtype="bf16")
    want = flash_cabi(dev, Q, K, V, causal=True, seq_lens=lens, rope_mode=cabi.ROPE_INTERLEAVED, bf16=True,
                      kernel=cabi.KERNEL_TCGEN05)
    assert np.array_equal(got, want)
    # fp32 kernel with the reference's (batch, seq) key mask: 6 chunks, the last one short
    B, H, S, D = 2, 40, 512, 128
    Q, K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(3))
    mask = (rng.random((B, S)) > 0.3).astype(np.float32)
    got = gpu.flash_attention2(Q, K, V, mask=mask)
    want = flash_cabi(dev, Q, K, V, mask=mask, mask_kind=cabi.MASK_KEY)
    assert np.array_equal(got, want)
