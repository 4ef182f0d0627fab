"""Linear projection (the steps on either side of attention): exact fp32 form and bf16 tensor-core form against
numpy, edge shapes, the packed QKV projection, and the projection -> attention -> projection chain the reference's
integration test builds (tests/test_integration.py:96-118 there)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import grilly_next
    g = grilly_next.Compute()
    yield g
    g.cleanup()


@pytest.mark.parametrize("M,K,N", [(300, 136, 200), (1, 8, 3), (128, 64, 128), (257, 1024, 129), (5, 72, 1)])
def test_linear_both_precisions(gpu, M, K, N):
    rng = np.random.default_rng(M + K + N)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = rng.standard_normal((N, K), dtype=np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    got = gpu.linear(x, w)
    assert got.shape == (M, N) and got.dtype == np.float32
    assert np.abs(got - want).max() <= 1e-4 * np.sqrt(K / 64)
    got = gpu.linear(x, w, b)
    assert np.abs(got - (want + b)).max() <= 1e-4 * np.sqrt(K / 64)
    # tensor-core form: operands rounded to bf16 once, float32 accumulation
    from oracle import attention_oracle as orc
    want16 = orc.round_bf16(x).astype(np.float64) @ orc.round_bf16(w).astype(np.float64).T + b
    got16 = gpu.linear(x, w, b, dtype="bf16")
    assert np.abs(got16 - want16).max() <= 2e-5 * K          # accumulation order only
    assert np.abs(got16 - (want + b)).max() <= 0.02 * np.sqrt(K)   # against the unrounded product


def test_linear_shapes_and_errors(gpu):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 7, 32), dtype=np.float32)
    w = rng.standard_normal((10, 32), dtype=np.float32)
    out = gpu.linear(x, w)
    assert out.shape == (2, 7, 10)
    np.testing.assert_allclose(out, x @ w.T, atol=1e-4)
    assert gpu.linear(x[0, 0], w).shape == (1, 10)                      # 1-D input: (1, out) as the reference returns it
    with pytest.raises(RuntimeError, match="Weight input_dim mismatch"):
        gpu.linear(x, w[:, :16])
    with pytest.raises(RuntimeError, match="bias must be 1D"):
        gpu.linear(x, w, np.zeros(3, np.float32))
    with pytest.raises(RuntimeError, match="multiple of 8"):
        gpu.linear(rng.standard_normal((4, 12), dtype=np.float32), rng.standard_normal((5, 12), dtype=np.float32), dtype="bf16")


def test_fused_qkv_projection_feeds_attention(gpu):
    rng = np.random.default_rng(4)
    B, S, hidden, H, D = 2, 96, 256, 4, 64
    x = rng.standard_normal((B, S, hidden), dtype=np.float32) * 0.5
    w = (rng.standard_normal((3 * H * D, hidden)) / np.sqrt(hidden)).astype(np.float32)
    b = rng.standard_normal(3 * H * D, dtype=np.float32) * 0.1
    qkv = gpu.fused_qkv_projection(x, w, b, num_heads=H, head_dim=D)
    assert qkv.shape == (B, S, 3 * H * D)
    want = x.reshape(-1, hidden).astype(np.float64) @ w.astype(np.float64).T + b
    assert np.abs(qkv.reshape(-1, 3 * H * D) - want).max() <= 1e-4
    # projection -> attention -> output projection
    q, k, v = (qkv[..., i * H * D:(i + 1) * H * D].reshape(B, S, H, D).transpose(0, 2, 1, 3).copy() for i in range(3))
    att = gpu.flash_attention2(q, k, v, causal=True)
    wo = (rng.standard_normal((hidden, H * D)) / np.sqrt(H * D)).astype(np.float32)
    out = gpu.linear(att.transpose(0, 2, 1, 3).reshape(B, S, H * D).copy(), wo)
    from oracle import attention_oracle as orc
    ref = orc.attention_4d(q, k, v, mask=orc.causal_length_mask(B, H, S, None, True))
    ref = ref.transpose(0, 2, 1, 3).reshape(B, S, H * D) @ wo.T
    assert out.shape == (B, S, hidden) and np.abs(out - ref).max() <= 2e-4
    qkv16 = gpu.fused_qkv_projection(x, w, b, num_heads=H, head_dim=D, dtype="bf16")
    assert np.abs(qkv16.reshape(-1, 3 * H * D) - want).max() <= 0.05
