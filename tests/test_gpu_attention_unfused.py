"""The unfused attention pieces and the attention backward pass on the GPU against their oracle (float32, 1e-4),
against the golden vectors of the reference's numpy backward, and chained against the fused kernel."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

pytestmark = pytest.mark.gpu

TOL = 1e-4


@pytest.fixture(scope="module")
def gpu():
    import grilly_next
    g = grilly_next.Compute()
    yield g
    g.cleanup()


SHAPES = [(1, 7, 1, 8), (2, 33, 3, 16), (1, 130, 4, 64), (2, 256, 2, 128), (1, 17, 5, 40)]


@pytest.mark.parametrize("B,S,H,D", SHAPES)
def test_scores_softmax_output_chain(gpu, B, S, H, D):
    from oracle import attention_unfused_oracle as uo
    rng = np.random.default_rng(B * 1000 + S + H + D)
    q, k, v = (rng.standard_normal((B, S, H, D), dtype=np.float32) for _ in range(3))
    scores = gpu.attention_scores(q, k)
    assert scores.shape == (B, H, S, S) and scores.dtype == np.float32
    assert np.abs(scores - uo.attention_scores(q, k)).max() <= TOL
    assert np.abs(gpu.attention_scores(q, k, 0.25) - uo.attention_scores(q, k, 0.25)).max() <= TOL * 4
    w = gpu.activation_softmax(scores)
    assert np.abs(w - uo.softmax(scores)).max() <= 1e-6
    np.testing.assert_allclose(w.sum(-1), 1.0, atol=1e-5)
    for causal in (False, True):
        out = gpu.attention_output(w, v, causal)
        assert out.shape == (B, S, H, D)
        assert np.abs(out - uo.attention_output(w, v, causal)).max() <= TOL


def test_chain_equals_the_fused_kernel(gpu):
    rng = np.random.default_rng(7)
    B, S, H, D = 2, 96, 4, 64
    q, k, v = (rng.standard_normal((B, S, H, D), dtype=np.float32) for _ in range(3))
    out = gpu.attention_output(gpu.activation_softmax(gpu.attention_scores(q, k)), v)
    t = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))      # the fused op takes (B,H,S,D)
    fused = gpu.flash_attention2(t(q), t(k), t(v))
    assert np.abs(t(out) - fused).max() <= TOL


def test_softmax_shapes_and_extremes(gpu):
    from oracle import attention_unfused_oracle as uo
    rng = np.random.default_rng(8)
    for shape in [(5,), (3, 1), (4, 300), (2, 3, 1025), (1, 1, 2, 7)]:
        x = (rng.standard_normal(shape) * 6).astype(np.float32)
        y = gpu.activation_softmax(x)
        assert y.shape == x.shape
        assert np.abs(y - uo.softmax(x)).max() <= 1e-6
    x = np.array([[1000.0, 1001.0, 999.0], [-80.0, 80.0, 0.0]], np.float32)
    assert np.abs(gpu.activation_softmax(x) - uo.softmax(x)).max() <= 1e-6


@pytest.mark.parametrize("case", ["b1h2s12d8", "b2h3s33d16", "b1h1s70d64"])
def test_backward_matches_reference_numpy_and_oracle(gpu, case):
    import make_backward_golden as mbg
    from oracle import attention_unfused_oracle as uo
    gold = np.load(os.path.join(HERE, "golden", "attention_backward_golden.npz"))
    go, q, k, v, attn, scale = mbg.backward_inputs(case)
    got = gpu.attention_backward(go, q, k, v, attn, scale)
    want = uo.attention_backward(go, q, k, v, attn, scale)
    for g, w, name in zip(got, want, ("grad_q", "grad_k", "grad_v")):
        assert g.shape == q.shape and g.dtype == np.float32
        assert np.abs(g - w).max() <= TOL, name
        assert np.abs(g - gold[f"{case}/{name}"]).max() <= TOL, name
    # scale 0 means 1/sqrt(D), which is what these cases use
    for g, w in zip(gpu.attention_backward(go, q, k, v, attn), want):
        assert np.abs(g - w).max() <= TOL


def test_backward_larger_shape(gpu):
    from oracle import attention_unfused_oracle as uo
    rng = np.random.default_rng(9)
    B, H, S, D = 2, 4, 200, 128
    q, k, v, go = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(4))
    attn = uo.softmax(np.einsum("bhid,bhjd->bhij", q, k) / np.sqrt(D)).astype(np.float32)
    got = gpu.attention_backward(go, q, k, v, attn)
    for g, w in zip(got, uo.attention_backward(go, q, k, v, attn)):
        assert np.abs(g - w).max() <= 2e-4


def test_argument_errors(gpu):
    z = np.zeros((1, 4, 2, 8), np.float32)
    with pytest.raises(RuntimeError, match="4D"):
        gpu.attention_scores(z[0], z[0])
    with pytest.raises(RuntimeError, match="shapes differ"):
        gpu.attention_scores(z, z[:, :3])
    with pytest.raises(RuntimeError, match="does not match"):
        gpu.attention_output(np.zeros((1, 2, 4, 5), np.float32), z)
    with pytest.raises(RuntimeError, match="shape of q"):
        gpu.attention_backward(z, z, z[:, :3], z, np.zeros((1, 4, 2, 2), np.float32))
    with pytest.raises(RuntimeError, match="attn_weights"):
        gpu.attention_backward(z, z, z, z, np.zeros((1, 4, 2, 3), np.float32))
