"""Pins of the oracle for the unfused attention pieces and the backward pass (CPU only).

The backward is compared with outputs of the reference's own numpy backward (tests/golden/make_backward_golden.py) and
with central differences; the three forward pieces, composed, with the golden vectors of the fused prefill path."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

import cases  # noqa: E402
import make_backward_golden as mbg  # noqa: E402
from oracle import attention_unfused_oracle as uo  # noqa: E402

GOLD = np.load(os.path.join(HERE, "golden", "attention_backward_golden.npz"))


@pytest.mark.parametrize("case", sorted(mbg.CASES))
def test_backward_matches_reference_numpy(case):
    gq, gk, gv = uo.attention_backward(*mbg.backward_inputs(case))
    for got, name in ((gq, "grad_q"), (gk, "grad_k"), (gv, "grad_v")):
        want = GOLD[f"{case}/{name}"]
        assert got.shape == want.shape
        assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())    # the reference sums in float32


def test_backward_matches_central_differences():
    go, q, k, v, _, scale = mbg.backward_inputs("b1h2s12d8")
    q, k, v, go = (t.astype(np.float64) for t in (q, k, v, go))

    def loss(q_, k_, v_):
        a = uo.softmax(np.einsum("bhid,bhjd->bhij", q_, k_) * scale)
        return float((np.einsum("bhij,bhjd->bhid", a, v_) * go).sum())

    attn = uo.softmax(np.einsum("bhid,bhjd->bhij", q, k) * scale)
    gq, gk, gv = uo.attention_backward(go, q, k, v, attn, scale)
    rng = np.random.default_rng(0)
    eps = 1e-6
    for which, grad in ((0, gq), (1, gk), (2, gv)):
        for _ in range(6):
            idx = tuple(rng.integers(0, n) for n in q.shape)
            args = [q.copy(), k.copy(), v.copy()]
            args[which][idx] += eps
            up = loss(*args)
            args[which][idx] -= 2 * eps
            dn = loss(*args)
            assert abs((up - dn) / (2 * eps) - grad[idx]) <= 1e-6 * max(1.0, abs(grad[idx]))


def test_forward_pieces_compose_to_the_golden_prefill():
    gold = np.load(os.path.join(HERE, "golden", "attention_golden.npz"))
    name = next(n for n, c in cases.PREFILL_CASES.items()
                if not c.get("rope") and not c.get("causal") and cases.seq_lens(c) is None and not c.get("mask"))
    c = cases.PREFILL_CASES[name]
    Q, K, V = cases.prefill_inputs(c)                      # (B,H,S,D)
    b, h = cases.sampled_heads(c)[0]
    q = Q[b:b + 1, h:h + 1].transpose(0, 2, 1, 3)          # (1,S,1,D): the layout the separate shaders use
    k = K[b:b + 1, h:h + 1].transpose(0, 2, 1, 3)
    v = V[b:b + 1, h:h + 1].transpose(0, 2, 1, 3)
    out = uo.attention_output(uo.softmax(uo.attention_scores(q, k)), v)
    want = gold[f"prefill/{name}/{b}_{h}"]
    assert np.abs(out[0, :, 0, :] - want).max() <= 2e-5


def test_causal_output_is_the_lower_triangle():
    rng = np.random.default_rng(5)
    w = rng.random((2, 3, 9, 9))
    v = rng.standard_normal((2, 9, 3, 4))
    out = uo.attention_output(w, v, causal=True)
    for q in range(9):
        want = np.einsum("bhk,bkhd->bhd", w[:, :, q, :q + 1], v[:, :q + 1])
        np.testing.assert_allclose(out[:, q], want, atol=1e-12)


def test_softmax_rows_sum_to_one_and_survive_large_inputs():
    x = np.array([[1000.0, 1001.0, 999.0], [-5e9, -5e9, -5e9]])
    y = uo.softmax(x)
    np.testing.assert_allclose(y.sum(-1), 1.0, atol=1e-12)
    np.testing.assert_allclose(y[1], 1 / 3, atol=1e-12)
