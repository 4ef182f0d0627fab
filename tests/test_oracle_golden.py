"""The oracle (numpy and C restatements) against the golden vectors made from the reference's
own numpy references -- the pin that lets the GPU parity tests trust the oracle."""
import os

import numpy as np
import pytest

import cases
from oracle import attention_oracle as orc
from oracle import c_oracle

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_golden.npz"))


def _rotated(c, Q, K):
    if c.get("rope"):
        pos = np.arange(c["S"])
        return orc.rope_interleaved(Q, pos, c["rope"]), orc.rope_interleaved(K, pos, c["rope"])
    return Q, K


@pytest.mark.parametrize("name", [n for n in cases.PREFILL_CASES if n != "cfg2"])
def test_numpy_prefill_matches_reference(name):
    c = cases.PREFILL_CASES[name]
    Q, K, V = cases.prefill_inputs(c)
    Q, K = _rotated(c, Q, K)
    lens = cases.seq_lens(c)
    m = orc.causal_length_mask(c["B"], c["H"], c["S"], lens, c["causal"])
    out = orc.attention_4d(Q, K, V, mask=m)
    for (b, h) in cases.sampled_heads(c):
        want = GOLD[f"prefill/{name}/{b}_{h}"]
        got = out[b, h].copy()
        if lens is not None:
            got[int(lens[b]):] = 0
        np.testing.assert_allclose(got, want, atol=2e-6, rtol=0)


@pytest.mark.parametrize("name", list(cases.PREFILL_CASES))
def test_c_prefill_matches_reference(name):
    c = cases.PREFILL_CASES[name]
    Q, K, V = cases.prefill_inputs(c)
    Q, K = _rotated(c, Q, K)
    heads = cases.sampled_heads(c)
    lens = cases.seq_lens(c)
    for (b, h) in heads:
        sl = None if lens is None else lens[b:b + 1]
        out = c_oracle.attention(Q[b:b + 1, h:h + 1], K[b:b + 1, h:h + 1], V[b:b + 1, h:h + 1],
                                 causal=c["causal"], seq_lens=sl)
        np.testing.assert_allclose(out[0, 0], GOLD[f"prefill/{name}/{b}_{h}"], atol=5e-6, rtol=0)


def test_dense_mask_convention():
    c = cases.PREFILL_CASES["tiny_s8_d64"]
    Q, K, V = cases.prefill_inputs(c)
    m = cases.random_dense_mask(c)
    np.testing.assert_allclose(orc.attention_4d(Q, K, V, mask=m),
                               GOLD["prefill_densemask/tiny_s8_d64"], atol=2e-6, rtol=0)
    # additive form of the same mask through the C restatement
    add = np.where(m[:, 0] > 0, 0.0, -1e9).astype(np.float32)
    np.testing.assert_allclose(c_oracle.attention(Q, K, V, mask_add=add),
                               GOLD["prefill_densemask/tiny_s8_d64"], atol=5e-6, rtol=0)


@pytest.mark.parametrize("name", list(cases.DECODE_CASES))
def test_decode_matches_reference(name):
    c = cases.DECODE_CASES[name]
    q, k, v = cases.decode_inputs(c)
    want = GOLD[f"decode/{name}"]
    got = orc.gqa_decode_attention(q, k, v, c["Hq"], c["Hkv"], c["D"])
    np.testing.assert_allclose(got, want, atol=1e-5 * max(1.0, c["scale"] * 10), rtol=0)
    got_c = c_oracle.gqa_decode(q, k, v)
    np.testing.assert_allclose(got_c, want, atol=1e-5 * max(1.0, c["scale"] * 10), rtol=0)


def test_decode_batch_independence_and_grouping():
    # the properties the reference's own CPU tests assert (tests/test_inference_ops.py:369-416)
    c = cases.DECODE_CASES["kat_b3"]
    q, k, v = cases.decode_inputs(c)
    full = orc.gqa_decode_attention(q, k, v, c["Hq"], c["Hkv"], c["D"])
    for b in range(c["B"]):
        one = orc.gqa_decode_attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], c["Hq"], c["Hkv"], c["D"])
        np.testing.assert_allclose(full[b:b + 1], one, atol=1e-5)
    g = c["Hq"] // c["Hkv"]
    scale = 1.0 / np.sqrt(c["D"])
    for qh in range(c["Hq"]):
        s = k[0, :, qh // g] @ q[0, 0, qh] * scale
        p = np.exp(s - s.max())
        p /= p.sum()
        np.testing.assert_allclose(full[0, 0, qh], p @ v[0, :, qh // g], atol=1e-5)


def test_rope_forms_are_rotations_and_differ():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 16, 3, 64), dtype=np.float32)           # (B,S,H,D)
    yh = orc.rope_half(x)
    yi = orc.rope_interleaved(x.transpose(0, 2, 1, 3), np.arange(16)).transpose(0, 2, 1, 3)
    # both preserve per-vector norms; position 0 is the identity; pairings differ
    np.testing.assert_allclose(np.linalg.norm(yh, axis=-1), np.linalg.norm(x, axis=-1), rtol=1e-5)
    np.testing.assert_allclose(np.linalg.norm(yi, axis=-1), np.linalg.norm(x, axis=-1), rtol=1e-5)
    np.testing.assert_allclose(yh[:, 0], x[:, 0], atol=1e-7)
    np.testing.assert_allclose(yi[:, 0], x[:, 0], atol=1e-7)
    assert np.abs(yh[:, 5] - yi[:, 5]).max() > 1e-2
    # tables reproduce the on-the-fly form (rope.glsl:109-125)
    th = np.arange(16)[:, None] * orc.rope_inv_freq(64, 10000.0)[None]
    np.testing.assert_allclose(orc.rope_half(x, cos=np.cos(th), sin=np.sin(th)), yh, atol=1e-6)
    # relative-position property of the rotated dot product
    q = rng.standard_normal((1, 1, 1, 64), dtype=np.float32)
    kk = rng.standard_normal((1, 1, 1, 64), dtype=np.float32)
    d1 = (orc.rope_interleaved(q, [7]) * orc.rope_interleaved(kk, [3])).sum()
    d2 = (orc.rope_interleaved(q, [104]) * orc.rope_interleaved(kk, [100])).sum()
    assert abs(d1 - d2) < 1e-4


def test_c_rope_matches_the_numpy_restatement():
    from oracle import c_oracle
    rng = np.random.default_rng(6)
    for shape, base, scaling in (((2, 3, 300, 128), 10000.0, 1.0), ((1, 1, 17, 64), 500000.0, 2.0)):
        x = rng.standard_normal(shape, dtype=np.float32)
        want = orc.rope_interleaved(x, np.arange(shape[2]), base, scaling)
        np.testing.assert_allclose(c_oracle.rope_interleaved(x, base, scaling), want, atol=1e-7, rtol=0)


def test_attention_mask_op():
    rng = np.random.default_rng(6)
    s = rng.standard_normal((2, 3, 5, 5), dtype=np.float32)
    c = orc.attention_mask(s, causal=True)
    assert np.all(c[:, :, np.triu_indices(5, 1)[0], np.triu_indices(5, 1)[1]] == np.float32(-1e9))
    assert np.all(np.tril(c[0, 0]) == np.tril(s[0, 0]))
    km = np.array([[1, 1, 0, 1, 0], [1, 0.4, 0.6, 1, 1]], np.float32)
    m = orc.attention_mask(s, mask=km, mask_value=-5.0)
    assert np.all(m[0, :, :, 2] == -5.0) and np.all(m[0, :, :, 4] == -5.0) and np.all(m[1, :, :, 1] == -5.0)
    assert np.all(m[1, :, :, 2] == s[1, :, :, 2])


def test_bf16_rounding_and_lse_merge():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.1415926, 65504.0, 1e-30], np.float32)
    r = orc.round_bf16(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.015625)   # ties to even
    assert np.all(np.abs(r - x) <= np.abs(x) * 2.0 ** -8)
    # merging split partials reproduces the unsplit softmax
    rng = np.random.default_rng(9)
    s = rng.standard_normal((3, 40)) * 3
    v = rng.standard_normal((40, 8))
    full = (np.exp(s - s.max(1, keepdims=True)) / np.exp(s - s.max(1, keepdims=True)).sum(1, keepdims=True)) @ v
    parts_o, parts_m, parts_l = [], [], []
    for lo, hi in ((0, 13), (13, 14), (14, 40)):
        m = s[:, lo:hi].max(1)
        p = np.exp(s[:, lo:hi] - m[:, None])
        parts_o.append(p @ v[lo:hi]); parts_m.append(m); parts_l.append(p.sum(1))
    np.testing.assert_allclose(orc.lse_merge(parts_o, parts_m, parts_l), full, atol=1e-6)
