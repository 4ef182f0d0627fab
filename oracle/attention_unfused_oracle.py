"""CPU oracle for the unfused attention pieces and the attention backward pass (TEST INFRASTRUCTURE, never the
product path).

Restates in numpy the index arithmetic of the reference's separate shaders; each function names the shader it follows
(Grillcheese-AI/grilly-next, paths relative to that project).  Sums run in float64 here, so the comparison with the
float32 kernels measures their rounding, not the order of a float32 sum.  `attention_backward` is pinned against outputs of the
reference's own numpy backward (VulkanBackwardOps.attention_backward, src/grilly_next/backend/autograd_core.py:617-655,
run unmodified by tests/golden/make_backward_golden.py) and against central differences of the forward.  The three
forward pieces are pinned through their composition: softmax(attention_scores) fed to attention_output must equal
the golden prefill vectors of the fused path; taken one by one the reference holds no test or vector for them.
"""
from __future__ import annotations

import numpy as np


def attention_scores(q, k, scale=0.0):
    """shaders/attention-scores.glsl:33-65: q, k (B,S,H,D) -> (B,H,S,S), score = sum_d q k * scale."""
    q = np.asarray(q, np.float64)
    k = np.asarray(k, np.float64)
    if scale == 0.0:
        scale = 1.0 / np.sqrt(q.shape[-1])
    return np.einsum("bqhd,bkhd->bhqk", q, k) * scale


def softmax(x):
    """shaders/activation-softmax.glsl:34-84: over the last axis; the maximum starts from -1e10."""
    x = np.asarray(x, np.float64)
    mx = np.maximum(x.max(axis=-1, keepdims=True), -1e10)
    e = np.exp(x - mx)
    return e / e.sum(axis=-1, keepdims=True)


def attention_output(weights, v, causal=False):
    """shaders/attention-output.glsl:28-70 (all keys) and attention-output-gpt.glsl:29-72 (keys k <= q only):
    weights (B,H,S,S), v (B,S,H,D) -> (B,S,H,D)."""
    w = np.asarray(weights, np.float64)
    v = np.asarray(v, np.float64)
    if causal:
        w = np.tril(w)
    return np.einsum("bhqk,bkhd->bqhd", w, v)


def attention_backward(grad_out, q, k, v, attn, scale=0.0):
    """shaders/attention-backward.glsl:73-195, all tensors (B,H,S,D), attn (B,H,S,S):
    pass 0  grad_V[j,d] = sum_i attn[i,j] gO[i,d];  pass 1  grad_attn[i,j] = sum_d gO[i,d] V[j,d];
    pass 2  gS = attn * (grad_attn - rowsum(attn * grad_attn)); grad_Q = scale gS K; grad_K = scale gS^T Q."""
    go, q, k, v, a = (np.asarray(t, np.float64) for t in (grad_out, q, k, v, attn))
    if scale == 0.0:
        scale = 1.0 / np.sqrt(q.shape[-1])
    gv = np.einsum("bhij,bhid->bhjd", a, go)
    ga = np.einsum("bhid,bhjd->bhij", go, v)
    gs = a * (ga - (a * ga).sum(axis=-1, keepdims=True))
    gq = scale * np.einsum("bhij,bhjd->bhid", gs, k)
    gk = scale * np.einsum("bhij,bhid->bhjd", gs, q)
    return gq, gk, gv
