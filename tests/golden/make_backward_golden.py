"""Generate tests/golden/attention_backward_golden.npz from the reference's own numpy attention backward.

Run in the build container, where the reference checkout is mounted:
    python tests/golden/make_backward_golden.py /path/to/reference

VulkanBackwardOps.attention_backward (src/grilly_next/backend/autograd_core.py:617-655) is imported from the
checkout and called unmodified on seeded inputs; only its OUTPUTS (float32) are stored.  The tests regenerate the
inputs from the same seeds (backward_inputs below).
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {"b1h2s12d8": (1, 2, 12, 8, 11), "b2h3s33d16": (2, 3, 33, 16, 12), "b1h1s70d64": (1, 1, 70, 64, 13)}


def backward_inputs(case):
    """Seeded (grad_out, q, k, v, attn, scale); attn is the float32 softmax of scale * q k^T (row sums 1)."""
    B, H, S, D, seed = CASES[case]
    rng = np.random.default_rng(seed)
    q, k, v, go = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(4))
    scale = np.float32(1.0 / np.sqrt(D))
    s = np.matmul(q, k.swapaxes(-2, -1)) * scale
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    attn = (e / e.sum(axis=-1, keepdims=True)).astype(np.float32)
    return go, q, k, v, attn, float(scale)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_backward_golden.py <checkout of Grillcheese-AI/grilly-next>")
    path = os.path.join(sys.argv[1], "src/grilly_next/backend/autograd_core.py")
    spec = importlib.util.spec_from_file_location("reference_autograd_core", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    ops = mod.VulkanBackwardOps()
    out = {}
    for name in CASES:
        gq, gk, gv = ops.attention_backward(*backward_inputs(name))
        out[name + "/grad_q"], out[name + "/grad_k"], out[name + "/grad_v"] = gq, gk, gv
    dst = os.path.join(HERE, "attention_backward_golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
