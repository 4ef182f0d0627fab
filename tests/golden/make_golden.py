"""Generate the golden vectors under tests/golden/ from the reference's own numpy references.

Run in the build container, where the reference checkout is mounted:
    python tests/golden/make_golden.py [/path/to/reference]

The reference test modules cannot be imported (they import grilly_next at module level), so the
two reference functions are taken out of the files by AST and executed unmodified:
    _ref_attention_4d          tests/test_attention.py:20-35
    _ref_gqa_decode_attention  tests/test_inference_ops.py:64-95
Inputs are regenerated from seeds by the tests (see tests/cases.py); only the reference OUTPUTS
are stored, as float32 inside compressed .npz files.  RoPE is not part of either reference
function: for the RoPE cases the inputs are rotated by oracle.attention_oracle.rope_interleaved
before the reference function is called, so those vectors pin the attention arithmetic only.
"""
import ast
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases  # noqa: E402
from oracle import attention_oracle as orc  # noqa: E402


def load_ref_function(path, name):
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            mod = ast.Module(body=[node], type_ignores=[])
            ns = {"np": np}
            exec(compile(mod, path, "exec"), ns)
            return ns[name]
    raise KeyError(name)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of Grillcheese-AI/grilly-next>")
    ref_root = sys.argv[1]
    ref_attn = load_ref_function(os.path.join(ref_root, "tests/test_attention.py"), "_ref_attention_4d")
    ref_gqa = load_ref_function(os.path.join(ref_root, "tests/test_inference_ops.py"),
                                "_ref_gqa_decode_attention")

    out = {}
    # ---- prefill cases (full tensors for small ones, sampled heads for the big ones)
    for name, c in cases.PREFILL_CASES.items():
        Q, K, V = cases.prefill_inputs(c)
        B, H, S, D = Q.shape
        heads = cases.sampled_heads(c)
        if c.get("rope"):
            pos = np.arange(S)
            Q = orc.rope_interleaved(Q, pos, c["rope"], 1.0)
            K = orc.rope_interleaved(K, pos, c["rope"], 1.0)
        lens = cases.seq_lens(c)
        for (b, h) in heads:
            m = orc.causal_length_mask(1, 1, S, None if lens is None else [lens[b]], c["causal"])
            o = ref_attn(Q[b:b + 1, h:h + 1], K[b:b + 1, h:h + 1], V[b:b + 1, h:h + 1], mask=m)
            if lens is not None:
                o[0, 0, int(lens[b]):] = 0.0   # padded query rows are defined as zero
            out[f"prefill/{name}/{b}_{h}"] = o[0, 0].astype(np.float32)
        print("prefill", name, len(heads), "heads")

    # ---- the reference's mask convention with an explicit dense mask (B,H,S,S)
    c = cases.PREFILL_CASES["tiny_s8_d64"]
    Q, K, V = cases.prefill_inputs(c)
    m = cases.random_dense_mask(c)
    out["prefill_densemask/tiny_s8_d64"] = ref_attn(Q, K, V, mask=m).astype(np.float32)

    # ---- GQA decode cases (shapes of tests/test_inference_ops.py:352-430 plus larger ones)
    for name, c in cases.DECODE_CASES.items():
        q, kc, vc = cases.decode_inputs(c)
        o = ref_gqa(q, kc, vc, c["Hq"], c["Hkv"], c["D"])
        out[f"decode/{name}"] = o.astype(np.float32)
        print("decode", name, o.shape)

    np.savez_compressed(os.path.join(HERE, "attention_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "attention_golden.npz"), len(out), "arrays")


if __name__ == "__main__":
    main()
