"""Thin wrappers around the grilly_core extension, one flat callable per bound op.

Same role and names as the reference's src/grilly_next/backend/_bridge.py:23-145 for the
attention / KV-cache ops; ops outside that subset are absent (getattr-guarded aliases only).
"""
try:
    import grilly_core as _core

    NATIVE_AVAILABLE = True
except ImportError:
    _core = None
    NATIVE_AVAILABLE = False


def _require():
    if not NATIVE_AVAILABLE:
        raise RuntimeError("grilly_core C++ extension not found. Build it with: "
                           "python grilly-next_b200/build.py")


def create_device(shader_dir: str = None):
    """Create a Device; shader_dir is accepted and ignored (kernels are linked in)."""
    _require()
    dev = _core.Device()
    if shader_dir is not None:
        dev.load_shaders(shader_dir)
    return dev


def flash_attention2(device, Q, K, V, mask=None, scale=0.0, tile_size_q=64, tile_size_k=64, **kwargs):
    return _core.flash_attention2(device, Q, K, V, mask, scale, tile_size_q, tile_size_k, **kwargs)


def flash_attention2_rope(device, Q, K, V, mask=None, scale=0.0, rope_base=10000.0, rope_scaling=1.0,
                          use_rope=True, **kwargs):
    return _core.flash_attention2_rope(device, Q, K, V, mask, scale, rope_base, rope_scaling, use_rope, **kwargs)


def rope(device, x, base=10000.0, scaling=1.0, cos=None, sin=None, mode="half"):
    return _core.rope(device, x, base, scaling, cos, sin, mode)


def attention_mask(device, scores, mask=None, causal=False, mask_value=-1e9):
    return _core.attention_mask(device, scores, mask, causal, mask_value)


def create_kv_cache(device, **kwargs):
    return _core.create_kv_cache(device, **kwargs)


def kv_cache_append(device, kv_cache, new_keys, new_values, **kwargs):
    return _core.kv_cache_append(device, kv_cache, new_keys, new_values, **kwargs)


def kv_cache_decode(device, kv_cache, seq=0):
    return _core.kv_cache_decode(device, kv_cache, seq)


def kv_cache_evict_h2o(device, kv_cache, attention_scores=None, num_evict=0):
    return _core.kv_cache_evict_h2o(device, kv_cache, attention_scores, num_evict)


def kv_cache_compact(device, kv_cache):
    return _core.kv_cache_compact(device, kv_cache)


def kv_cache_evict_speculative(device, kv_cache, hidden_states=None, hidden_dim=0):
    return _core.kv_cache_evict_speculative(device, kv_cache, hidden_states, hidden_dim)


def kv_cache_token_meta(device, kv_cache, seq=0):
    return _core.kv_cache_token_meta(device, kv_cache, seq)


def destroy_kv_cache(device, kv_cache):
    return _core.destroy_kv_cache(device, kv_cache)


def gqa_attention(device, q, k_cache, v_cache=None, cache_len=None, scale=0.0, **kwargs):
    return _core.gqa_attention(device, q, k_cache, v_cache, cache_len, scale, **kwargs)


def decode_step(device, kv_cache, q, k_new, v_new, **kwargs):
    return _core.decode_step(device, kv_cache, q, k_new, v_new, **kwargs)


KVCache = getattr(_core, "KVCache", None)
Device = getattr(_core, "Device", None)


def swizzle_kv(device, input, wave_size=32, reverse=False):
    return _core.swizzle_kv(device, input, wave_size, reverse)


# Names of the reference's bridge (src/grilly_next/backend/_bridge.py:23-145) outside the attention /
# KV-cache path: present, so that callers written against the reference import cleanly, and every one
# of them raises RuntimeError saying that this build does not cover it.  There is no CPU fallback.
def _outside(name):
    def op(device=None, *args, **kwargs):
        _require()
        return getattr(_core, name)(device, *args, **kwargs)
    op.__name__ = name
    op.__doc__ = f"{name}: outside the attention / KV-cache path of this build; raises RuntimeError."
    return op


def linear(device, x, weight, bias=None, **kwargs):
    """GPU linear projection: output = x @ W^T + bias (dtype="bf16" selects the tensor-core kernel)."""
    return _core.linear(device, x, weight, bias, **kwargs)


def fused_qkv_projection(device, x, w_qkv, b_qkv=None, num_heads=8, head_dim=64, **kwargs):
    return _core.fused_qkv_projection(device, x, w_qkv, b_qkv, num_heads, head_dim, **kwargs)


def attention_scores(device, q, k, scale=0.0):
    """scores (B,H,S,S) = scale * Q K^T for q, k laid out (B,S,H,D) (shader attention-scores)."""
    return _core.attention_scores(device, q, k, scale)


def softmax(device, x):
    """Softmax over the last axis (shader activation-softmax)."""
    return _core.softmax(device, x)


def attention_output(device, weights, v, causal=False):
    """weights (B,H,S,S) . v (B,S,H,D); causal=True is shader attention-output-gpt."""
    return _core.attention_output(device, weights, v, causal)


def attention_backward(device, grad_output, q, k, v, attn_weights, scale=0.0):
    """(grad_q, grad_k, grad_v), all (B,H,S,D) (shader attention-backward)."""
    return _core.attention_backward(device, grad_output, q, k, v, attn_weights, scale)


for _name in ("linear_cpu", "relu", "gelu", "silu", "tanh_act", "layernorm", "conv1d", "conv2d",
              "hamming_search"):
    globals()[_name] = _outside(_name)
del _name
