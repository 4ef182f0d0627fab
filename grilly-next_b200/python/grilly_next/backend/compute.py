"""VulkanCompute: the reference's backend class (src/grilly_next/backend/compute.py:28-111),
attention / KV-cache methods only, dispatching to the CUDA build of grilly_core."""
from . import _bridge


class VulkanCompute:
    """C++ compute backend. All ops dispatch through grilly_core; there is no Python fallback."""

    def __init__(self, shader_dir: str = None):
        if not _bridge.NATIVE_AVAILABLE:
            raise RuntimeError("grilly_core C++ extension not found. Build it with: "
                               "python grilly-next_b200/build.py")
        self._device = _bridge.create_device(shader_dir)

    @property
    def device(self):
        return self._device

    def cleanup(self):
        self._device = None

    # ---- prefill
    def flash_attention2(self, Q, K, V, mask=None, **kwargs):
        return _bridge.flash_attention2(self._device, Q, K, V, mask, **kwargs)

    def flash_attention2_rope(self, Q, K, V, mask=None, **kwargs):
        return _bridge.flash_attention2_rope(self._device, Q, K, V, mask, **kwargs)

    def rope(self, x, **kwargs):
        return _bridge.rope(self._device, x, **kwargs)

    def attention_mask(self, scores, mask=None, **kwargs):
        return _bridge.attention_mask(self._device, scores, mask, **kwargs)

    # ---- KV cache
    def create_kv_cache(self, **kwargs):
        return _bridge.create_kv_cache(self._device, **kwargs)

    def kv_cache_append(self, kv_cache, new_keys, new_values, **kwargs):
        return _bridge.kv_cache_append(self._device, kv_cache, new_keys, new_values, **kwargs)

    def kv_cache_decode(self, kv_cache, seq=0):
        return _bridge.kv_cache_decode(self._device, kv_cache, seq)

    def kv_cache_evict_h2o(self, kv_cache, attention_scores=None, num_evict=0):
        return _bridge.kv_cache_evict_h2o(self._device, kv_cache, attention_scores, num_evict)

    def kv_cache_evict_speculative(self, kv_cache, hidden_states=None, hidden_dim=0):
        return _bridge.kv_cache_evict_speculative(self._device, kv_cache, hidden_states, hidden_dim)

    def kv_cache_compact(self, kv_cache):
        return _bridge.kv_cache_compact(self._device, kv_cache)

    def kv_cache_token_meta(self, kv_cache, seq=0):
        return _bridge.kv_cache_token_meta(self._device, kv_cache, seq)

    def destroy_kv_cache(self, kv_cache):
        return _bridge.destroy_kv_cache(self._device, kv_cache)

    def swizzle_kv(self, input, wave_size=32, reverse=False):
        return _bridge.swizzle_kv(self._device, input, wave_size, reverse)

    # ---- decode
    def gqa_attention(self, q, k_cache, v_cache=None, **kwargs):
        return _bridge.gqa_attention(self._device, q, k_cache, v_cache, **kwargs)

    def decode_step(self, kv_cache, q, k_new, v_new, **kwargs):
        return _bridge.decode_step(self._device, kv_cache, q, k_new, v_new, **kwargs)


    # ---- the projections on either side of attention
    def linear(self, x, weight, bias=None, **kwargs):
        return _bridge.linear(self._device, x, weight, bias, **kwargs)

    def fused_qkv_projection(self, x, w_qkv, b_qkv=None, **kwargs):
        return _bridge.fused_qkv_projection(self._device, x, w_qkv, b_qkv, **kwargs)

    # ---- the unfused attention pieces and the backward pass
    def attention_scores(self, q, k, scale=0.0):
        return _bridge.attention_scores(self._device, q, k, scale)

    def activation_softmax(self, x):
        return _bridge.softmax(self._device, x)

    def attention_output(self, weights, v, causal=False):
        return _bridge.attention_output(self._device, weights, v, causal)

    def attention_backward(self, grad_output, q, k, v, attn_weights, scale=0.0):
        return _bridge.attention_backward(self._device, grad_output, q, k, v, attn_weights, scale)

    # ---- methods of the reference class outside the attention / KV-cache path (compute.py:56-111 there):
    # present and callable; each raises RuntimeError saying that this build does not cover it
    def activation_relu(self, x, **kwargs):
        return _bridge.relu(self._device, x)

    def activation_gelu(self, x, **kwargs):
        return _bridge.gelu(self._device, x)

    def activation_silu(self, x, **kwargs):
        return _bridge.silu(self._device, x)

    def activation_tanh(self, x, **kwargs):
        return _bridge.tanh_act(self._device, x)

    def layernorm(self, x, gamma, beta, eps=1e-5, **kwargs):
        return _bridge.layernorm(self._device, x, gamma, beta, eps)

    def conv2d(self, input, weight, bias=None, **kwargs):
        return _bridge.conv2d(self._device, input, weight, bias, **kwargs)

    def conv1d(self, input, weight, bias=None, **kwargs):
        return _bridge.conv1d(self._device, input, weight, bias, **kwargs)

    def hamming_search(self, query, cache):
        return _bridge.hamming_search(self._device, query, cache)
