"""The MLA latent path of the KV cache: the CPU reference fused_attention_cpu (no GPU needed) and, on a GPU,
create_kv_cache with the reference's default arguments (compression_ratio=4): append = down-projection of
[K | V], kv_cache_decode = up-projection, against numpy.  Parity unpinned: the reference holds no test for the
path and leaves its projection matrices uninitialised; the matrices here are the test's own."""
import numpy as np
import pytest


def _mla_reference(Q, latents, w_up, H, D, mask=None, scale=None):
    """numpy restatement of cpp/src/experimental/fused_attention.cpp:255-357."""
    B, _, S, _ = Q.shape
    T = latents.shape[0] // H
    kv = (latents.astype(np.float64) @ w_up.astype(np.float64)).reshape(T, H, 2 * D)
    K, V = kv[..., :D], kv[..., D:]
    scale = 1.0 / np.sqrt(D) if scale is None else scale
    out = np.empty(Q.shape, np.float64)
    for b in range(B):
        for h in range(H):
            s = (Q[b, h].astype(np.float64) @ K[:, h].T) * scale
            if mask is not None:
                s = s + mask[b]
            p = np.exp(s - s.max(axis=-1, keepdims=True))
            p /= p.sum(axis=-1, keepdims=True)
            out[b, h] = p @ V[:, h]
    return out.astype(np.float32)


def test_fused_attention_cpu_matches_numpy():
    import grilly_core
    rng = np.random.default_rng(21)
    B, H, S, D, L, T = 2, 3, 5, 16, 4, 9
    Q = rng.standard_normal((B, H, S, D), dtype=np.float32)
    latents = rng.standard_normal((T * H, L), dtype=np.float32)
    w_up = rng.standard_normal((L, 2 * D), dtype=np.float32)
    got = grilly_core.fused_attention_cpu(Q, latents, w_up, cached_tokens=T, num_heads=H, head_dim=D, latent_dim=L)
    assert got.shape == (B, H, S, D)
    np.testing.assert_allclose(got, _mla_reference(Q, latents, w_up, H, D), atol=2e-5)
    mask = np.where(rng.random((B, S, T)) < 0.3, -1e9, 0.0).astype(np.float32)
    mask[:, :, 0] = 0.0
    got = grilly_core.fused_attention_cpu(Q, latents, w_up, mask=mask, cached_tokens=T, num_heads=H, head_dim=D,
                                          latent_dim=L, scale=0.2)
    np.testing.assert_allclose(got, _mla_reference(Q, latents, w_up, H, D, mask=mask, scale=0.2), atol=2e-5)
    with pytest.raises(RuntimeError, match="w_up"):
        grilly_core.fused_attention_cpu(Q, latents, w_up[:, :5], cached_tokens=T, num_heads=H, head_dim=D, latent_dim=L)


@pytest.mark.gpu
def test_default_kv_cache_is_the_mla_latent_cache():
    import grilly_core
    ctx = grilly_core.Device()
    rng = np.random.default_rng(22)
    kv = grilly_core.create_kv_cache(ctx, max_cache_tokens=100)        # the reference's defaults: 8 heads, D 64, ratio 4
    H, D, L = 8, 64, 16
    w_down = (rng.standard_normal((2 * D, L)) / np.sqrt(2 * D)).astype(np.float32)
    w_up = (rng.standard_normal((L, 2 * D)) / np.sqrt(L)).astype(np.float32)
    k = rng.standard_normal((70, H, D), dtype=np.float32)
    v = rng.standard_normal((70, H, D), dtype=np.float32)
    grilly_core.kv_cache_append(ctx, kv, k[:1], v[:1])
    got = grilly_core.kv_cache_decode(ctx, kv)                          # zero matrices until they are set
    assert not got["keys"].any() and not got["values"].any()
    grilly_core.kv_cache_set_mla_weights(ctx, kv, w_down, w_up)
    grilly_core.kv_cache_append(ctx, kv, k[1:40], v[1:40])
    grilly_core.kv_cache_append(ctx, kv, k[40:], v[40:])
    assert kv.current_len == 70
    lat = np.concatenate([k, v], axis=-1).astype(np.float64) @ w_down.astype(np.float64)     # (70, H, L)
    lat[0] = 0.0                                                         # the first token went in before the weights
    np.testing.assert_allclose(grilly_core.kv_cache_latents(ctx, kv), lat, atol=2e-5)
    full = lat @ w_up.astype(np.float64)
    got = grilly_core.kv_cache_decode(ctx, kv)
    assert got["keys"].shape == (70, H, D)
    np.testing.assert_allclose(got["keys"], full[..., :D], atol=5e-5)
    np.testing.assert_allclose(got["values"], full[..., D:], atol=5e-5)
    # the CPU reference attends over exactly these latents
    Q = rng.standard_normal((1, H, 3, D), dtype=np.float32)
    lat32 = grilly_core.kv_cache_latents(ctx, kv).reshape(70 * H, L)
    out = grilly_core.fused_attention_cpu(Q, lat32, w_up, cached_tokens=70, num_heads=H, head_dim=D, latent_dim=L)
    np.testing.assert_allclose(out, _mla_reference(Q, lat32, w_up, H, D), atol=2e-5)
    s = kv.stats()
    assert s["current_tokens"] == 70 and abs(s["compression_ratio"] - 8.0) < 1e-6
    with pytest.raises(RuntimeError, match="MLA"):
        grilly_core.gqa_attention(ctx, Q[:, :, :1].transpose(0, 2, 1, 3).copy(), kv)
    with pytest.raises(RuntimeError, match="max_cache_tokens"):
        grilly_core.kv_cache_append(ctx, kv, np.zeros((64, H, D), np.float32), np.zeros((64, H, D), np.float32))
    grilly_core.destroy_kv_cache(ctx, kv)


@pytest.mark.gpu
def test_gemm_f32_follows_the_shader_order():
    import ctypes as C
    from grilly_next import cabi
    dev = cabi.Device(0)
    try:
        rng = np.random.default_rng(23)
        for (M, K, N) in ((37, 50, 19), (16, 16, 16), (1, 130, 3)):
            A = rng.standard_normal((M, K), dtype=np.float32)
            B = rng.standard_normal((K, N), dtype=np.float32)
            a, b, c = dev.upload(A), dev.upload(B), dev.malloc(M * N * 4)
            cabi.check(dev.L.grl_gemm_f32(dev.h, a, b, c, M, K, N))
            dev.sync()
            got = dev.download(c, (M, N), np.float32)
            want = np.zeros((M, N), np.float32)
            for k in range(K):                              # ascending k, separate multiply and add, all in float32
                want = (want + (A[:, k:k + 1] * B[k:k + 1, :]).astype(np.float32)).astype(np.float32)
            assert np.array_equal(got, want)
    finally:
        dev.close()
