"""Device-resident tensors and the device group of the Python module: same kernels as the host-array
path, so results must be bit-identical to it."""
import numpy as np
import pytest

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def core():
    import grilly_core
    return grilly_core


@pytest.fixture(scope="module")
def ctx(core):
    return core.Device()


def test_round_trip_and_properties(core, ctx):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((3, 5, 7), dtype=np.float32)
    t = core.DeviceTensor.from_numpy(ctx, a)
    assert t.shape == (3, 5, 7) and t.dtype == "fp32" and t.nbytes == a.nbytes and t.data_ptr != 0
    assert np.array_equal(t.to_numpy(), a)
    tb = core.DeviceTensor.from_numpy(ctx, a, dtype="bf16")
    assert tb.dtype == "bf16" and tb.nbytes == a.size * 2
    assert np.array_equal(tb.to_numpy(), orc.round_bf16(a))          # round-to-nearest-even on the device
    buf = np.empty_like(a)
    assert tb.to_numpy(out=buf) is buf or np.shares_memory(tb.to_numpy(out=buf), buf)
    t.copy_from_numpy(a * 2)
    assert np.array_equal(t.to_numpy(), a * 2)
    e = core.DeviceTensor.empty(ctx, (2, 4), "fp32")
    assert e.shape == (2, 4)
    with pytest.raises(RuntimeError, match="dtype"):
        core.DeviceTensor.from_numpy(ctx, a, dtype="fp8")


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_flash_on_device_tensors_equals_host_path(core, ctx, dtype):
    rng = np.random.default_rng(2)
    B, H, S, D = 2, 4, 384, 128
    Q, K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(3))
    lens = np.array([384, 200], np.int32)
    kw = dict(causal=True, seq_lens=lens, rope_theta=10000.0)
    want = core.flash_attention2(ctx, Q, K, V, dtype=dtype, **kw)
    tq, tk, tv = (core.DeviceTensor.from_numpy(ctx, x, dtype=dtype) for x in (Q, K, V))
    out = core.flash_attention2(ctx, tq, tk, tv, **kw)
    assert isinstance(out, core.DeviceTensor) and out.dtype == "fp32" and out.shape == (B, H, S, D)
    ctx.synchronize()
    assert np.array_equal(out.to_numpy(), want)
    # out=: reuse a result tensor
    again = core.flash_attention2(ctx, tq, tk, tv, out=out, **kw)
    assert again.data_ptr == out.data_ptr
    assert np.array_equal(again.to_numpy(), want)
    with pytest.raises(RuntimeError, match="causal / seq_lens"):
        core.flash_attention2(ctx, tq, tk, tv, mask=np.ones((B, S), np.float32))
    with pytest.raises(RuntimeError, match="same shape"):
        core.flash_attention2(ctx, tq, tk, core.DeviceTensor.empty(ctx, (B, H, S, 64), dtype))


def test_decode_on_device_tensors_equals_host_path(core, ctx):
    rng = np.random.default_rng(3)
    B, Hq, Hkv, D, T = 2, 8, 2, 128, 150
    k0 = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v0 = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    caches = []
    for _ in range(2):
        kv = core.create_kv_cache(ctx, max_seq_len=512, num_heads=Hkv, head_dim=D, compression_ratio=1,
                                  max_cache_tokens=512, batch_size=B)
        core.kv_cache_append(ctx, kv, k0, v0, rope_theta=10000.0)
        caches.append(kv)
    for step in range(3):
        q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        kn = rng.standard_normal((B, 1, Hkv, D), dtype=np.float32)
        vn = rng.standard_normal((B, 1, Hkv, D), dtype=np.float32)
        want = core.decode_step(ctx, caches[0], q, kn, vn)
        tq, tk, tv = (core.DeviceTensor.from_numpy(ctx, x) for x in (q, kn, vn))
        got = core.decode_step(ctx, caches[1], tq, tk, tv)
        assert np.array_equal(got.to_numpy(), want)
        assert caches[1].current_len == caches[0].current_len == T + step + 1
    q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
    want = core.gqa_attention(ctx, q, caches[0])
    got = core.gqa_attention(ctx, core.DeviceTensor.from_numpy(ctx, q), caches[1])
    assert np.array_equal(got.to_numpy(), want)
    for kv in caches:
        core.destroy_kv_cache(ctx, kv)


def test_device_group_splits_heads(core, ctx):
    import torch
    n = min(2, torch.cuda.device_count())
    group = core.DeviceGroup(n)
    assert len(group) == n and group[0].gpu_index == 0
    rng = np.random.default_rng(4)
    B, H, S, D = 2, 6, 256, 64
    Q, K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(3))
    lens = np.array([256, 100], np.int32)
    want = core.flash_attention2(ctx, Q, K, V, causal=True, seq_lens=lens)
    got = group.flash_attention2(Q, K, V, causal=True, seq_lens=lens)
    assert np.array_equal(got, want)
    with pytest.raises(RuntimeError, match="devices asked for"):
        core.DeviceGroup(99)


def test_names_outside_this_build_say_so(core, ctx):
    for name in ("relu", "gelu", "layernorm", "conv2d", "hamming_search"):
        with pytest.raises(RuntimeError, match="outside the attention"):
            getattr(core, name)(ctx)
