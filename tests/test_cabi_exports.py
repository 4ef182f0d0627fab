"""CPU checks of the drop-in boundary: the C-ABI library loads and exports every symbol that
include/grilly_cuda.h declares, and the Python mirror of the reference package imports."""
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "grilly_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(grl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from grilly_next import cabi
    L = cabi.lib()
    names = _declared()
    assert len(names) >= 30
    for n in names:
        assert hasattr(L, n), f"{n} declared in grilly_cuda.h but not exported"
    assert sorted(cabi.SYMBOLS) == names, "cabi.SYMBOLS is out of step with the header"


def test_struct_sizes_match_header_layout(tmp_path):
    # POD parameter blocks are passed by pointer: the ctypes mirrors must have the C layout.
    # Ask the C compiler for the truth.
    import ctypes as C
    import subprocess
    from grilly_next import cabi
    src = tmp_path / "sz.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "grilly_cuda.h"\n'
        'int main(void){printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(grl_kv_layout), sizeof(grl_flash_params),'
        ' sizeof(grl_append_params), sizeof(grl_decode_params), sizeof(grl_device_info),'
        ' offsetof(grl_flash_params, status), offsetof(grl_append_params, update_lens),'
        ' offsetof(grl_decode_params, partial_out), offsetof(grl_decode_params, exchange),'
        ' sizeof(grl_exchange_params), offsetof(grl_exchange_params, flag_slots),'
        ' sizeof(grl_kv_meta), offsetof(grl_append_params, pos_offsets)); return 0;}\n')
    exe = tmp_path / "sz"
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    subprocess.check_call([cc, "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    want = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    got = [C.sizeof(cabi.KVLayout), C.sizeof(cabi.FlashParams), C.sizeof(cabi.AppendParams),
           C.sizeof(cabi.DecodeParams), C.sizeof(cabi.DeviceInfo), cabi.FlashParams.status.offset,
           cabi.AppendParams.update_lens.offset, cabi.DecodeParams.partial_out.offset,
           cabi.DecodeParams.exchange.offset, C.sizeof(cabi.ExchangeParams), cabi.ExchangeParams.flag_slots.offset,
           C.sizeof(cabi.KVMeta), cabi.AppendParams.pos_offsets.offset]
    assert got == want


def test_python_surface_matches_reference_names():
    import grilly_core
    import grilly_next
    from grilly_next.backend import _bridge
    assert grilly_next.VULKAN_AVAILABLE is True
    assert grilly_next.Compute is grilly_next.VulkanCompute
    for n in ("flash_attention2", "create_kv_cache", "kv_cache_append", "kv_cache_decode",
              "kv_cache_evict_h2o", "swizzle_kv", "cleanup"):
        assert hasattr(grilly_next.Compute, n)
    for n in ("create_device", "flash_attention2", "create_kv_cache", "kv_cache_append", "kv_cache_decode",
              "kv_cache_evict_h2o", "kv_cache_compact", "destroy_kv_cache"):
        assert hasattr(_bridge, n)
    for n in ("Device", "KVCache", "flash_attention2", "flash_attention2_rope", "gqa_attention", "rope",
              "attention_mask", "decode_step"):
        assert hasattr(grilly_core, n)
    doc = grilly_core.flash_attention2.__doc__
    for kw in ("mask", "scale", "tile_size_q", "tile_size_k"):
        assert kw in doc


def test_no_device_means_a_loud_error_not_a_fallback():
    from grilly_next import cabi
    import ctypes as C
    L = cabi.lib()
    n = C.c_int(-1)
    rc = L.grl_device_count(C.byref(n))
    if rc == 0 and n.value > 0:
        pytest.skip("a GPU is present")
    import grilly_next
    with pytest.raises(RuntimeError):
        grilly_next.Compute()
    h = C.c_void_p()
    assert L.grl_device_open(0, C.byref(h)) != 0
    assert len(L.grl_last_error()) > 0


def test_host_bf16_rounding_matches_oracle():
    # the chunked upload path rounds on the host threads; it must give the bits the device cast gives
    import grilly_core
    from oracle import attention_oracle as orc
    rng = np.random.default_rng(0)
    x = rng.standard_normal(300_001, dtype=np.float32) * np.float32(10.0) ** rng.integers(-30, 30, 300_001).astype(np.float32)
    special = np.array([0.0, -0.0, np.inf, -np.inf, 1.0, 1.00390625, 1.01171875, 3.3895314e38, 1e-40, -1e-45],
                       np.float32)                      # ties to even both ways, overflow to inf, denormals
    x[: len(special)] = special
    got = grilly_core._host_round_bf16(x)
    assert got.dtype == np.uint16 and np.array_equal(got, orc.to_bf16_bits(x))
    assert grilly_core._host_round_bf16(np.array([np.nan], np.float32))[0] == 0x7FFF
    assert np.array_equal(grilly_core._host_round_bf16(x[:100]), orc.to_bf16_bits(x[:100]))   # single-thread path
