"""ctypes view of libgrilly_cuda.so, the C ABI declared in include/grilly_cuda.h.

Used by the parity tests and the benchmark to drive device-resident buffers directly; the
product path for Python users is grilly_core.  Loading fails loudly when the library is missing.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.normpath(os.path.join(_HERE, "..", "..", "lib", "libgrilly_cuda.so"))

F32, BF16, FP8_INT4 = 0, 1, 2
ROPE_NONE, ROPE_INTERLEAVED, ROPE_HALF = 0, 1, 2
MASK_NONE, MASK_KEY, MASK_BSS, MASK_BHSS = 0, 1, 2, 3
KERNEL_AUTO, KERNEL_SIMT_F32, KERNEL_TCGEN05 = 0, 1, 2
ERR_TIMEOUT = -4

# every symbol that include/grilly_cuda.h declares
SYMBOLS = [
    "grl_last_error", "grl_device_count", "grl_device_open", "grl_device_close", "grl_device_get_info",
    "grl_device_use_stream", "grl_malloc", "grl_free", "grl_host_alloc", "grl_host_free", "grl_memcpy_h2d",
    "grl_memcpy_d2h", "grl_memcpy_d2d", "grl_memset", "grl_sync", "grl_event_create", "grl_event_create_untimed", "grl_event_destroy",
    "grl_event_record", "grl_event_wait", "grl_event_sync", "grl_event_elapsed_ms", "grl_graph_begin", "grl_graph_end", "grl_graph_launch",
    "grl_graph_destroy", "grl_launch_count", "grl_cast", "grl_flash_fwd", "grl_rope", "grl_attention_mask",
    "grl_kv_append", "grl_kv_gather", "grl_swizzle_kv", "grl_kv_score_accumulate", "grl_kv_mass_accumulate", "grl_kv_evict_lowest", "grl_kv_evict_heuristic",
    "grl_kv_compact_scratch_bytes", "grl_kv_compact", "grl_evict_head_scratch_bytes", "grl_evict_head_train",
    "grl_evict_head_predict", "grl_decode_pick_splits", "grl_decode_workspace_bytes", "grl_gqa_decode",
    "grl_gqa_decode_static", "grl_lse_merge", "grl_ipc_export", "grl_ipc_import", "grl_ipc_release",
    "grl_exchange_merge", "grl_exchange_reset", "grl_device_set_wait_limits", "grl_tensor_map_cache_stats",
    "grl_rope_table_prepare", "grl_group_unique_id", "grl_group_init_rank", "grl_group_info", "grl_group_allgather",
    "grl_linear", "grl_gemm_f32", "grl_mla_concat", "grl_mla_split", "grl_group_allreduce_max_f64", "grl_group_allgather_merge", "grl_group_sync", "grl_group_destroy",
    "grl_attention_scores", "grl_softmax", "grl_attention_output", "grl_attention_backward",
]


class DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("ordinal", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("sm_count", C.c_int32), ("total_mem_bytes", C.c_int64), ("l2_bytes", C.c_int64),
                ("smem_per_block_optin", C.c_int64)]


class FlashParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
                ("in_dtype", C.c_int32), ("out_dtype", C.c_int32),
                ("batch", C.c_int32), ("heads", C.c_int32), ("seq_len", C.c_int32), ("head_dim", C.c_int32),
                ("scale", C.c_float), ("causal", C.c_int32), ("seq_lens", C.c_void_p),
                ("mask", C.c_void_p), ("mask_kind", C.c_int32),
                ("rope_mode", C.c_int32), ("rope_theta", C.c_float), ("rope_scaling", C.c_float),
                ("kernel", C.c_int32), ("status", C.c_void_p)]


class KVLayout(C.Structure):
    _fields_ = [("k_pages", C.c_void_p), ("v_pages", C.c_void_p), ("cache_dtype", C.c_int32),
                ("block_table", C.c_void_p), ("seq_lens", C.c_void_p),
                ("batch", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("page_tokens", C.c_int32), ("max_pages", C.c_int32), ("num_pages", C.c_int32), ("scales", C.c_void_p)]


class AppendParams(C.Structure):
    _fields_ = [("kv", KVLayout), ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("q_in", C.c_void_p),
                ("q_out", C.c_void_p), ("n_new", C.c_int32), ("num_q_heads", C.c_int32),
                ("rope_mode", C.c_int32), ("rope_theta", C.c_float), ("rope_scaling", C.c_float),
                ("pos_base", C.c_int32), ("update_lens", C.c_int32), ("pos_offsets", C.c_void_p)]


class KVMeta(C.Structure):
    _fields_ = [("cum_score", C.c_void_p), ("tombstone", C.c_void_p), ("relevance", C.c_void_p),
                ("evicted", C.c_void_p), ("capacity", C.c_int32)]


class ExchangeParams(C.Structure):
    _fields_ = [("local_partial", C.c_void_p), ("inbox", C.c_void_p), ("flags", C.c_void_p),
                ("peer_inbox", C.POINTER(C.c_void_p)), ("peer_flags", C.POINTER(C.c_void_p)),
                ("seq", C.c_void_p), ("out", C.c_void_p),
                ("rank", C.c_int32), ("world", C.c_int32), ("rows", C.c_int32), ("head_dim", C.c_int32),
                ("flag_slots", C.c_int32), ("low_latency", C.c_int32), ("wait_cycles", C.c_uint64)]


class DecodeParams(C.Structure):
    _fields_ = [("kv", KVLayout), ("q", C.c_void_p), ("out", C.c_void_p), ("num_q_heads", C.c_int32),
                ("scale", C.c_float), ("n_splits", C.c_int32), ("max_seq_len", C.c_int32),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("partial_out", C.c_void_p),
                ("force_simt", C.c_int32), ("scores_out", C.c_void_p), ("scores_ld", C.c_int32),
                ("exchange", C.POINTER(ExchangeParams))]


class GrlError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"[{code}] {msg}")
        self.code = code


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} not found: build it with python grilly-next_b200/build.py")
        _lib = C.CDLL(LIB_PATH)
        _lib.grl_last_error.restype = C.c_char_p
        _lib.grl_launch_count.restype = C.c_int64
        _lib.grl_sync.argtypes = [C.c_void_p, C.c_uint64]
        for n in ("grl_malloc", "grl_host_alloc"):
            getattr(_lib, n).restype = C.c_int
        _lib.grl_malloc.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]
        _lib.grl_free.argtypes = [C.c_void_p, C.c_void_p]
        _lib.grl_host_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
        _lib.grl_host_free.argtypes = [C.c_void_p]
        for n in ("grl_memcpy_h2d", "grl_memcpy_d2h", "grl_memcpy_d2d"):
            getattr(_lib, n).argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        _lib.grl_memset.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t]
        _lib.grl_cast.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_size_t]
        _lib.grl_device_use_stream.argtypes = [C.c_void_p, C.c_void_p]
        _lib.grl_event_record.argtypes = [C.c_void_p, C.c_void_p]
        _lib.grl_event_wait.argtypes = [C.c_void_p, C.c_void_p]
        _lib.grl_event_elapsed_ms.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]
        _lib.grl_event_destroy.argtypes = [C.c_void_p]
        _lib.grl_graph_begin.argtypes = [C.c_void_p]
        _lib.grl_graph_end.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        _lib.grl_graph_launch.argtypes = [C.c_void_p, C.c_void_p]
        _lib.grl_graph_destroy.argtypes = [C.c_void_p]
        _lib.grl_flash_fwd.argtypes = [C.c_void_p, C.POINTER(FlashParams)]
        _lib.grl_kv_append.argtypes = [C.c_void_p, C.POINTER(AppendParams)]
        _lib.grl_gqa_decode.argtypes = [C.c_void_p, C.POINTER(DecodeParams)]
        _lib.grl_gqa_decode_static.argtypes = [C.c_void_p, C.POINTER(DecodeParams)]
        _lib.grl_ipc_export.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        _lib.grl_ipc_import.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]
        _lib.grl_ipc_release.argtypes = [C.c_void_p, C.c_void_p]
        _lib.grl_exchange_merge.argtypes = [C.c_void_p, C.POINTER(ExchangeParams)]
        _lib.grl_exchange_reset.argtypes = [C.c_void_p, C.POINTER(ExchangeParams)]
        _lib.grl_device_set_wait_limits.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64]
        _lib.grl_tensor_map_cache_stats.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        _lib.grl_rope_table_prepare.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float]
        _lib.grl_linear.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
        _lib.grl_attention_scores.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float]
        _lib.grl_softmax.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        _lib.grl_attention_output.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5
        _lib.grl_attention_backward.argtypes = [C.c_void_p] * 10 + [C.c_int] * 4 + [C.c_float]
        _lib.grl_gemm_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        _lib.grl_mla_concat.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        _lib.grl_mla_split.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        _lib.grl_group_unique_id.argtypes = [C.c_void_p]
        _lib.grl_group_init_rank.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
        _lib.grl_group_info.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]
        _lib.grl_group_allgather.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        _lib.grl_group_allreduce_max_f64.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        _lib.grl_group_allgather_merge.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                                   C.c_uint64]
        _lib.grl_group_sync.argtypes = [C.c_void_p, C.c_uint64]
        _lib.grl_group_destroy.argtypes = [C.c_void_p]
        _lib.grl_decode_pick_splits.argtypes = [C.c_void_p, C.POINTER(DecodeParams), C.POINTER(C.c_int)]
        _lib.grl_decode_workspace_bytes.argtypes = [C.POINTER(DecodeParams), C.c_int, C.POINTER(C.c_size_t)]
        _lib.grl_kv_gather.argtypes = [C.c_void_p, C.POINTER(KVLayout), C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        _lib.grl_lse_merge.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t, C.c_int, C.c_int, C.c_int,
                                       C.c_void_p]
        _lib.grl_rope.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float,
                                  C.c_float, C.c_int, C.c_void_p, C.c_void_p]
        _lib.grl_attention_mask.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.c_float]
        _lib.grl_device_open.argtypes = [C.c_int, C.POINTER(C.c_void_p)]
        _lib.grl_device_close.argtypes = [C.c_void_p]
        _lib.grl_device_get_info.argtypes = [C.c_void_p, C.POINTER(DeviceInfo)]
        _lib.grl_event_create.argtypes = [C.POINTER(C.c_void_p)]
    return _lib


def check(rc):
    if rc != 0:
        raise GrlError(rc, lib().grl_last_error().decode())


class Device:
    """Owns a grl_device handle and offers numpy <-> HBM helpers around the raw entry points."""

    def __init__(self, ordinal=0):
        self.L = lib()
        h = C.c_void_p()
        check(self.L.grl_device_open(ordinal, C.byref(h)))
        self.h = h
        info = DeviceInfo()
        check(self.L.grl_device_get_info(self.h, C.byref(info)))
        self.info = info
        self._allocs = []

    def close(self):
        if self.h:
            for p in self._allocs:
                self.L.grl_free(self.h, p)
            self._allocs = []
            self.L.grl_device_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def malloc(self, nbytes):
        p = C.c_void_p()
        check(self.L.grl_malloc(self.h, int(nbytes), C.byref(p)))
        self._allocs.append(p)
        return p

    def free(self, p):
        self._allocs = [a for a in self._allocs if a.value != p.value]
        check(self.L.grl_free(self.h, p))

    def upload(self, arr):
        import numpy as np
        arr = np.ascontiguousarray(arr)
        p = self.malloc(max(arr.nbytes, 16))
        check(self.L.grl_memcpy_h2d(self.h, p, arr.ctypes.data_as(C.c_void_p), arr.nbytes))
        self.sync()
        return p

    def download(self, p, shape, dtype):
        import numpy as np
        out = np.empty(shape, dtype=dtype)
        check(self.L.grl_memcpy_d2h(self.h, out.ctypes.data_as(C.c_void_p), p, out.nbytes))
        self.sync()
        return out

    def upload_bf16(self, arr_f32):
        """float32 array -> device bf16 buffer through the device cast kernel."""
        src = self.upload(arr_f32.astype("float32", copy=False))
        dst = self.malloc(arr_f32.size * 2)
        check(self.L.grl_cast(self.h, src, F32, dst, BF16, arr_f32.size))
        self.sync()
        self.free(src)
        return dst

    def sync(self, timeout_ns=0):
        check(self.L.grl_sync(self.h, timeout_ns))

    def event(self):
        e = C.c_void_p()
        check(self.L.grl_event_create(C.byref(e)))
        return e

    def record(self, ev):
        check(self.L.grl_event_record(self.h, ev))

    def elapsed_ms(self, e0, e1):
        ms = C.c_float()
        check(self.L.grl_event_elapsed_ms(e0, e1, C.byref(ms)))
        return ms.value
