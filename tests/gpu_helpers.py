"""Helpers for the GPU parity tests: drive the C ABI (ctypes) with numpy inputs."""
import ctypes as C

import numpy as np

from grilly_next import cabi
from oracle import attention_oracle as orc


def flash_cabi(dev, Q, K, V, *, causal=False, seq_lens=None, mask=None, mask_kind=cabi.MASK_NONE,
               rope_mode=cabi.ROPE_NONE, rope_theta=10000.0, rope_scaling=1.0, bf16=False,
               kernel=cabi.KERNEL_AUTO, scale=0.0, out_bf16=False):
    B, H, S, D = Q.shape
    up = dev.upload_bf16 if bf16 else dev.upload
    q, k, v = up(Q), up(K), up(V)
    o = dev.malloc(Q.size * (2 if out_bf16 else 4))
    p = cabi.FlashParams()
    p.q, p.k, p.v, p.o = q, k, v, o
    p.in_dtype = cabi.BF16 if bf16 else cabi.F32
    p.out_dtype = cabi.BF16 if out_bf16 else cabi.F32
    p.batch, p.heads, p.seq_len, p.head_dim = B, H, S, D
    p.scale = scale
    p.causal = int(causal)
    keep = []
    if seq_lens is not None:
        sl = dev.upload(np.asarray(seq_lens, np.int32)); keep.append(sl)
        p.seq_lens = sl
    if mask is not None:
        m = dev.upload(np.asarray(mask, np.float32)); keep.append(m)
        p.mask, p.mask_kind = m, mask_kind
    p.rope_mode, p.rope_theta, p.rope_scaling = rope_mode, rope_theta, rope_scaling
    p.kernel = kernel
    cabi.check(dev.L.grl_flash_fwd(dev.h, C.byref(p)))
    dev.sync()
    if out_bf16:
        out = orc.from_bf16_bits(dev.download(o, Q.shape, np.uint16))
    else:
        out = dev.download(o, Q.shape, np.float32)
    for x in [q, k, v, o] + keep:
        dev.free(x)
    return out



def quant_v_offsets(P, D):
    """(P, D/2) byte offsets of the packed value bytes inside one (page, kv head) block of the quantised cache: token
    pairs, D bytes per pair, words [even token bytes 2w, 2w+1 | odd token bytes 2w, 2w+1] ordered [w % 8][w // 8]
    with the [w % 8] index XOR-swizzled by the pair index (quant_v_off in csrc/common.cuh)."""
    t = np.arange(P)[:, None]
    j = np.arange(D // 2)[None, :]
    w, G = j >> 1, D // 32
    pw = ((w & 7) ^ ((t >> 1) & 7)) * G + (w >> 3)
    return (t >> 1) * D + pw * 4 + (t & 1) * 2 + (j & 1)


class PagedCache:
    """Device-side paged cache driven through the C ABI (block table = identity allocation)."""

    def __init__(self, dev, B, Hkv, D, max_tokens, page_tokens=64, dtype=cabi.BF16, shuffle_pages=False, seed=0):
        self.dev, self.B, self.Hkv, self.D, self.P, self.dtype = dev, B, Hkv, D, page_tokens, dtype
        self.max_pages = (max_tokens + page_tokens - 1) // page_tokens
        n_pages = self.max_pages * B
        rows = n_pages * Hkv * page_tokens
        self.scales = None
        if dtype == cabi.FP8_INT4:        # one key byte, half a value byte per element, one float16 scale per 32
            self.k_pages, self.v_pages = dev.malloc(rows * D), dev.malloc(rows * D // 2)
            self.scales = dev.malloc(rows * (D // 32) * 2)
        else:
            esz = 2 if dtype == cabi.BF16 else 4
            self.k_pages, self.v_pages = dev.malloc(rows * D * esz), dev.malloc(rows * D * esz)
        table = np.arange(n_pages, dtype=np.int32)
        if shuffle_pages:
            np.random.default_rng(seed).shuffle(table)
        self.table_host = table.reshape(B, self.max_pages)
        self.block_table = dev.upload(self.table_host)
        self.seq_lens = dev.upload(np.zeros(B, np.int32))
        self.lens = np.zeros(B, np.int64)

    def layout(self):
        l = cabi.KVLayout()
        l.k_pages, l.v_pages, l.cache_dtype = self.k_pages, self.v_pages, self.dtype
        l.block_table, l.seq_lens = self.block_table, self.seq_lens
        l.batch, l.num_kv_heads, l.head_dim, l.page_tokens, l.max_pages = self.B, self.Hkv, self.D, self.P, self.max_pages
        l.num_pages = self.max_pages * self.B
        l.scales = self.scales
        return l

    def append(self, k_new, v_new, q=None, rope_mode=cabi.ROPE_NONE, theta=10000.0, scaling=1.0, pos_base=0,
               pos_offsets=None):
        """k_new/v_new (B,n,Hkv,D) float32; q (B,n,Hq,D) or None. Returns rotated q (or None)."""
        dev = self.dev
        n = k_new.shape[1]
        kd, vd = dev.upload(k_new.astype(np.float32)), dev.upload(v_new.astype(np.float32))
        p = cabi.AppendParams()
        p.kv = self.layout()
        p.k_new, p.v_new = kd, vd
        p.n_new = n
        qd = qo = None
        if q is not None:
            qd = dev.upload(q.astype(np.float32)); qo = dev.malloc(q.nbytes)
            p.q_in, p.q_out, p.num_q_heads = qd, qo, q.shape[2]
        p.rope_mode, p.rope_theta, p.rope_scaling, p.pos_base, p.update_lens = rope_mode, theta, scaling, pos_base, 1
        if pos_offsets is not None:
            p.pos_offsets = pos_offsets
        cabi.check(dev.L.grl_kv_append(dev.h, C.byref(p)))
        dev.sync()
        self.lens += n
        out = None
        if q is not None:
            out = dev.download(qo, q.shape, np.float32)
            dev.free(qd); dev.free(qo)
        dev.free(kd); dev.free(vd)
        return out

    def gather(self, b):
        T = int(self.lens[b])
        dev = self.dev
        ok, ov = dev.malloc(max(T, 1) * self.Hkv * self.D * 4), dev.malloc(max(T, 1) * self.Hkv * self.D * 4)
        l = self.layout()
        cabi.check(dev.L.grl_kv_gather(dev.h, C.byref(l), b, T, ok, ov))
        dev.sync()
        k = dev.download(ok, (T, self.Hkv, self.D), np.float32)
        v = dev.download(ov, (T, self.Hkv, self.D), np.float32)
        dev.free(ok); dev.free(ov)
        return k, v

    def decode(self, q, n_splits=0, scale=0.0, partial=False, force_simt=False):
        dev = self.dev
        B, _, Hq, D = q.shape
        qd = dev.upload(q.astype(np.float32))
        od = dev.malloc(q.nbytes)
        p = cabi.DecodeParams()
        p.kv = self.layout()
        p.q, p.out, p.num_q_heads, p.scale, p.n_splits = qd, od, Hq, scale, n_splits
        p.max_seq_len = int(self.lens.max())
        p.force_simt = int(force_simt)
        ns = C.c_int()
        cabi.check(dev.L.grl_decode_pick_splits(dev.h, C.byref(p), C.byref(ns)))
        wb = C.c_size_t()
        cabi.check(dev.L.grl_decode_workspace_bytes(C.byref(p), ns.value, C.byref(wb)))
        ws = dev.malloc(wb.value)
        p.n_splits, p.workspace, p.workspace_bytes = ns.value, ws, wb.value
        pd = None
        rows = B * Hq
        if partial:
            pd = dev.malloc(rows * (D + 2) * 4)
            p.partial_out = pd
        cabi.check(dev.L.grl_gqa_decode(dev.h, C.byref(p)))
        dev.sync()
        if partial:
            out = dev.download(pd, (rows * (D + 2),), np.float32)
            dev.free(pd)
        else:
            out = dev.download(od, q.shape, np.float32)
        for x in (qd, od, ws):
            dev.free(x)
        self.last_splits = ns.value
        return out
