// GQA decode over the paged bf16 cache, head_dim 128 or 64, pages of 64, 32 or 16 tokens: the fast path.
//
// Replaces shaders/gqa-attention.glsl:34-130 like decode_splitkv.cu, for the geometry of the
// benchmark configurations.  One CTA owns (split, kv head, sequence); a producer warp streams
// whole (page, kv head) slabs -- 16 KiB of K and 16 KiB of V, each contiguous in HBM -- into a
// 3-stage shared-memory ring with TMA (128-byte swizzle, mbarrier complete_tx); four compute
// warps each take 16 of the page's 64 tokens and run QK^T and PV on tensor cores
// (mma.sync m16n8k16, the group's query heads padded to the 16-row operand, q split into
// bf16 hi+lo so that its fp32 precision survives), with a private fp32 online softmax in the
// exp2 domain.  K and V cross HBM -> SM exactly once; the four warps' partials are merged in
// shared memory and leave the CTA as (O un-normalised, m, l), the layout lse_merge_kernel reads.
//
// The same kernel, instantiated for the quantised cache (GRL_FP8_INT4: FP8-E4M3 keys, INT4 values, one float16 scale
// per 32 key elements, cpp/src/ops/kv_cache.cpp:272-399 and :500-577), streams 12.5 KiB per (page, kv head) instead
// of 32 and dequantises in registers: key bytes become f16 by three integer operations per pair (every code is an
// exact f16 once divided by 256), the four scale groups of a head accumulate separately and are combined with 1/scale per
// token; value nibbles become f16 by one logic operation and one subtraction per pair (1024 + n or 64 + n in the
// mantissa, minus the offset and the code's bias), with 1/scale folded into P.  The contraction indices of both
// products are permuted so that every operand register is a plain 32-bit piece of what was loaded.
#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace grl {
namespace dmma {

constexpr int P = 64;               // tokens per ring stage: one 64-token page, or two / four smaller ones side by side
constexpr int D = 128;              // head_dim of the quantised instance (the bf16 instances carry theirs as HD)
constexpr int kThreads = 160;       // 4 compute warps + 1 producer warp
// The shared-memory ring of the two instances.  After the ring: 128 bytes of barriers and flags, 1 KiB of per-warp
// scratch (1/scale of a warp's 16 tokens x 4 groups), 1 KiB of slack for the 1024-byte alignment of the ring.
template <bool QUANT, int HD> struct Ring {
    static constexpr int SLAB = P * HD * 2;             // 64 tokens of K (or V) for one kv head: 16 KiB at head_dim 128
    static constexpr int STAGE = 2 * SLAB;              // K then V
    static constexpr int NST = 3 * 128 / HD;            // ring stages: 96 KiB in flight per CTA
};
constexpr int QK_BYTES = P * D;          // 8 KiB of key bytes per 64 tokens of a kv head
constexpr int QV_BYTES = P * D / 2;      // 4 KiB of packed value nibbles
constexpr int QS_BYTES = P * (D / 32) * 2;   // 512 B of float16 scales
template <> struct Ring<true, 128> {
    static constexpr int SLAB = 0;
    static constexpr int NST = 6;
    static constexpr int STAGE = 13 * 1024;  // keys at 0, values at 8 KiB, scales at 12 KiB
};
template <bool QUANT, int HD> struct Smem {
    static constexpr int BAR = Ring<QUANT, HD>::NST * Ring<QUANT, HD>::STAGE;
    static constexpr int TOTAL = BAR + 128 + 1024 + 1024;
};
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kEmpty = -1e30f;

struct Args {
    const int32_t* block_table;
    const int32_t* seq_lens;
    const uint8_t* v_q;         // quantised cache: the value pool (plain bulk copies; the key pool goes through tmK)
    const uint16_t* scales;     // quantised cache: float16 bit patterns, (rows, D/32)
    const float* q;
    float* part;
    float* out;
    int32_t* status;
    int B, Hq, Hkv, max_pages, n_splits, group;
    int page, ppt;          // tokens per page (64, 32 or 16) and pages per 64-token stage
    float scale;
    int direct;
    // fused merge: the last CTA of a (sequence, kv head) to arrive merges the head's splits
    int fuse;               // 0: leave the splits to lse_merge_kernel
    int32_t* counters;      // arrival counters, zero between launches; [kDoneSlot] counts finished heads
    float* partial_out;     // != NULL: merged rows leave un-normalised as [O | m | l]
    float* scores_out;      // != NULL: (B*Hq, scores_ld) scaled scores, natural-log domain
    int scores_ld;
    PeerExchange x;         // x.world > 1: the merged rows are exchanged with the peers and merged again
    long long wait_limit;   // cycle budget of every mbarrier wait
};
constexpr int kDoneSlot = grl_device::kCounterSlots;
constexpr int kMaxFusedSplits = 256;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// The same test, but the thread may stay suspended in hardware for up to hint_ns while the phase is incomplete: a
// waiter that is far ahead of what it waits for then takes no issue slots.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D += A * B with A rows 8..15 all zero (a1 = a3 = 0): the query heads of one GQA group fill rows 0..7.
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
}
// Plain (untiled) bulk copy global -> shared, 16-byte aligned on both sides, completing on an mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar) : "memory");
}
// f16 form of the same product.  Rows 8..15 of the accumulator (d[2], d[3]) multiply the zero half of A: they stay
// whatever they were and are never read, but they stay in place -- the instruction wants four consecutive registers,
// and carving two live ones out of the quad costs a move and a clear around every product.
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
}
// All sixteen rows of A live (the transposed value product: rows are head_dim elements, columns query heads).
__device__ __forceinline__ void mma_f16_full(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The first product of a chain: C is zero (no register needs clearing for it).
__device__ __forceinline__ void mma_f16_first(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%9,%9,%9,%9};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// FP8-E4M3 codes to f16x2 by integer operations (the conversion instruction runs on the slow special-function
// pipe).  A code s eeee mmm becomes the f16 s 0eeee mmm0000000, which is the code's value (the reference's decoder,
// kv_cache.cpp:540-552: 2^(e-7) (1 + m/8), or m 2^-9 for e = 0) divided by 256, denormals included; the factor is
// folded into q.  Bytes (0, 2) of a word make one register, bytes (1, 3) the other: the byte permute puts each code
// under a copy of its sign, the shift brings exponent and mantissa into place and the sign to bit 15, the mask
// clears what the shift dragged along.
__device__ __forceinline__ uint32_t prmt(uint32_t w, uint32_t selector) {   // a selector digit >= 8 replicates the byte's sign
    uint32_t r;
    asm("prmt.b32 %0, %1, %1, %2;" : "=r"(r) : "r"(w), "r"(selector));
    return r;
}
__device__ __forceinline__ uint32_t e4m3_pair02_f16x2(uint32_t w) { return (prmt(w, 0xA280u) << 7) & 0xBF80BF80u; }
__device__ __forceinline__ uint32_t e4m3_pair13_f16x2(uint32_t w) { return (prmt(w, 0xB391u) << 7) & 0xBF80BF80u; }
// Value codes to f16x2 (low half: even token of the pair, high half: odd token): the nibble is placed in the mantissa of
// 1024 (bits 0-3) or of 64 (bits 4-7), and the offset plus the code's bias of 8 is subtracted, which is exact in f16.
__device__ __forceinline__ uint32_t nib_lo(uint32_t w) {
    const uint32_t v = (w & 0x000F000Fu) | 0x64006400u, off = 0x64086408u;    // 1032, 1032
    __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&v), *reinterpret_cast<const __half2*>(&off));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) {
    const uint32_t v = (w & 0x00F000F0u) | 0x54005400u, off = 0x54805480u;    // 72, 72
    __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&v), *reinterpret_cast<const __half2*>(&off));
    return *reinterpret_cast<uint32_t*>(&r);
}
// 1/scale from the stored float16 bit pattern, as the reference's decode forms it (kv_cache.cpp:517-533): bits moved
// into a float32, not converted; a scale that is not positive gives 1.
__device__ __forceinline__ float inv_scale_bits(uint32_t h) {
    const uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x03FFu;
    const float sc = e == 0 ? (float)m * 5.9604644775390625e-08f
                            : __uint_as_float(((h & 0x8000u) << 16) | ((e + 112u) << 23) | (m << 13));
    return sc > 0.f ? __fdividef(1.0f, sc) : 1.0f;     // within an ulp of the reference's quotient
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct Ctx {
    uint32_t bars;
    volatile int* abort;
    int32_t* status;
    long long limit;
};
// relaxed: the waiter is ahead of its consumers by the whole ring (the producer lane): it waits suspended instead of
// competing for issue slots with the compute warp that shares its scheduler.
__device__ __forceinline__ bool wait_bar(const Ctx& c, int bar, uint32_t parity, bool relaxed = false) {
    const uint32_t addr = c.bars + bar * 8;
    if (mbar_try_wait(addr, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (relaxed ? mbar_try_wait_suspend(addr, parity, 20000u) : mbar_try_wait(addr, parity)) return true;
        if (*c.abort) return false;
        if (clock64() - t0 > c.limit) {
            *c.abort = 1;
            if (c.status && atomicCAS(c.status, 0, GRL_ERR_TIMEOUT) == 0) {
                c.status[1] = (2 << 28) | bar;
                c.status[2] = blockIdx.x;
                c.status[3] = blockIdx.y | (blockIdx.z << 16);
            }
            return false;
        }
    }
}

// byte offset inside a slab of element (token row, column d): two 64-column halves, 128-byte swizzle
__device__ __forceinline__ uint32_t slab_off(int row, int d) {
    return (uint32_t)((d >> 6) * (P * 128) + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4));
}

template <bool QUANT, int HD>
__global__ void __launch_bounds__(kThreads, 2)
decode_mma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const Args a) {
    static_assert(HD == 128 || (HD == 64 && !QUANT), "head_dim 128, or 64 over the bf16 cache");
    constexpr int D = HD;
    constexpr int NST = Ring<QUANT, HD>::NST, STAGE = Ring<QUANT, HD>::STAGE, SMEM_BAR = Smem<QUANT, HD>::BAR;
    constexpr int SLAB = Ring<QUANT, HD>::SLAB;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw_addr);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int len = max(0, min(a.seq_lens[b], a.max_pages * a.page));   // never past the block table
    const int n_pages = (len + P - 1) / P;        // 64-token stages ("pages" below)
    const int pps = (n_pages + a.n_splits - 1) / a.n_splits;
    const int p_begin = min(n_pages, split * pps), p_end = min(n_pages, (split + 1) * pps);
    const int32_t* bt = a.block_table + (size_t)b * a.max_pages;

    int* abort_flag = reinterpret_cast<int*>(smem + SMEM_BAR + 2 * NST * 8);
    Ctx ctx{base + SMEM_BAR, abort_flag, a.status, a.wait_limit};
    auto full = [&](int s) { return ctx.bars + (uint32_t)s * 8u; };
    auto empty = [&](int s) { return ctx.bars + (uint32_t)(NST + s) * 8u; };
    if (tid == 0) {
        for (int s = 0; s < NST; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const int g = lane >> 2, t4 = lane & 3;      // mma row / column-pair index of this lane
    float o[D / 8][4];
    float m_run = kEmpty, l_run = 0.f;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

    if (warp == 4) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmK)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmV)) : "memory");
            int issued = 0;
            for (int p = p_begin; p < p_end; ++p) {
                const int i = p - p_begin, s = i % NST, it = i / NST;
                if (it > 0 && !wait_bar(ctx, NST + s, (it - 1) & 1, true)) break;
                // the pages of this stage that hold tokens of the sequence (all of them but in the last stage); rows of
                // the stage that no copy fills keep what they held: their tokens are past the length and masked
                const int np = min(a.ppt, (len - p * P + a.page - 1) / a.page);
                const uint32_t dst = base + (uint32_t)s * STAGE;
                if constexpr (QUANT) {
                    mbar_expect_tx(full(s), (uint32_t)np * a.page * (D + D / 2 + D / 16));
                    for (int j = 0; j < np; ++j) {
                        const int blk = bt[p * a.ppt + j] * a.Hkv + kvh;
                        // rows of 128 key bytes under the 128-byte swizzle; a page's value and scale blocks are contiguous
                        tma_load_2d(dst + j * a.page * 128, &tmK, 0, blk * a.page, full(s));
                        bulk_load(dst + QK_BYTES + j * a.page * (D / 2), a.v_q + (size_t)blk * a.page * (D / 2), a.page * (D / 2), full(s));
                        bulk_load(dst + QK_BYTES + QV_BYTES + j * a.page * (D / 16), a.scales + (size_t)blk * a.page * (D / 32),
                                  a.page * (D / 16), full(s));
                    }
                } else {
                    mbar_expect_tx(full(s), (uint32_t)np * a.page * D * 4);
                    for (int j = 0; j < np; ++j) {
                        const int row0 = (bt[p * a.ppt + j] * a.Hkv + kvh) * a.page;
#pragma unroll
                        for (int c0 = 0; c0 < D; c0 += 64) {        // 64-column boxes (128 bytes: the swizzle span)
                            tma_load_2d(dst + (c0 / 64) * (P * 128) + j * a.page * 128, &tmK, c0, row0, full(s));
                            tma_load_2d(dst + SLAB + (c0 / 64) * (P * 128) + j * a.page * 128, &tmV, c0, row0, full(s));
                        }
                    }
                }
                issued = i + 1;
            }
            if (*ctx.abort) {   // copies already issued must land before the shared memory is released
                const long long t0 = clock64();
                for (int i = max(0, issued - NST); i < issued; ++i)
                    while (!mbar_try_wait(full(i % NST), (i / NST) & 1) && clock64() - t0 < ctx.limit) {}
            }
        }
    } else if constexpr (QUANT) {
        // ------------------------------------------------------------------ compute over the quantised cache
        // Element permutation of the two products.  QK^T: k-step (grp, w) of lane (g, t4) covers elements
        // 32 grp + 8 t4 + 4 w + {0,2 | 1,3} = one 32-bit word of key bytes.  PV runs transposed (rows elements,
        // columns heads): row g | g + 8 of tile (grp, j) is element 32 grp + 4 g + 2 j | + 1, and the k index
        // pairs (2 t4, 2 t4 + 1 | + 8) are the token pairs (8 warp + 2 t4 | + 1) of the value block (quant_v_off).
        // Tokens: column n of score tile nt is token 2 n + nt of the warp's 16 (so that a half-warp's key loads hit
        // all banks once), and a lane's four scores are the four consecutive tokens 4 t4 .. 4 t4 + 3.
        const int qh0 = kvh * a.group;
        uint32_t qf[8][2];
        {
            const float sc = a.scale * kLog2e * 256.f;      // the key registers hold code / 256
            const float* qrow = a.q + ((size_t)b * a.Hq + qh0 + g) * D;
            const bool live = g < a.group;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live) v = *reinterpret_cast<const float4*>(qrow + 32 * (ks >> 1) + 8 * t4 + 4 * (ks & 1));
                qf[ks][0] = pack_f16(v.x * sc, v.z * sc);      // with the key codes of bytes 0 and 2 of the word
                qf[ks][1] = pack_f16(v.y * sc, v.w * sc);      // bytes 1 and 3
            }
        }
        float* inv_w = reinterpret_cast<float*>(smem + SMEM_BAR + 128) + warp * 64;   // [16 tokens][4 groups]
        bool ok = true;
        for (int p = p_begin; p < p_end && ok; ++p) {
            const int i = p - p_begin, s = i % NST, it = i / NST;
            ok = __all_sync(0xffffffffu, wait_bar(ctx, s, it & 1));
            if (!ok) break;
            const uint8_t* kst = smem + s * STAGE;
            const uint8_t* vst = kst + QK_BYTES;
            const uint8_t* sst = vst + QV_BYTES;
            const int tok0 = p * P + 16 * warp;
            if (tok0 < len) {
                {   // 1/scale of this warp's tokens: lane -> token lane/2, groups 2*(lane&1) and the next; 0 past the end
                    const int tl = lane >> 1, g2 = (lane & 1) * 2;
                    const uint32_t hh = *reinterpret_cast<const uint32_t*>(sst + ((16 * warp + tl) * 4 + g2) * 2);
                    const bool live_t = tok0 + tl < len;
                    *reinterpret_cast<float2*>(inv_w + tl * 4 + g2) =
                        make_float2(live_t ? inv_scale_bits(hh & 0xFFFFu) : 0.f, live_t ? inv_scale_bits(hh >> 16) : 0.f);
                }
                __syncwarp();
                float inv[2][2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float4 v = *reinterpret_cast<const float4*>(inv_w + (4 * t4 + 2 * e + nt) * 4);
                        inv[nt][e][0] = v.x; inv[nt][e][1] = v.y; inv[nt][e][2] = v.z; inv[nt][e][3] = v.w;
                    }
                // ---- S = q K^T for 16 tokens, one accumulator per scale group, combined with 1/scale
                float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int row = 16 * warp + 2 * g + nt;     // column n of tile nt is token 2 n + nt of the slice
#pragma unroll
                    for (int grp = 0; grp < 4; ++grp) {
                        const int chunk = (2 * grp + (t4 >> 1)) ^ (row & 7);
                        const uint2 kb = *reinterpret_cast<const uint2*>(kst + row * 128 + chunk * 16 + (t4 & 1) * 8);
                        float c[4];
                        mma_f16_first(c, qf[2 * grp][0], qf[2 * grp][1], e4m3_pair02_f16x2(kb.x), e4m3_pair13_f16x2(kb.x));
                        mma_f16(c, qf[2 * grp + 1][0], qf[2 * grp + 1][1], e4m3_pair02_f16x2(kb.y), e4m3_pair13_f16x2(kb.y));
                        sacc[nt][0] = fmaf(c[0], inv[nt][0][grp], sacc[nt][0]);
                        sacc[nt][1] = fmaf(c[1], inv[nt][1][grp], sacc[nt][1]);
                    }
                }
                // ---- online softmax for head row g.  Only the last tile of a sequence has tokens past its end: they
                // get the "empty" score there, so the common path carries no per-token predicate
                if (tok0 + 16 > len) {
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e)
                            if (tok0 + 4 * t4 + 2 * e + nt >= len) sacc[nt][e] = kEmpty;
                }
                if (a.scores_out && g < a.group) {
                    float* srow = a.scores_out + ((size_t)b * a.Hq + qh0 + g) * a.scores_ld + tok0 + 4 * t4;
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e)
                            if (tok0 + 4 * t4 + 2 * e + nt < len) srow[2 * e + nt] = sacc[nt][e] * 0.6931471805599453f;
                }
                float mx = fmaxf(fmaxf(sacc[0][0], sacc[0][1]), fmaxf(sacc[1][0], sacc[1][1]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run, mx);
                const float corr = ex2(m_run - m_new);
                float pv[2][2];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) pv[nt][e] = ex2(sacc[nt][e] - m_new);    // 0 for an "empty" score
                const float ps = (pv[0][0] + pv[0][1]) + (pv[1][0] + pv[1][1]);
                l_run = l_run * corr + ps;
                m_run = m_new;
                if (__any_sync(0xffffffffu, corr != 1.f)) {
                    // the accumulator columns of this lane are heads 2 t4 and 2 t4 + 1: their factors live in other lanes
                    const float ca = __shfl_sync(0xffffffffu, corr, 8 * t4), cb = __shfl_sync(0xffffffffu, corr, 8 * t4 + 4);
#pragma unroll
                    for (int n = 0; n < 8; ++n) { o[n][0] *= ca; o[n][2] *= ca; o[n][1] *= cb; o[n][3] *= cb; }
                }
                // ---- O^T += V^T (P / scale)^T: rows are head_dim elements, columns heads, so all sixteen rows of the
                // product work and P is used as it comes out of S (pairs of tokens per head).  The two token pairs of
                // this lane, 16 value bytes (all four groups) each
                // (this lane's tokens 4 t4 .. 4 t4 + 3 of the slice: pairs 2 t4 and 2 t4 + 1; the 16-byte pieces of a
                // pair are stored XOR-swizzled by the pair index, which keeps the eight lanes of a quarter-warp on
                // different banks)
                const int pr = 8 * warp + 2 * t4;
                const uint4 va = *reinterpret_cast<const uint4*>(vst + pr * 128 + ((g ^ (pr & 7)) << 4));
                const uint4 vb = *reinterpret_cast<const uint4*>(vst + (pr + 1) * 128 + ((g ^ ((pr + 1) & 7)) << 4));
                const uint32_t xa[4] = {va.x, va.y, va.z, va.w}, xb[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
                for (int grp = 0; grp < 4; ++grp) {
                    // B of the value product: k pairs are (even, odd) tokens of a pair = (tile 0, tile 1) of a column
                    const uint32_t pa0 = pack_f16(pv[0][0] * inv[0][0][grp], pv[1][0] * inv[1][0][grp]);
                    const uint32_t pa2 = pack_f16(pv[0][1] * inv[0][1][grp], pv[1][1] * inv[1][1][grp]);
                    const uint32_t x = xa[grp], y = xb[grp], xs = x >> 8, ys = y >> 8;
                    // nibble n of the even | odd token of a pair as f16x2: 1024 + n (low nibble) or 64 + n (high
                    // nibble) by one logic operation, then n - 8 exactly by one subtraction
                    // rows g | g + 8 of tile (grp, j) are elements 32 grp + 4 g + 2 j | + 1
                    mma_f16_full(o[2 * grp], nib_lo(x), nib_hi(x), nib_lo(y), nib_hi(y), pa0, pa2);
                    mma_f16_full(o[2 * grp + 1], nib_lo(xs), nib_hi(xs), nib_lo(ys), nib_hi(ys), pa0, pa2);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty(s));
        }
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    } else {
        // ------------------------------------------------------------------ compute: tokens [16*warp, 16*warp+16) of every page
        const int qh0 = kvh * a.group;
        // A fragments of q (rows = heads of the group, zero beyond), pre-scaled into the exp2 domain, hi + lo bf16
        uint32_t qhi[D / 16][2], qlo[D / 16][2];
        {
            const float sc = a.scale * kLog2e;
            const float* qrow = a.q + ((size_t)b * a.Hq + qh0 + g) * D;
            const bool live = g < a.group;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int d = 16 * ks + 8 * h + 2 * t4;
                    float x0 = 0.f, x1 = 0.f;
                    if (live) { const float2 v = *reinterpret_cast<const float2*>(qrow + d); x0 = v.x * sc; x1 = v.y * sc; }
                    const float h0 = __bfloat162float(__float2bfloat16_rn(x0)), h1 = __bfloat162float(__float2bfloat16_rn(x1));
                    qhi[ks][h] = pack_bf16(h0, h1);
                    qlo[ks][h] = pack_bf16(x0 - h0, x1 - h1);
                }
            }
        }
        bool ok = true;
        for (int p = p_begin; p < p_end && ok; ++p) {
            const int i = p - p_begin, s = i % NST, it = i / NST;
            ok = __all_sync(0xffffffffu, wait_bar(ctx, s, it & 1));
            if (!ok) break;
            const uint32_t kbase = base + (uint32_t)s * STAGE, vbase = kbase + SLAB;
            const int tok0 = p * P + 16 * warp;                 // first token of this warp's slice
            if (tok0 < len) {
                if (tok0 + 16 > len) {
                    // rows past the end of the sequence hold whatever the page held: zero them in V
                    // (their probabilities are zero, but 0 * NaN is not)
                    for (int c = lane; c < 16 * (D / 8); c += 32) {
                        const int r = 16 * warp + c / (D / 8), ch = c % (D / 8);
                        if (p * P + r >= len)
                            *reinterpret_cast<uint4*>(smem + s * STAGE + SLAB + slab_off(r, ch * 8)) = make_uint4(0, 0, 0, 0);
                    }
                    __syncwarp();
                }
                // ---- S = q K^T for 16 tokens: two 8-token n-tiles
                float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                const int mat = lane >> 3;
                {
                    const int row = 16 * warp + (lane & 7) + ((mat >> 1) << 3);
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        uint32_t kb[4];
                        ldmatrix_x4(kbase + slab_off(row, 16 * ks + ((mat & 1) << 3)), kb);
                        mma_16816(sacc[0], qhi[ks][0], qhi[ks][1], kb[0], kb[1]);
                        mma_16816(sacc[1], qhi[ks][0], qhi[ks][1], kb[2], kb[3]);
                        mma_16816(sacc[0], qlo[ks][0], qlo[ks][1], kb[0], kb[1]);
                        mma_16816(sacc[1], qlo[ks][0], qlo[ks][1], kb[2], kb[3]);
                    }
                }
                // ---- online softmax for head row g (lanes with the same g share the row)
                float mx = kEmpty;
                bool valid[2][2];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        valid[nt][e] = tok0 + nt * 8 + 2 * t4 + e < len;
                        if (valid[nt][e]) mx = fmaxf(mx, sacc[nt][e]);
                    }
                if (a.scores_out && g < a.group) {      // what H2O eviction accumulates; off on the plain path
                    float* srow = a.scores_out + ((size_t)b * a.Hq + qh0 + g) * a.scores_ld + tok0 + 2 * t4;
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e)
                            if (valid[nt][e]) srow[nt * 8 + e] = sacc[nt][e] * 0.6931471805599453f;
                }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run, mx);
                const float corr = ex2(m_run - m_new);
                float pv[2][2], ps = 0.f;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        pv[nt][e] = valid[nt][e] ? ex2(sacc[nt][e] - m_new) : 0.f;
                        ps += pv[nt][e];
                    }
                l_run = l_run * corr + ps;
                m_run = m_new;
                if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
                    for (int n = 0; n < D / 8; ++n) { o[n][0] *= corr; o[n][1] *= corr; }
                }
                const uint32_t pa0 = pack_bf16(pv[0][0], pv[0][1]), pa2 = pack_bf16(pv[1][0], pv[1][1]);
                // ---- O += P V: 16 tokens x head_dim, two 8-wide d n-tiles per ldmatrix
                {
                    const int row = 16 * warp + (lane & 7) + ((mat & 1) << 3);
#pragma unroll
                    for (int dn = 0; dn < D / 16; ++dn) {
                        uint32_t vb[4];
                        ldmatrix_x4_trans(vbase + slab_off(row, 16 * dn + ((mat >> 1) << 3)), vb);
                        mma_16816(o[2 * dn], pa0, pa2, vb[0], vb[1]);
                        mma_16816(o[2 * dn + 1], pa0, pa2, vb[2], vb[3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty(s));
        }
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    }

    // ---- merge the four warps' partials (the ring is idle now: reuse it)
    __syncthreads();
    float* sm_o = reinterpret_cast<float*>(smem);                 // [4 warps][8 heads][128]
    float* sm_m = sm_o + 4 * 8 * D;                               // [4][8]
    float* sm_l = sm_m + 32;
    if (warp < 4) {
        if constexpr (QUANT) {
            // tile (grp, j): columns are heads 2 t4 | 2 t4 + 1, rows elements 32 grp + 4 g + 2 j | + 1
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const int d0 = 32 * (n >> 1) + 4 * g + 2 * (n & 1);
                *reinterpret_cast<float2*>(&sm_o[(warp * 8 + 2 * t4) * D + d0]) = make_float2(o[n][0], o[n][2]);
                *reinterpret_cast<float2*>(&sm_o[(warp * 8 + 2 * t4 + 1) * D + d0]) = make_float2(o[n][1], o[n][3]);
            }
        } else {
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
                *reinterpret_cast<float2*>(&sm_o[(warp * 8 + g) * D + n * 8 + 2 * t4]) = make_float2(o[n][0], o[n][1]);
        }
        if (t4 == 0) { sm_m[warp * 8 + g] = m_run; sm_l[warp * 8 + g] = l_run; }
    }
    __syncthreads();
    const int rows = a.B * a.Hq;
    for (int idx = tid; idx < a.group * D; idx += kThreads) {
        const int h = idx / D, d = idx % D;
        float mt = kEmpty;
#pragma unroll
        for (int w = 0; w < 4; ++w) mt = fmaxf(mt, sm_m[w * 8 + h]);
        float ov = 0.f, lt = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float wgt = ex2(sm_m[w * 8 + h] - mt);
            ov = fmaf(wgt, sm_o[(w * 8 + h) * D + d], ov);
            lt = fmaf(wgt, sm_l[w * 8 + h], lt);
        }
        const int row = b * a.Hq + kvh * a.group + h;
        if (a.direct) {
            a.out[(size_t)row * D + d] = lt > 0.f ? ov / lt : 0.f;
        } else {
            float* part = a.part + (size_t)split * rows * (D + 2);
            part[(size_t)row * D + d] = ov;
            if (d == 0) {
                part[(size_t)rows * D + row] = mt * 0.6931471805599453f;   // back to the natural-log domain
                part[(size_t)rows * D + rows + row] = lt;
            }
        }
    }
    if (a.direct || !a.fuse) return;

    // ---- fused merge: whoever arrives last for this (sequence, kv head) combines its splits
    __threadfence();
    __syncthreads();
    int* s_flag = reinterpret_cast<int*>(smem + SMEM_BAR + 2 * NST * 8 + 8);
    const int slot = b * a.Hkv + kvh;
    if (tid == 0) {
        const int t = atomicAdd(&a.counters[slot], 1);
        const int last = (t == a.n_splits - 1);
        if (last) a.counters[slot] = 0;          // nobody else touches the slot before the next launch
        *s_flag = last;
    }
    __syncthreads();
    if (!*s_flag) return;
    __threadfence();
    float* sm_w = reinterpret_cast<float*>(smem);              // [8 heads][256 splits]: m, then the weights
    float* sm_ls = sm_w + 8 * kMaxFusedSplits;                 // [8][256]: l of every split
    float* sm_mt = sm_ls + 8 * kMaxFusedSplits;                // [8] max (natural log), [8] l
    float* sm_res = sm_mt + 16;                                // [8][128] merged un-normalised rows
    const size_t pstride = (size_t)rows * (D + 2);
    const int row0 = b * a.Hq + kvh * a.group;
    for (int idx = tid; idx < a.group * a.n_splits; idx += kThreads) {
        const int h = idx / a.n_splits, s = idx % a.n_splits;
        const float* ml = a.part + (size_t)s * pstride + (size_t)rows * D + row0 + h;
        sm_w[h * kMaxFusedSplits + s] = __ldcg(ml);
        sm_ls[h * kMaxFusedSplits + s] = __ldcg(ml + rows);
    }
    __syncthreads();
    for (int h = warp; h < a.group; h += kThreads / 32) {
        float mt = kEmpty;
        for (int s = lane; s < a.n_splits; s += 32) mt = fmaxf(mt, sm_w[h * kMaxFusedSplits + s]);
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, sh));
        float lt = 0.f;
        for (int s = lane; s < a.n_splits; s += 32) {
            const float w = __expf(sm_w[h * kMaxFusedSplits + s] - mt);
            sm_w[h * kMaxFusedSplits + s] = w;
            lt = fmaf(w, sm_ls[h * kMaxFusedSplits + s], lt);
        }
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) lt += __shfl_xor_sync(0xffffffffu, lt, sh);
        if (lane == 0) { sm_mt[h] = mt; sm_mt[8 + h] = lt; }
    }
    __syncthreads();
    const PeerExchange& x = a.x;
    const bool exchange = x.world > 1;
    // Merged un-normalised rows into shared memory.  A thread owns two columns of one head and has the loads of
    // up to 16 splits in flight: the partials sit in L2, so the chain is latency, not bandwidth.
    for (int c = tid; c < a.group * (D / 2); c += kThreads) {
        const int h = c / (D / 2), d2 = c % (D / 2);
        const float* col = a.part + (size_t)(row0 + h) * D + 2 * d2;     // 8-byte aligned: D and pstride are even
        float2 acc = make_float2(0.f, 0.f);
        for (int s0 = 0; s0 < a.n_splits; s0 += 16) {
            float2 v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (s0 + j < a.n_splits) v[j] = __ldcg(reinterpret_cast<const float2*>(col + (size_t)(s0 + j) * pstride));
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (s0 + j < a.n_splits) {
                    const float w = sm_w[h * kMaxFusedSplits + s0 + j];
                    acc.x = fmaf(w, v[j].x, acc.x);
                    acc.y = fmaf(w, v[j].y, acc.y);
                }
        }
        *reinterpret_cast<float2*>(&sm_res[h * D + 2 * d2]) = acc;
    }
    __syncthreads();
    if (!exchange) {
        for (int idx = tid; idx < a.group * D; idx += kThreads) {
            const int h = idx / D;
            const float lt = sm_mt[8 + h];
            if (a.partial_out) a.partial_out[(size_t)row0 * D + idx] = sm_res[idx];
            else a.out[(size_t)row0 * D + idx] = lt > 0.f ? sm_res[idx] / lt : 0.f;
        }
        if (a.partial_out && tid < a.group) {
            a.partial_out[(size_t)rows * D + row0 + tid] = sm_mt[tid];
            a.partial_out[(size_t)rows * D + rows + row0 + tid] = sm_mt[8 + tid];
        }
        return;
    }

    // ---- cross-GPU exchange of this head's rows.  An item is one float of the head's part: group*D values of
    // O, then group maxima, then group sums; every 8-byte inbox element carries the step number next to the
    // value, so a reader that sees the number sees the value: neither a fence nor a flag between the peers.
    const unsigned int e = *x.seq + 1;
    const int par = e & 1;
    const int n_items = a.group * (D + 2);
    auto item_off = [&](int i) -> size_t {       // offset of item i inside a part laid out [O | m | l]
        if (i < a.group * D) return (size_t)row0 * D + i;
        i -= a.group * D;
        return i < a.group ? (size_t)rows * D + row0 + i : (size_t)rows * D + rows + row0 + (i - a.group);
    };
    auto item_val = [&](int i) -> float {
        if (i < a.group * D) return sm_res[i];
        i -= a.group * D;
        return i < a.group ? sm_mt[i] : sm_mt[8 + (i - a.group)];
    };
    const int total = (x.world - 1) * n_items;
    for (int it = tid; it < total; it += kThreads) {
        const int pi = it / n_items, i = it - pi * n_items, r = pi + (pi >= x.rank);
        reinterpret_cast<uint2*>(x.peer_inbox[r])[((size_t)par * x.world + x.rank) * pstride + item_off(i)] =
            make_uint2(__float_as_uint(item_val(i)), e);
    }
    // Poll the peers' items of this head, all peers side by side: a thread issues the loads of up to 16 missing
    // items before it examines any, so a round is one trip to L2 whatever the number of peers.
    float* sm_in = sm_res + 8 * D;                 // [world-1][n_items]
    constexpr int kChunk = 16;
    bool ok = true;
    const long long t0 = clock64();
    for (int base_it = 0; base_it < total && ok; base_it += kChunk * kThreads) {
        unsigned int pending = 0;
        unsigned int off[kChunk];                  // element offset inside the local inbox
#pragma unroll
        for (int j = 0; j < kChunk; ++j) {
            const int it = base_it + j * kThreads + tid;
            off[j] = 0;
            if (it < total) {
                const int pi = it / n_items, i = it - pi * n_items, r = pi + (pi >= x.rank);
                off[j] = (unsigned int)(((size_t)par * x.world + r) * pstride + item_off(i));
                pending |= 1u << j;
            }
        }
        const uint2* inbox = reinterpret_cast<const uint2*>(x.inbox);
        while (pending) {
            uint2 v[kChunk];
#pragma unroll
            for (int j = 0; j < kChunk; ++j)
                if (pending >> j & 1u) v[j] = ld_pair_volatile(inbox + off[j]);
#pragma unroll
            for (int j = 0; j < kChunk; ++j)
                if ((pending >> j & 1u) && v[j].y == e) {
                    sm_in[base_it + j * kThreads + tid] = __uint_as_float(v[j].x);
                    pending &= ~(1u << j);
                }
            if (pending && clock64() - t0 > x.wait_cycles) {
                ok = false;
                if (a.status && atomicCAS(a.status, 0, GRL_ERR_TIMEOUT) == 0) {
                    const int it = base_it + (__ffs(pending) - 1) * kThreads + tid, pi = it / n_items;
                    a.status[1] = (3 << 28) | (pi + (pi >= x.rank));     // a peer that did not post
                    a.status[2] = (int)e;
                    a.status[3] = x.rank;
                }
                break;
            }
        }
    }
    ok = __syncthreads_and(ok);                    // the whole CTA agrees: no row is written after a timeout
    if (ok) {
        for (int idx = tid; idx < a.group * D; idx += kThreads) {
            const int h = idx / D;
            float mt = sm_mt[h];
            for (int pi = 0; pi < x.world - 1; ++pi) mt = fmaxf(mt, sm_in[pi * n_items + a.group * D + h]);
            const float w0 = __expf(sm_mt[h] - mt);
            float ov = w0 * sm_res[idx], lt = w0 * sm_mt[8 + h];
            for (int pi = 0; pi < x.world - 1; ++pi) {
                const float* in = sm_in + pi * n_items;
                const float w = __expf(in[a.group * D + h] - mt);
                ov = fmaf(w, in[idx], ov);
                lt = fmaf(w, in[a.group * D + a.group + h], lt);
            }
            a.out[(size_t)row0 * D + idx] = lt > 0.f ? ov / lt : 0.f;
        }
    }
    // the head that finishes last advances the step counter for the next launch (every head has read it by
    // then); after a timeout the counter stays, grl_sync reports the failure and grl_exchange_reset on every
    // rank puts the ranks back in step
    if (tid == 0 && ok) {
        const int heads = a.B * a.Hkv;
        if (atomicAdd(&a.counters[kDoneSlot], 1) == heads - 1) {
            a.counters[kDoneSlot] = 0;
            *x.seq = e;
        }
    }
}

// The K (or V) pool as a 2-D bf16 tensor (rows = pages * Hkv * page tokens, head_dim columns); box = 64 columns x
// one page of one kv head.
static int make_pool_map(grl_device* dev, CUtensorMap* tm, const void* pool, uint64_t rows, int head_dim, int page_tokens) {
    TmapKey k{};
    k.ptr = pool; k.rank = 2; k.swizzle_128b = 1;
    k.dims[0] = (uint64_t)head_dim; k.dims[1] = rows;
    k.strides[0] = (uint64_t)head_dim * 2;
    k.box[0] = 64; k.box[1] = (uint32_t)page_tokens;
    return get_tensor_map(dev, k, tm);
}

}  // namespace dmma

bool decode_mma_supported(const grl_decode_params* p) {
    const grl_kv_layout& kv = p->kv;
    const int group = p->num_q_heads / kv.num_kv_heads;
    const bool geometry = (kv.page_tokens == 64 || kv.page_tokens == 32 || kv.page_tokens == 16) && group >= 1 && group <= 8 &&
                          ((uintptr_t)kv.k_pages % 16 == 0) && ((uintptr_t)kv.v_pages % 16 == 0);
    if (kv.cache_dtype == GRL_FP8_INT4)
        return geometry && kv.head_dim == 128 && kv.scales && ((uintptr_t)kv.scales % 16 == 0) && ((uintptr_t)p->q % 16 == 0);
    return kv.cache_dtype == GRL_BF16 && geometry && (kv.head_dim == 128 || kv.head_dim == 64) && ((uintptr_t)p->q % 8 == 0);
}

template <bool QUANT, int HD>
static int launch_instance(grl_device* dev, const CUtensorMap& tk, const CUtensorMap& tv, const dmma::Args& a, dim3 grid) {
    using namespace dmma;
    static bool attr_set[64] = {};
    if (!attr_set[dev->ordinal & 63]) {      // a function attribute belongs to the device that was current
        GRL_CUDA(cudaFuncSetAttribute(decode_mma_kernel<QUANT, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Smem<QUANT, HD>::TOTAL));
        attr_set[dev->ordinal & 63] = true;
    }
    decode_mma_kernel<QUANT, HD><<<grid, kThreads, Smem<QUANT, HD>::TOTAL, dev->stream>>>(tk, tv, a);
    GRL_LAUNCHED(QUANT ? "decode_mma_kernel<quantised>" : "decode_mma_kernel");
    return GRL_OK;
}

int decode_mma_launch(grl_device* dev, const grl_decode_params* p, int n_splits, float scale, bool direct, bool fuse) {
    using namespace dmma;
    const grl_kv_layout& kv = p->kv;
    const uint64_t pages = kv.num_pages > 0 ? (uint64_t)kv.num_pages : (uint64_t)kv.batch * kv.max_pages;
    const uint64_t rows = pages * kv.num_kv_heads * kv.page_tokens;
    const bool quant = kv.cache_dtype == GRL_FP8_INT4;
    CUtensorMap tk, tv;
    int rc;
    if (quant) {
        // the key pool as a 2-D byte tensor (rows, 128); box = one page of one kv head; values and scales are
        // contiguous per (page, kv head) and travel as plain bulk copies
        TmapKey k{};
        k.ptr = kv.k_pages; k.rank = 2; k.swizzle_128b = 1; k.bytes = 1;
        k.dims[0] = D; k.dims[1] = rows;
        k.strides[0] = (uint64_t)D;
        k.box[0] = D; k.box[1] = (uint32_t)kv.page_tokens;
        rc = get_tensor_map(dev, k, &tk);
        tv = tk;
    } else {
        rc = make_pool_map(dev, &tk, kv.k_pages, rows, kv.head_dim, kv.page_tokens);
        if (!rc) rc = make_pool_map(dev, &tv, kv.v_pages, rows, kv.head_dim, kv.page_tokens);
    }
    if (rc) return rc;
    Args a{};
    a.v_q = static_cast<const uint8_t*>(kv.v_pages); a.scales = static_cast<const uint16_t*>(kv.scales);
    a.block_table = kv.block_table; a.seq_lens = kv.seq_lens; a.q = p->q;
    a.part = (float*)p->workspace; a.out = p->out; a.status = dev->d_status;
    a.B = kv.batch; a.Hq = p->num_q_heads; a.Hkv = kv.num_kv_heads; a.max_pages = kv.max_pages;
    a.page = kv.page_tokens; a.ppt = P / kv.page_tokens;
    a.n_splits = n_splits; a.group = p->num_q_heads / kv.num_kv_heads;
    a.scale = scale; a.direct = direct ? 1 : 0;
    a.fuse = fuse ? 1 : 0; a.counters = dev->d_counters; a.partial_out = p->partial_out;
    a.scores_out = p->scores_out; a.scores_ld = p->scores_ld;
    a.x.world = 1;
    a.wait_limit = dev->wait_limit_cycles;
    if (p->exchange) {
        GRL_REQUIRE(fuse && !direct, "the fused cross-GPU merge needs the split-KV path");
        rc = fill_peer_exchange(dev, p->exchange, &a.x);
        if (rc) return rc;
        const int heads = kv.batch * kv.num_kv_heads;
        GRL_REQUIRE(heads <= dev->prop.multiProcessorCount,
                    "fused cross-GPU merge: B*Hkv = %d exceeds the %d SMs (waiting CTAs must leave room for the rest)",
                    heads, dev->prop.multiProcessorCount);
        GRL_REQUIRE(p->exchange->low_latency, "the exchange inside the decode kernel uses the low-latency inbox "
                                              "format ({value, step} pairs): set low_latency");
        GRL_REQUIRE(p->out, "out is NULL");
    }
    dev->status_dirty = true;
    dim3 grid(n_splits, kv.num_kv_heads, kv.batch);
    if (quant) return launch_instance<true, 128>(dev, tk, tv, a, grid);
    return kv.head_dim == 64 ? launch_instance<false, 64>(dev, tk, tv, a, grid) : launch_instance<false, 128>(dev, tk, tv, a, grid);
}

}  // namespace grl
