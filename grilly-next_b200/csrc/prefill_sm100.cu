// Blackwell (sm_100a) flash-attention forward for bf16 inputs, head_dim 128 or 64.
//
// Replaces the S^2/(64*64) dispatch+barrier pairs of ops::flashAttention2
// (cpp/src/ops/attention.cpp:125-141) and the per-(q,k) thread of flash-attention2-rope.glsl
// by one launch in which a CTA owns TWO 128-row query tiles (256 rows) of one (batch, head) and
// streams the K/V tiles once for both:
//
//   warp 1       TMA producer: both Q tiles once, then K/V tiles (128 keys x 128 dims, two
//                64-column boxes, 128-byte swizzle) into a 2-stage shared-memory ring.
//   warps 12-15  RoPE: rotate each K tile in place in shared memory, fence.proxy.async, hand the
//                tile to the MMA warp.  (Each softmax warpgroup rotates its own Q tile once.)
//   warps 0, 2   one thread per query tile issues tcgen05.mma: S_t = Q_t K^T (A,B from shared memory, K-major)
//                into TMEM, then O_t += P_t V with P_t read from TMEM and V as an MN-major
//                shared-memory operand; per 64-key step i the issue order is PV0_i, QK0_i+2, PV1_i, QK1_i+2.
//   warps 4-7 / 8-11  softmax warpgroup of query tile 0 / 1, one thread per query row:
//                tcgen05.ld of the S row, causal / length predicate, fp32 online softmax in the
//                exp2 domain, P written back to TMEM as packed bf16, O rescaled in TMEM only when
//                the row maximum moved by more than 2^8 (the stale maximum stays the reference,
//                so the result is exact), final O / l to global memory.
//
// S is produced in 64-key halves into two TMEM buffers per tile, so that QK^T of step i+1 and i+2
// runs while the softmax of step i is still busy and P.V of step i does not gate the next scores.
// TMEM columns of tile t: S halves at t*256 + {0, 64} (P overlays the first 32 columns of its
// half), O at t*256 + 128.  Every mbarrier wait is bounded; on expiry the CTA records an error, drains
// its copies and returns.
#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tmem_ops.cuh"

namespace grl {

namespace sm100 {

constexpr int BM = 128;            // query rows per tile (TMEM lanes)
constexpr int NQ = 2;              // query tiles per CTA
constexpr int BN = 128;            // keys per tile
constexpr int NSTAGE = 2;
constexpr int HALF_BYTES = BM * 64 * 2;     // one 64-column box: 16 KiB
constexpr int TILE_BYTES = 2 * HALF_BYTES;  // 32 KiB: a Q/K/V tile of head_dim 128 (two boxes), and the stride between
                                            // tile buffers for either head_dim (head_dim 64 fills the first box only)
constexpr int kThreads = 512;      // four warpgroups: MMA + TMA (+2 idle warps) | softmax 0 | softmax 1 | RoPE
constexpr int WARP_MMA = 0, WARP_TMA = 1, WARP_MMA1 = 2, WARP_SOFTMAX0 = 4, WARP_ROT0 = 12;   // warp 3 idle
// Register budget per warpgroup (setmaxnreg); 2*128*160 + 128*112 + 128*80 = 65536.
constexpr int REGS_SOFTMAX = 160, REGS_ROPE = 112, REGS_MISC = 80;
// setmaxnreg.inc is served only from what setmaxnreg.dec of the SAME CTA released (never from the SM's
// unallocated registers): if the budgets exceeded threads x launch-bound registers, the increase would wait
// forever.
static_assert(2 * REGS_SOFTMAX + REGS_ROPE + REGS_MISC <= 4 * 128, "setmaxnreg budgets exceed the CTA's register allocation");
constexpr int SMEM_Q = 0;
constexpr int SMEM_K = SMEM_Q + NQ * TILE_BYTES;
constexpr int SMEM_V = SMEM_K + NSTAGE * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_V + NSTAGE * TILE_BYTES;
constexpr int SMEM_TOTAL = SMEM_BAR + 256 + 1024;  // + barrier block + alignment slack
constexpr int kHeadGroup = 32;      // (batch, head) slices scheduled together under a causal mask
constexpr int BH = 64;              // keys per softmax step: S is computed in 64-key halves, double-buffered
constexpr uint32_t TMEM_COLS = 512;
// TMEM columns of query tile t: S half-buffer b at t*256 + b*64 (P overlays its first 32 columns),
// O at t*256 + 128.
constexpr uint32_t TMEM_TILE = 256, TMEM_O = 128;

enum Bar { Q_FULL = 0, Q_READY = Q_FULL + NQ, K_FULL = Q_READY + NQ, K_READY = K_FULL + NSTAGE,
           K_EMPTY = K_READY + NSTAGE, V_FULL = K_EMPTY + NSTAGE, V_EMPTY = V_FULL + NSTAGE,
           S_FULL = V_EMPTY + NSTAGE, P_READY = S_FULL + 2 * NQ, O_DONE = P_READY + 2 * NQ, EXP_TURN = O_DONE + NQ,
           NUM_BARS = EXP_TURN + NQ };
// S_FULL / P_READY are indexed [t * 2 + buffer]: a barrier per S half-buffer, so that a waiter can
// never fall two phases behind (the next use of a buffer needs this waiter's own arrival first).
static_assert(NUM_BARS * 8 + 16 <= 256, "barrier block");

struct Args {
    void* o;
    const int32_t* seq_lens;
    const float2* rope;   // (S, 64) cos/sin, or NULL
    int32_t* status;      // device int32[4]: [0] error code, [1] mask of stuck barriers, [2] block x, [3] block y
    int B, H, S, n_qp;
    int causal, rope_mode;
    float scale_log2;
    long long wait_limit;   // cycle budget of every mbarrier wait
};

// kind::f16 instruction descriptor: D=f32 (bit 4), A=B=bf16 (bits 7,10), N>>3 at bit 17, M>>4 at bit 24;
// bit 16 set = B operand is MN-major (the V tile, whose contiguous dimension is head_dim = N).
constexpr uint32_t IDESC_QK = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);  // N = 64 keys
template <int HD> struct IdescPV {   // N = head_dim output columns, B (the V tile) MN-major
    static constexpr uint32_t value =
        (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BM >> 4) << 24) | (1u << 16);
};

struct Ctx {
    uint32_t bars;          // shared address of barrier 0
    volatile int* abort;    // shared abort flag
    int32_t* status;
    long long limit;        // cycles a wait may take before the CTA gives up
};

// Bounded wait.  Returns false when the CTA is aborting (this wait or another one ran out).
// Polling is deliberately not back to back: spinning warps take issue slots and shared-memory
// cycles from the warps that do the work (measured: ~8% of the kernel's throughput).
__device__ __forceinline__ bool wait_bar(const Ctx& c, int bar, uint32_t parity) {
    const uint32_t addr = c.bars + bar * 8;
    if (mbar_try_wait(addr, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait(addr, parity)) return true;
        if (*c.abort) {
            if (c.status) atomicOr(reinterpret_cast<unsigned int*>(c.status) + 1, (1u << 28) | (1u << bar));
            return false;
        }
        if (clock64() - t0 > c.limit) {
            *c.abort = 1;
            if (c.status) {
                // [0] error code, [1] bit mask of the barriers that were being waited on, [2],[3] first CTA
                atomicOr(reinterpret_cast<unsigned int*>(c.status) + 1, (1u << 28) | (1u << bar));
                if (atomicCAS(c.status, 0, GRL_ERR_TIMEOUT) == 0) {
                    c.status[2] = (parity << 16) | (threadIdx.x << 20);
                    c.status[3] = blockIdx.x;
                }
            }
            return false;
        }
    }
}

// Whole-warp form: every lane polls (a single polling lane plus a broadcast was measured slower),
// and the vote leaves the warp converged and unanimous about aborting.
__device__ __forceinline__ bool wait_bar_warp(const Ctx& c, int bar, uint32_t parity) {
    return __all_sync(0xffffffffu, wait_bar(c, bar, parity));
}

// In-place RoPE of one 128 x 128 bf16 tile held as two 64-column boxes with 128-byte swizzle:
// element (r, d) lives at box d/64, byte r*128 + ((d%64)/8 ^ (r%8))*16 + (d%8)*2.
//
// A thread keeps one 16-byte column chunk and walks down the rows in a fixed stride, so that its
// rotation frequencies never change: it reads cos/sin of its first row from the table once per tile
// and advances them by the angle-addition recurrence (c,s) <- (c*cd - s*sd, s*cd + c*sd) with the
// per-thread step (cd, sd) = cos/sin(stride * inv_freq), read once per kernel from table row `stride`.
// Rows past the end of the sequence hold zeros (TMA fill) and stay zero under any rotation.
struct RopeState {
    float cd[8], sd[8];   // step rotation; 4 pairs (interleaved) or 8 pairs (rotate_half) per thread
};

// Thread rt of the 128 owns one 16-byte chunk column and walks down the rows with a fixed stride.  Interleaved
// pairs: HD/8 chunk columns, stride 1024/HD rows (8 at head_dim 128, 16 at 64); rotate_half: HD/16 chunk columns
// of the first half, stride 2048/HD rows, the partner chunk HD/16 columns further on.
template <int HD>
__device__ __forceinline__ void rope_init(RopeState& st, const float2* __restrict__ rope, int S, int mode, int rt) {
    constexpr int HALF = HD / 2;
    if (mode == GRL_ROPE_INTERLEAVED) {
        constexpr int CH = HD / 8, STRIDE = 128 / CH;
        const float2* t = rope + (size_t)min(STRIDE, S - 1) * HALF + (rt % CH) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 v = __ldg(t + e); st.cd[e] = v.x; st.sd[e] = v.y; }
    } else {
        constexpr int CHH = HD / 16, STRIDE = 128 / CHH;
        const float2* t = rope + (size_t)min(STRIDE, S - 1) * HALF + (rt % CHH) * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) { const float2 v = __ldg(t + e); st.cd[e] = v.x; st.sd[e] = v.y; }
    }
}

// cos/sin of a thread's first row of a tile: fetched ahead of the tile itself (the table read is an L2
// round trip that would otherwise sit between the tile's arrival and its rotation).
struct RopeStart {
    float4 v[4];
};
template <int HD>
__device__ __forceinline__ RopeStart rope_load_start(int pos0, int S, const float2* __restrict__ rope, int mode, int rt) {
    constexpr int HALF = HD / 2;
    RopeStart r;
    if (mode == GRL_ROPE_INTERLEAVED) {
        constexpr int CH = HD / 8;
        const float4* t = reinterpret_cast<const float4*>(rope + (size_t)min(pos0 + rt / CH, S - 1) * HALF + (rt % CH) * 4);
        r.v[0] = __ldg(t); r.v[1] = __ldg(t + 1);
        r.v[2] = r.v[3] = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        constexpr int CHH = HD / 16;
        const float4* t = reinterpret_cast<const float4*>(rope + (size_t)min(pos0 + rt / CHH, S - 1) * HALF + (rt % CHH) * 8);
#pragma unroll
        for (int e = 0; e < 4; ++e) r.v[e] = __ldg(t + e);
    }
    return r;
}

template <int HD>
__device__ __forceinline__ void rope_tile(uint32_t tile, const RopeStart& start, int mode, int rt, const RopeState& st) {
    if (mode == GRL_ROPE_INTERLEAVED) {
        // chunk c = 4 adjacent pairs (2i, 2i+1); rows r0, r0+STRIDE, ... : r % 8 stays r0 % 8, so the swizzle term is fixed
        constexpr int CH = HD / 8, STRIDE = 128 / CH;
        const int c = rt % CH, r0 = rt / CH;
        uint32_t p = tile + (c >> 3) * HALF_BYTES + r0 * 128 + (((c & 7) ^ (r0 & 7)) << 4);
        const float4 t0 = start.v[0], t1 = start.v[1];
        // two pairs per packed operation: C = (c_e, c_e+1), S = (s_e, s_e+1)
        float2 C[2] = {make_float2(t0.x, t0.z), make_float2(t1.x, t1.z)};
        float2 Sn[2] = {make_float2(t0.y, t0.w), make_float2(t1.y, t1.w)};
        const float2 Cd[2] = {make_float2(st.cd[0], st.cd[1]), make_float2(st.cd[2], st.cd[3])};
        const float2 Sd[2] = {make_float2(st.sd[0], st.sd[1]), make_float2(st.sd[2], st.sd[3])};
        const float2 Sdn[2] = {make_float2(-st.sd[0], -st.sd[1]), make_float2(-st.sd[2], -st.sd[3])};
#pragma unroll 4
        for (int k = 0; k < 128 / STRIDE; ++k, p += STRIDE * 128) {
            uint4 v = lds128(p);
            uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float2 X0 = make_float2(__uint_as_float(w[2 * h] << 16), __uint_as_float(w[2 * h + 1] << 16));
                const float2 X1 = make_float2(__uint_as_float(w[2 * h] & 0xffff0000u), __uint_as_float(w[2 * h + 1] & 0xffff0000u));
                const float2 Snn = make_float2(-Sn[h].x, -Sn[h].y);
                const float2 Y0 = __ffma2_rn(X1, Snn, __fmul2_rn(X0, C[h]));      // x0 c - x1 s
                const float2 Y1 = __ffma2_rn(X1, C[h], __fmul2_rn(X0, Sn[h]));    // x0 s + x1 c
                __nv_bfloat162 o0 = __floats2bfloat162_rn(Y0.x, Y1.x), o1 = __floats2bfloat162_rn(Y0.y, Y1.y);
                w[2 * h] = *reinterpret_cast<uint32_t*>(&o0);
                w[2 * h + 1] = *reinterpret_cast<uint32_t*>(&o1);
                const float2 nC = __ffma2_rn(Sn[h], Sdn[h], __fmul2_rn(C[h], Cd[h]));   // c cd - s sd
                Sn[h] = __ffma2_rn(C[h], Sd[h], __fmul2_rn(Sn[h], Cd[h]));             // s cd + c sd
                C[h] = nC;
            }
            sts128(p, make_uint4(w[0], w[1], w[2], w[3]));
        }
    } else {
        // rotate_half: pairs (d, d + HD/2); the partner chunk lies HD/16 chunk columns further on (the same offset of
        // the second box at head_dim 128, four chunks along the row at 64); rows r0, r0+STRIDE, ...
        constexpr int CHH = HD / 16, STRIDE = 128 / CHH;
        const int cc = rt % CHH, r0 = rt / CHH, cb = cc + CHH;
        uint32_t p = tile + r0 * 128 + ((cc ^ (r0 & 7)) << 4);
        const uint32_t pb_off = (uint32_t)((cb >> 3) * HALF_BYTES + (((cb & 7) ^ (r0 & 7)) << 4)) - (uint32_t)((cc ^ (r0 & 7)) << 4);
        float cs[8], sn[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float4 v = start.v[e];
            cs[2 * e] = v.x; sn[2 * e] = v.y; cs[2 * e + 1] = v.z; sn[2 * e + 1] = v.w;
        }
#pragma unroll 2
        for (int k = 0; k < 128 / STRIDE; ++k, p += STRIDE * 128) {
            uint4 a = lds128(p), b = lds128(p + pb_off);
            uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float a0 = __uint_as_float(wa[e] << 16), a1 = __uint_as_float(wa[e] & 0xffff0000u);
                const float b0 = __uint_as_float(wb[e] << 16), b1 = __uint_as_float(wb[e] & 0xffff0000u);
                const float c0 = cs[2 * e], s0 = sn[2 * e], c1 = cs[2 * e + 1], s1 = sn[2 * e + 1];
                __nv_bfloat162 lo = __floats2bfloat162_rn(a0 * c0 - b0 * s0, a1 * c1 - b1 * s1);
                __nv_bfloat162 hi = __floats2bfloat162_rn(b0 * c0 + a0 * s0, b1 * c1 + a1 * s1);
                wa[e] = *reinterpret_cast<uint32_t*>(&lo);
                wb[e] = *reinterpret_cast<uint32_t*>(&hi);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float nc = cs[e] * st.cd[e] - sn[e] * st.sd[e];
                sn[e] = sn[e] * st.cd[e] + cs[e] * st.sd[e];
                cs[e] = nc;
            }
            sts128(p, make_uint4(wa[0], wa[1], wa[2], wa[3]));
            sts128(p + pb_off, make_uint4(wb[0], wb[1], wb[2], wb[3]));
        }
    }
}

template <typename TOut>
__device__ __forceinline__ void store_row_chunk(TOut* dst, const uint32_t (&r)[32], float f);
template <>
__device__ __forceinline__ void store_row_chunk<float>(float* dst, const uint32_t (&r)[32], float f) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(dst)[i] =
            make_float4(__uint_as_float(r[4 * i]) * f, __uint_as_float(r[4 * i + 1]) * f,
                        __uint_as_float(r[4 * i + 2]) * f, __uint_as_float(r[4 * i + 3]) * f);
}
template <>
__device__ __forceinline__ void store_row_chunk<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t (&r)[32], float f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 o = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2 * e]) * f,
                                                     __uint_as_float(r[8 * i + 2 * e + 1]) * f);
            w[e] = *reinterpret_cast<uint32_t*>(&o);
        }
        reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

template <typename TOut, int HD>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base_addr = (raw_addr + 1023u) & ~1023u;   // swizzled tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + (base_addr - raw_addr);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // 1-D grid over (batch*heads) x (query tile pairs).  Causal: the work of a tile pair grows with its index,
    // so within a group of kHeadGroup heads CTAs are handed out longest pair first and the shortest ones form
    // the tail; groups follow one another so that the K/V of the heads in flight (1 MiB per head at S=2048) stay
    // in L2 between the pairs that share them.  Otherwise all pairs cost the same and the pairs of one head
    // stay adjacent.
    const int n_qp = a.n_qp, n_bh = a.B * a.H;
    int qp, bh;
    if (a.causal) {
        const int per_group = kHeadGroup * n_qp;
        const int g = (int)blockIdx.x / per_group, r = (int)blockIdx.x % per_group;
        const int gsize = min(kHeadGroup, n_bh - g * kHeadGroup);
        qp = n_qp - 1 - r / gsize;
        bh = g * kHeadGroup + r % gsize;
    } else {
        qp = (int)blockIdx.x % n_qp;
        bh = (int)blockIdx.x / n_qp;
    }
    const int b = bh / a.H;
    const int S = a.S;
    const int q0 = qp * (NQ * BM);
    const int len = a.seq_lens ? min(a.seq_lens[b], S) : S;
    TOut* O = reinterpret_cast<TOut*>(a.o) + (size_t)bh * S * HD;

    if (q0 >= len) {  // padded query rows are defined as zero
        const int rows = min(NQ * BM, S - q0);
        for (int idx = tid; idx < rows * HD; idx += kThreads) store_from_float<TOut>(O + (size_t)q0 * HD + idx, 0.f);
        return;
    }
    {   // an earlier CTA failed: leave, as a whole CTA
        const int failed = (tid == 0 && a.status) ? (*reinterpret_cast<volatile int32_t*>(a.status) != 0) : 0;
        if (__syncthreads_or(failed)) return;
    }

    // kv tiles that query tile t attends to (0 when all of its rows are padding)
    int n_kt[NQ];
#pragma unroll
    for (int t = 0; t < NQ; ++t) {
        const int qt0 = q0 + t * BM;
        const int k_end = a.causal ? min(len, qt0 + BM) : len;
        n_kt[t] = (qt0 < len) ? (k_end + BN - 1) / BN : 0;
    }
    // 64-key softmax steps of tile t (the second half of its last K tile may be wholly invisible)
    int n_half[NQ];
#pragma unroll
    for (int t = 0; t < NQ; ++t) {
        const int qt0 = q0 + t * BM;
        const int k_end = a.causal ? min(len, qt0 + BM) : len;
        n_half[t] = (qt0 < len) ? (k_end + BH - 1) / BH : 0;
    }
    const int n_total = max(n_kt[0], n_kt[1]);
    const bool use_rope = a.rope_mode != GRL_ROPE_NONE;

    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SMEM_BAR + NUM_BARS * 8);
    int* abort_flag = reinterpret_cast<int*>(smem + SMEM_BAR + NUM_BARS * 8 + 4);
    Ctx ctx{base_addr + SMEM_BAR, abort_flag, a.status, a.wait_limit};
    auto bar = [&](int i) { return ctx.bars + (uint32_t)i * 8u; };

    auto load_tile = [&](uint32_t dst, const CUtensorMap* tm, int row, int full_bar) {
        mbar_expect_tx(bar(full_bar), (HD / 64) * HALF_BYTES);
        tma_load_3d(dst, tm, 0, row, bh, bar(full_bar));
        if (HD == 128) tma_load_3d(dst + HALF_BYTES, tm, 64, row, bh, bar(full_bar));
    };
    if (warp == WARP_TMA && lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmQ)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmK)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmV)) : "memory");
        for (int t = 0; t < NQ; ++t) {
            mbar_init(bar(Q_FULL + t), 1);
            mbar_init(bar(Q_READY + t), 128);
            for (int bf = 0; bf < 2; ++bf) {
                mbar_init(bar(S_FULL + 2 * t + bf), 1);
                mbar_init(bar(P_READY + 2 * t + bf), 128);
            }
            mbar_init(bar(O_DONE + t), 1);
            mbar_init(bar(EXP_TURN + t), 128);
        }
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(bar(K_FULL + s), 1);
            mbar_init(bar(K_READY + s), 128);
            mbar_init(bar(K_EMPTY + s), 2);   // one arrival per reading query tile (twice from a lone reader)
            mbar_init(bar(V_FULL + s), 1);
            mbar_init(bar(V_EMPTY + s), 2);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
        // The first loads need no "empty" wait: put them in flight now, behind nothing but the barrier
        // initialisation, while the other warps are still setting up.  QK(0,0) needs Q0 and K0 first.
        load_tile(base_addr + SMEM_Q, &tmQ, q0, Q_FULL);
        load_tile(base_addr + SMEM_K, &tmK, 0, K_FULL);
        if (n_kt[1] > 0) load_tile(base_addr + SMEM_Q + TILE_BYTES, &tmQ, q0 + BM, Q_FULL + 1);
        load_tile(base_addr + SMEM_V, &tmV, 0, V_FULL);
        if (n_total > 1) {
            load_tile(base_addr + SMEM_K + TILE_BYTES, &tmK, BN, K_FULL + 1);
            load_tile(base_addr + SMEM_V + TILE_BYTES, &tmV, BN, V_FULL + 1);
        }
    }
    if (warp == WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp < WARP_SOFTMAX0) {
      reg_dec<REGS_MISC>();
      if (warp == WARP_TMA) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int issued = 2 * min(n_total, NSTAGE);   // K/V tile loads in flight (K_j = 2j, V_j = 2j+1): the first stages
            bool ok = true;
            for (int j = NSTAGE; j < n_total && ok; ++j) {
                const int s = j % NSTAGE, it = j / NSTAGE;
                ok = wait_bar(ctx, K_EMPTY + s, (it - 1) & 1);
                if (!ok) break;
                load_tile(base_addr + SMEM_K + s * TILE_BYTES, &tmK, j * BN, K_FULL + s);
                issued = 2 * j + 1;
                ok = wait_bar(ctx, V_EMPTY + s, (it - 1) & 1);
                if (!ok) break;
                load_tile(base_addr + SMEM_V + s * TILE_BYTES, &tmV, j * BN, V_FULL + s);
                issued = 2 * j + 2;
            }
            if (*ctx.abort) {
                // Drain: copies already issued must land before the CTA's shared memory is released.
                const long long t0 = clock64();
                while (!mbar_try_wait(bar(Q_FULL), 0) && clock64() - t0 < ctx.limit) {}
                if (n_kt[1] > 0)
                    while (!mbar_try_wait(bar(Q_FULL + 1), 0) && clock64() - t0 < ctx.limit) {}
                for (int x = max(0, issued - 2 * NSTAGE); x < issued; ++x) {
                    const int j = x >> 1, s = j % NSTAGE, it = j / NSTAGE;
                    const uint32_t bb = bar(((x & 1) ? V_FULL : K_FULL) + s);
                    while (!mbar_try_wait(bb, it & 1) && clock64() - t0 < ctx.limit) {}
                }
            }
        }
      } else if (warp == WARP_MMA || warp == WARP_MMA1) {
        // ------------------------------------------------------------------ MMA issuers: one thread per query tile
        // Each tile has its own in-order chain  wait P -> P.V(i) -> Q.K^T(i+2)  issued by its own thread, so that
        // one tile's softmax never holds up the other tile's tensor work; the tensor pipe interleaves the two.
        const int t = (warp == WARP_MMA) ? 0 : 1;
        if (lane == 0 && n_half[t] > 0) {
            bool ok = true;
            const uint32_t qa = desc_lo(base_addr + SMEM_Q + t * TILE_BYTES, 16);
            const uint32_t k_lo = desc_lo(base_addr + SMEM_K, 16), v_lo = desc_lo(base_addr + SMEM_V, HALF_BYTES);
            const int nh = n_half[t], other_tiles = n_kt[t ^ 1];
            const uint32_t s_tmem = tmem_base + (uint32_t)t * TMEM_TILE, o_tmem = s_tmem + TMEM_O;
            // A K or V tile (two 64-key steps) is released once per reading tile: the K_EMPTY / V_EMPTY barriers
            // count two arrivals, and a tile that reads a K/V tile alone arrives twice.
            auto release = [&](int bar_id, int j) {
                mma_commit(bar(bar_id));
                if (j >= other_tiles) mma_commit(bar(bar_id));
            };
            // S_t[i & 1] = Q_t K[64 keys of step i]^T
            auto issue_qk = [&](int i) -> bool {
                const int j = i >> 1, s = j % NSTAGE, it = j / NSTAGE;
                if (!wait_bar(ctx, (use_rope ? K_READY : K_FULL) + s, it & 1)) return false;
                tc_fence_after();
                const uint32_t d_tmem = s_tmem + (uint32_t)(i & 1) * BH;
                const uint32_t kb = k_lo + (uint32_t)s * (TILE_BYTES >> 4) + (uint32_t)(i & 1) * ((BH * 128) >> 4);  // rows 64.. of each box
                mma_ss2<false>(d_tmem, qa, kb, IDESC_QK);
#pragma unroll
                for (int ks = 1; ks < HD / 16; ++ks) {
                    const uint32_t off = (uint32_t)(((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4);
                    mma_ss2<true>(d_tmem, qa + off, kb + off, IDESC_QK);
                }
                mma_commit(bar(S_FULL + 2 * t + (i & 1)));
                if ((i & 1) || i + 1 >= nh) release(K_EMPTY + s, j);   // last step of this tile on K tile j
                return true;
            };
            ok = wait_bar(ctx, (use_rope ? Q_READY : Q_FULL) + t, 0);
            for (int i = 0; i < 2 && i < nh && ok; ++i) ok = issue_qk(i);   // two steps of S ahead of the softmax
            for (int i = 0; i < nh && ok; ++i) {
                const int j = i >> 1, s = j % NSTAGE, it = j / NSTAGE;
                ok = wait_bar(ctx, P_READY + 2 * t + (i & 1), (i >> 1) & 1);
                if (ok) ok = wait_bar(ctx, V_FULL + s, it & 1);
                if (!ok) break;
                tc_fence_after();
                // O_t += P_t[step i] V[64 keys]: A = P in TMEM (16 keys = 8 packed columns per k-step), B = 16 key
                // rows of V = 2 KiB per k-step, MN-major (64-column boxes HALF_BYTES apart = LBO, 8-row groups
                // 1 KiB apart = SBO).
                const uint32_t p_tmem = s_tmem + (uint32_t)(i & 1) * BH;
                const uint32_t vb = v_lo + (uint32_t)s * (TILE_BYTES >> 4) + (uint32_t)(i & 1) * ((BH * 128) >> 4);
                mma_ts2(o_tmem, p_tmem, vb, IdescPV<HD>::value, i > 0);
#pragma unroll
                for (int ks = 1; ks < BH / 16; ++ks)
                    mma_ts2(o_tmem, p_tmem + ks * 8, vb + (uint32_t)ks * (2048 >> 4), IdescPV<HD>::value, 1u);
                mma_commit(bar(O_DONE + t));
                if ((i & 1) || i + 1 >= nh) release(V_EMPTY + s, j);
                if (i + 2 < nh) ok = issue_qk(i + 2);   // reuses buffer i & 1: in order after PV(t, i)
            }
        }
      }
    } else if (warp >= WARP_ROT0) {
        // ------------------------------------------------------------------ RoPE on the K tiles
        reg_dec<REGS_ROPE>();
        if (use_rope) {
            const int rt = tid - WARP_ROT0 * 32;
            RopeState st;
            rope_init<HD>(st, a.rope, S, a.rope_mode, rt);
            bool ok = true;
            RopeStart cur = rope_load_start<HD>(0, S, a.rope, a.rope_mode, rt);
            for (int j = 0; j < n_total && ok; ++j) {
                const int s = j % NSTAGE, it = j / NSTAGE;
                const RopeStart nxt = rope_load_start<HD>((j + 1) * BN, S, a.rope, a.rope_mode, rt);   // for the next tile
                ok = wait_bar_warp(ctx, K_FULL + s, it & 1);
                if (!ok) break;
                rope_tile<HD>(base_addr + SMEM_K + s * TILE_BYTES, cur, a.rope_mode, rt, st);
                cur = nxt;
                fence_async_smem();
                mbar_arrive(bar(K_READY + s));
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax / correction / epilogue
        reg_inc<REGS_SOFTMAX>();
        const int t = (warp - WARP_SOFTMAX0) >> 2;  // query tile of this warpgroup
        const int row = tid & 127;                 // TMEM lane == query row of the tile
        const int qt0 = q0 + t * BM;
        const int row_g = qt0 + row;
        const int n = n_kt[t];
        if (n == 0) {
            // every row of this tile is padding: zeros (rows inside the tensor only)
            if (row_g < S) {
                uint32_t z[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) z[i] = 0u;
#pragma unroll
                for (int ch = 0; ch < HD / 32; ++ch) store_row_chunk<TOut>(O + (size_t)row_g * HD + ch * 32, z, 0.f);
            }
        } else {
            const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
            const uint32_t s_addr = lane_addr + (uint32_t)t * TMEM_TILE, o_addr = s_addr + TMEM_O;
            bool ok = true;
            if (use_rope) {   // this warpgroup rotates its own Q tile
                RopeState st;
                rope_init<HD>(st, a.rope, S, a.rope_mode, row);
                const RopeStart start = rope_load_start<HD>(qt0, S, a.rope, a.rope_mode, row);
                ok = wait_bar_warp(ctx, Q_FULL + t, 0);
                if (ok) {
                    rope_tile<HD>(base_addr + SMEM_Q + t * TILE_BYTES, start, a.rope_mode, row, st);
                    fence_async_smem();
                    mbar_arrive(bar(Q_READY + t));
                }
            }
            float m_ref = -INFINITY, l = 0.f;
            const int nh = n_half[t];
            // The two softmax warpgroups take turns in the exponential phase (it saturates the MUFU unit they
            // share): a warpgroup starts its exponentials when the other has finished its own, and spends its
            // loads, maxima, stores and barrier hops while the other one exponentiates.  Only for the steps that
            // both tiles have.
            const int nc = min(n_half[0], n_half[1]);
            if (t == 1 && nc > 0) mbar_arrive(bar(EXP_TURN + 0));   // tile 0 goes first
            for (int i = 0; i < nh && ok; ++i) {
                const int bf = i & 1, k0 = i * BH;
                ok = wait_bar_warp(ctx, S_FULL + 2 * t + bf, (i >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
                uint32_t sr[BH];
                tmem_ld_x64_sync(s_addr + bf * BH, sr);
                const bool need_mask = (a.causal && k0 + BH - 1 > qt0) || (k0 + BH > len);  // warpgroup-uniform
                if (need_mask) {
                    const int limit = min(a.causal ? row_g : 0x7fffffff, len - 1) - k0;  // last visible column
#pragma unroll
                    for (int c = 0; c < BH; ++c)
                        if (c > limit) sr[c] = 0xff800000u;   // -inf
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains, 3-input max
#pragma unroll
                for (int c = 0; c < BH; c += 8) {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        mx4[e] = max3(mx4[e], __uint_as_float(sr[c + 2 * e]), __uint_as_float(sr[c + 2 * e + 1]));
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                const float m_new = fmaxf(m_ref, mx * a.scale_log2);
                bool o_waited = false;
                if (i == 0) {
                    m_ref = (m_new == -INFINITY) ? 0.f : m_new;
                } else {
                    const bool need = m_new > m_ref + 8.f;
                    if (__any_sync(0xffffffffu, need)) {
                        ok = wait_bar_warp(ctx, O_DONE + t, (i - 1) & 1);   // PV(t, i-1) has written O
                        if (!ok) break;
                        o_waited = true;
                        tc_fence_after();
                        const float f = need ? ex2(m_ref - m_new) : 1.f;
                        if (need) m_ref = m_new;
                        l *= f;
#pragma unroll
                        for (int ch = 0; ch < HD / 32; ++ch) {
                            uint32_t orow[32];
                            tmem_ld_x32_sync(o_addr + ch * 32, orow);
#pragma unroll
                            for (int e = 0; e < 32; ++e) orow[e] = __float_as_uint(__uint_as_float(orow[e]) * f);
                            tmem_st_x32(o_addr + ch * 32, orow);
                        }
                        tmem_st_wait();
                    }
                }
                if (i < nc) {
                    ok = wait_bar_warp(ctx, EXP_TURN + t, i & 1);
                    if (!ok) break;
                }
                // p = exp2(s * scale_log2 - m_ref): packed two-wide FMA and add, scalar ex2 (MUFU)
                const float2 sc2 = make_float2(a.scale_log2, a.scale_log2), nm2 = make_float2(-m_ref, -m_ref);
                float2 rs4[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
                for (int ch = 0; ch < BH / 32; ++ch) {      // 32 keys -> 16 packed columns per store
                    uint32_t pk[16];
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        float2 x = make_float2(__uint_as_float(sr[ch * 32 + c]), __uint_as_float(sr[ch * 32 + c + 1]));
                        x = __ffma2_rn(x, sc2, nm2);
                        const float2 pe = make_float2(ex2(x.x), ex2(x.y));
                        rs4[(c >> 1) & 3] = __fadd2_rn(rs4[(c >> 1) & 3], pe);
                        __nv_bfloat162 pp = __floats2bfloat162_rn(pe.x, pe.y);   // even key in the low half
                        pk[c >> 1] = *reinterpret_cast<uint32_t*>(&pp);
                    }
                    tmem_st_x16(s_addr + bf * BH + ch * 16, pk);
                }
                if (t == 0 ? (i < nc) : (i + 1 < nc)) mbar_arrive(bar(EXP_TURN + (t ^ 1)));   // the other tile's turn
                l += ((rs4[0].x + rs4[0].y) + (rs4[1].x + rs4[1].y)) + ((rs4[2].x + rs4[2].y) + (rs4[3].x + rs4[3].y));
                tmem_st_wait();
                // Consume the phase of PV(t, i-1) BEFORE arriving: after the arrival PV(t, i) may complete too,
                // and a waiter that then looks for the parity of phase i-1 would find the barrier two phases
                // ahead and never return.  PV(t, i-1) was issued a whole softmax step ago: no stall here.
                if (i >= 1 && !o_waited) {
                    ok = wait_bar_warp(ctx, O_DONE + t, (i - 1) & 1);
                    if (!ok) break;
                }
                tc_fence_before();
                mbar_arrive(bar(P_READY + 2 * t + bf));
            }
            const int n = nh;
            if (ok) ok = wait_bar_warp(ctx, O_DONE + t, (n - 1) & 1);
            if (ok) {
                tc_fence_after();
                const bool zero = (row_g >= len) || !(l > 0.f);
                const float inv = zero ? 0.f : 1.f / l;
                if constexpr (sizeof(TOut) == 4) {
                    // Each thread holds one 512-byte output row; written directly, a warp store would touch 32
                    // rows.  Transpose through shared memory instead (this tile's Q buffer is dead: all of its
                    // QK^T have completed): 32 rows x 64 columns per pass, 16-byte chunks XOR-swizzled by row, then
                    // every warp store writes 256 contiguous bytes of one row.
                    const uint32_t stage = base_addr + SMEM_Q + t * TILE_BYTES + (warp & 3) * 8192;
                    const int row_w0 = qt0 + (warp & 3) * 32;
#pragma unroll
                    for (int pass = 0; pass < HD / 64; ++pass) {
#pragma unroll
                        for (int ch = 0; ch < 2; ++ch) {
                            uint32_t orow[32];
                            tmem_ld_x32_sync(o_addr + pass * 64 + ch * 32, orow);
#pragma unroll
                            for (int c = 0; c < 8; ++c) {
                                const int chunk = ch * 8 + c;
                                sts128(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4),
                                       make_uint4(__float_as_uint(__uint_as_float(orow[4 * c]) * inv),
                                                  __float_as_uint(__uint_as_float(orow[4 * c + 1]) * inv),
                                                  __float_as_uint(__uint_as_float(orow[4 * c + 2]) * inv),
                                                  __float_as_uint(__uint_as_float(orow[4 * c + 3]) * inv)));
                            }
                        }
                        __syncwarp();
#pragma unroll 8
                        for (int rr = 0; rr < 32; ++rr) {
                            const float2 v = lds64f(stage + rr * 256 + (((lane >> 1) ^ (rr & 15)) << 4) + (lane & 1) * 8);
                            if (row_w0 + rr < S)
                                *reinterpret_cast<float2*>(reinterpret_cast<float*>(O) + (size_t)(row_w0 + rr) * HD + pass * 64 + 2 * lane) = v;
                        }
                        __syncwarp();
                    }
                } else {
#pragma unroll
                    for (int ch = 0; ch < HD / 32; ++ch) {
                        uint32_t orow[32];
                        tmem_ld_x32_sync(o_addr + ch * 32, orow);   // warp-collective: no divergence here
                        if (row_g < S) store_row_chunk<TOut>(O + (size_t)row_g * HD + ch * 32, orow, inv);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == WARP_MMA) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// (B*H, S, head_dim) bf16 tensor, box = 64 columns x 128 rows x 1, 128-byte swizzle, zero fill out of bounds.
static int make_map(grl_device* dev, CUtensorMap* tm, const void* ptr, int BH, int S, int HD) {
    TmapKey k{};
    k.ptr = ptr; k.rank = 3; k.swizzle_128b = 1;
    k.dims[0] = HD; k.dims[1] = (uint64_t)S; k.dims[2] = (uint64_t)BH;
    k.strides[0] = (uint64_t)HD * 2; k.strides[1] = (uint64_t)S * HD * 2;
    k.box[0] = 64; k.box[1] = BM; k.box[2] = 1;
    return get_tensor_map(dev, k, tm);
}

}  // namespace sm100

int flash_fwd_sm100(grl_device* dev, const grl_flash_params* p, float scale, const float2* rope, int32_t* status) {
    using namespace sm100;
    GRL_REQUIRE(p->head_dim == 128 || p->head_dim == 64, "the tcgen05 prefill kernel needs head_dim 128 or 64 (got %d)", p->head_dim);
    GRL_REQUIRE(p->in_dtype == GRL_BF16, "the tcgen05 prefill kernel takes bf16 Q/K/V (cast with grl_cast first)");
    GRL_REQUIRE(!p->mask, "the tcgen05 prefill kernel takes causal / seq_lens masks only");
    GRL_REQUIRE(scale > 0.f, "scale must be positive");
    GRL_REQUIRE(((uintptr_t)p->q % 16 == 0) && ((uintptr_t)p->k % 16 == 0) && ((uintptr_t)p->v % 16 == 0) &&
                    ((uintptr_t)p->o % 16 == 0),
                "Q/K/V/O must be 16-byte aligned");
    const int BH = p->batch * p->heads;
    CUtensorMap tq, tk, tv;
    const int HD = p->head_dim;
    int rc = make_map(dev, &tq, p->q, BH, p->seq_len, HD);
    if (!rc) rc = make_map(dev, &tk, p->k, BH, p->seq_len, HD);
    if (!rc) rc = make_map(dev, &tv, p->v, BH, p->seq_len, HD);
    if (rc) return rc;
    Args a{};
    a.o = p->o; a.seq_lens = p->seq_lens; a.rope = rope; a.status = status;
    a.B = p->batch; a.H = p->heads; a.S = p->seq_len;
    a.causal = p->causal; a.rope_mode = p->rope_mode;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.wait_limit = dev->wait_limit_cycles;
    a.n_qp = (p->seq_len + NQ * BM - 1) / (NQ * BM);
    dim3 grid((unsigned)BH * a.n_qp);
    static bool attr_set[64] = {};
    if (!attr_set[dev->ordinal & 63]) {      // a function attribute belongs to the device that was current
        GRL_CUDA(cudaFuncSetAttribute(flash_fwd_sm100_kernel<float, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        GRL_CUDA(cudaFuncSetAttribute(flash_fwd_sm100_kernel<__nv_bfloat16, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        GRL_CUDA(cudaFuncSetAttribute(flash_fwd_sm100_kernel<float, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        GRL_CUDA(cudaFuncSetAttribute(flash_fwd_sm100_kernel<__nv_bfloat16, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        attr_set[dev->ordinal & 63] = true;
    }
    const bool f32 = p->out_dtype == GRL_F32;
    if (HD == 128) {
        if (f32) flash_fwd_sm100_kernel<float, 128><<<grid, kThreads, SMEM_TOTAL, dev->stream>>>(tq, tk, tv, a);
        else flash_fwd_sm100_kernel<__nv_bfloat16, 128><<<grid, kThreads, SMEM_TOTAL, dev->stream>>>(tq, tk, tv, a);
    } else {
        if (f32) flash_fwd_sm100_kernel<float, 64><<<grid, kThreads, SMEM_TOTAL, dev->stream>>>(tq, tk, tv, a);
        else flash_fwd_sm100_kernel<__nv_bfloat16, 64><<<grid, kThreads, SMEM_TOTAL, dev->stream>>>(tq, tk, tv, a);
    }
    GRL_LAUNCHED("flash_fwd_sm100_kernel");
    return GRL_OK;
}

}  // namespace grl
