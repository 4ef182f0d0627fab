// Linear projection y = x W^T + b on the Blackwell tensor cores (bf16 operands, fp32 accumulation and
// output), plus the exact fp32 form.
//
// Replaces ops::linear (cpp/src/ops/linear.cpp:20-82, shader fnn-linear) and the fused QKV projection
// (shaders/fused-qkv-projection.glsl:40-74: the same product with the packed [W_q; W_k; W_v] weight),
// i.e. the steps on either side of attention.  x is (M, K) row-major, W (N, K) row-major -- both K-major,
// which is what tcgen05.mma wants from shared memory -- and y (M, N).
//
// One CTA computes a 128 x 128 tile of y: warp 0 streams 128 x 64 boxes of x and W through a four-stage
// shared-memory ring with TMA (128-byte swizzle; rows and columns past the edge arrive as zeros), one thread of
// warp 1 issues four 128x128x16 tcgen05.mma per stage into a TMEM accumulator (128 lanes x 128 fp32 columns),
// and warps 4-7 read the accumulator back, add the bias and write rows through a shared-memory transpose so
// that every warp store covers contiguous bytes of one row.  Every mbarrier wait is bounded.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tmem_ops.cuh"

namespace grl {
namespace lin {

using namespace sm100;

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int NST = 3;             // 96 KiB of ring: two CTAs per SM, so one CTA's epilogue overlaps the other's products
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE = A_BYTES + B_BYTES;   // 16 + 16 KiB
constexpr int SMEM_BAR = NST * STAGE;
constexpr int SMEM_TOTAL = SMEM_BAR + 128 + 1024;
constexpr int kThreads = 256;      // warp 0 TMA, warp 1 MMA, warps 2-3 idle, warps 4-7 epilogue (TMEM lanes 0..127)
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

struct Args {
    const float* bias;     // (N) or NULL
    float* y;              // (M, N)
    int32_t* status;
    int M, N, K;
    long long wait_limit;
};

__device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, volatile int* abort, const Args& a, int which) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort) return false;
        if (clock64() - t0 > a.wait_limit) {
            *abort = 1;
            if (a.status && atomicCAS(a.status, 0, GRL_ERR_TIMEOUT) == 0) {
                a.status[1] = (5 << 28) | which;
                a.status[2] = blockIdx.x;
                a.status[3] = blockIdx.y;
            }
            return false;
        }
    }
}

__global__ void __launch_bounds__(kThreads, 2)
linear_sm100_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const Args a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int n_k = (a.K + BK - 1) / BK;

    const uint32_t bars = base + SMEM_BAR;
    auto full = [&](int s) { return bars + (uint32_t)s * 8u; };
    auto empty = [&](int s) { return bars + (uint32_t)(NST + s) * 8u; };
    const uint32_t acc_full = bars + 2 * NST * 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SMEM_BAR + (2 * NST + 1) * 8);
    volatile int* abort = reinterpret_cast<volatile int*>(smem + SMEM_BAR + (2 * NST + 1) * 8 + 4);

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmX)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmW)) : "memory");
        for (int s = 0; s < NST; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        mbar_init(acc_full, 1);
        *abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(128) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            for (int k = 0; k < n_k; ++k) {
                const int s = k % NST, it = k / NST;
                if (it > 0 && !wait(empty(s), (it - 1) & 1, abort, a, NST + s)) break;
                const uint32_t dst = base + (uint32_t)s * STAGE;
                mbar_expect_tx(full(s), STAGE);
                tma_load_2d(dst, &tmX, k * BK, m0, full(s));
                tma_load_2d(dst + A_BYTES, &tmW, k * BK, n0, full(s));
                issued = k + 1;
            }
            if (*abort) {     // copies already issued must land before the shared memory is released
                const long long t0 = clock64();
                for (int k = max(0, issued - NST); k < issued; ++k)
                    while (!mbar_try_wait(full(k % NST), (k / NST) & 1) && clock64() - t0 < a.wait_limit) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int k = 0; k < n_k && ok; ++k) {
                const int s = k % NST, it = k / NST;
                ok = wait(full(s), it & 1, abort, a, s);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_lo = desc_lo(base + (uint32_t)s * STAGE, 16), b_lo = desc_lo(base + (uint32_t)s * STAGE + A_BYTES, 16);
                if (k == 0) mma_ss2<false>(tmem, a_lo, b_lo, IDESC);
                else mma_ss2<true>(tmem, a_lo, b_lo, IDESC);
#pragma unroll
                for (int ks = 1; ks < BK / 16; ++ks) mma_ss2<true>(tmem, a_lo + (uint32_t)(ks * 32 >> 4), b_lo + (uint32_t)(ks * 32 >> 4), IDESC);
                mma_commit(empty(s));                 // the stage is free once these MMAs have read it
            }
            if (ok) mma_commit(acc_full);
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue: TMEM -> (+ bias) -> global
        const bool ok = __all_sync(0xffffffffu, wait(acc_full, 0, abort, a, 2 * NST));
        if (ok) {
            tc_fence_after();
            const int w = warp & 3;
            const uint32_t t_addr = tmem + ((uint32_t)(w * 32) << 16);
            // the ring is idle now (every MMA has completed): 8 KiB of it per warp stage 32 rows x 64 columns
            const uint32_t stage = base + (uint32_t)w * 8192;
            const int row_w0 = m0 + w * 32;
            const bool vec2 = (a.N % 2) == 0;
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t r[32];
                    tmem_ld_x32_sync(t_addr + pass * 64 + ch * 32, r);
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const int chunk = ch * 8 + c;
                        sts128(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4), make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]));
                    }
                }
                __syncwarp();
                const int col = n0 + pass * 64 + 2 * lane;
                float b0 = 0.f, b1 = 0.f;
                if (a.bias) {
                    if (col < a.N) b0 = __ldg(a.bias + col);
                    if (col + 1 < a.N) b1 = __ldg(a.bias + col + 1);
                }
#pragma unroll 8
                for (int rr = 0; rr < 32; ++rr) {
                    const float2 v = lds64f(stage + rr * 256 + (((lane >> 1) ^ (rr & 15)) << 4) + (lane & 1) * 8);
                    const int row = row_w0 + rr;
                    if (row < a.M) {
                        float* dst = a.y + (size_t)row * a.N + col;
                        if (vec2 && col + 1 < a.N) *reinterpret_cast<float2*>(dst) = make_float2(v.x + b0, v.y + b1);
                        else {
                            if (col < a.N) dst[0] = v.x + b0;
                            if (col + 1 < a.N) dst[1] = v.y + b1;
                        }
                    }
                }
                __syncwarp();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128) : "memory");
}

// Exact fp32 form: the arithmetic of fnn-linear / fused-qkv-projection (one dot product per output, k ascending),
// 16 x 16 tiles in shared memory.
__global__ void __launch_bounds__(256) linear_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                          const float* __restrict__ bias, float* __restrict__ y, int M,
                                                          int K, int N) {
    __shared__ float xs[16][17], ws[16][17];
    const int lx = threadIdx.x & 15, ly = threadIdx.x >> 4;
    const int m = blockIdx.y * 16 + ly, n = blockIdx.x * 16 + lx;
    float acc = 0.f;
    for (int k0 = 0; k0 < K; k0 += 16) {
        xs[ly][lx] = (m < M && k0 + lx < K) ? x[(size_t)m * K + k0 + lx] : 0.f;
        const int wn = blockIdx.x * 16 + ly;
        ws[ly][lx] = (wn < N && k0 + lx < K) ? w[(size_t)wn * K + k0 + lx] : 0.f;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) acc = fmaf(xs[ly][kk], ws[lx][kk], acc);
        __syncthreads();
    }
    if (m < M && n < N) y[(size_t)m * N + n] = acc + (bias ? bias[n] : 0.f);
}

}  // namespace lin
}  // namespace grl

using namespace grl;

extern "C" int grl_linear(grl_device* dev, const void* x, const void* w, const float* bias, float* y, int m, int k, int n,
                          int in_dtype) {
    GRL_REQUIRE(dev && x && w && y, "NULL argument");
    GRL_REQUIRE(m > 0 && k > 0 && n > 0, "bad shape (%d,%d,%d)", m, k, n);
    GRL_REQUIRE(in_dtype == GRL_F32 || in_dtype == GRL_BF16, "unknown in_dtype");
    DeviceGuard g(dev->ordinal);
    if (in_dtype == GRL_F32) {
        lin::linear_f32_kernel<<<dim3((n + 15) / 16, (m + 15) / 16), 256, 0, dev->stream>>>(
            static_cast<const float*>(x), static_cast<const float*>(w), bias, y, m, k, n);
        GRL_LAUNCHED("linear_f32_kernel");
        return GRL_OK;
    }
    GRL_REQUIRE(k % 8 == 0, "the tensor-core projection needs the inner dimension to be a multiple of 8 (got %d): rows must "
                            "start on 16-byte boundaries for TMA", k);
    GRL_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)y % 8 == 0), "x, w must be 16-byte aligned");
    CUtensorMap tx, tw;
    TmapKey kx{}, kw{};
    kx.ptr = x; kx.rank = 2; kx.swizzle_128b = 1; kx.dims[0] = (uint64_t)k; kx.dims[1] = (uint64_t)m; kx.strides[0] = (uint64_t)k * 2;
    kx.box[0] = lin::BK; kx.box[1] = lin::BM;
    kw = kx; kw.ptr = w; kw.dims[1] = (uint64_t)n; kw.box[1] = lin::BN;
    int rc = get_tensor_map(dev, kx, &tx);
    if (!rc) rc = get_tensor_map(dev, kw, &tw);
    if (rc) return rc;
    lin::Args a{};
    a.bias = bias; a.y = y; a.status = dev->d_status; a.M = m; a.N = n; a.K = k; a.wait_limit = dev->wait_limit_cycles;
    dev->status_dirty = true;
    static bool attr_set[64] = {};
    if (!attr_set[dev->ordinal & 63]) {
        GRL_CUDA(cudaFuncSetAttribute(lin::linear_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lin::SMEM_TOTAL));
        attr_set[dev->ordinal & 63] = true;
    }
    dim3 grid((n + lin::BN - 1) / lin::BN, (m + lin::BM - 1) / lin::BM);
    lin::linear_sm100_kernel<<<grid, lin::kThreads, lin::SMEM_TOTAL, dev->stream>>>(tx, tw, a);
    GRL_LAUNCHED("linear_sm100_kernel");
    return GRL_OK;
}
