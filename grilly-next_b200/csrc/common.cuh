// Shared host/device helpers for the C-ABI kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "grilly_cuda.h"

namespace grl {
// Key of a cached tiled tensor map (bf16 elements): everything cuTensorMapEncodeTiled is given.
struct TmapKey {
    const void* ptr;
    uint32_t rank;
    uint32_t swizzle_128b;     // 1: 128-byte swizzle, 0: none
    uint64_t dims[3];
    uint64_t strides[2];       // bytes, dimensions 1..rank-1
    uint32_t box[3];
    uint32_t bytes;            // 1: uint8 elements; 0: bf16 (two bytes)
};
constexpr long long kDefaultWaitLimitCycles = 2000000000LL;       // ~1 s at 2 GHz: mbarrier waits inside a kernel
constexpr long long kDefaultPeerWaitLimitCycles = 1000000000LL;   // ~0.5 s: a peer GPU that never posts
}  // namespace grl

struct grl_device {
    int ordinal = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;   // the stream launches go to (own_stream or an adopted one)
    cudaDeviceProp prop{};
    std::mutex mu;
    // RoPE cos/sin tables, float2 (cos, sin) per (position, pair), one per (head_dim, theta bits,
    // scaling bits); a table covers `first` positions and is replaced by a longer one on demand.
    std::map<std::tuple<int, uint32_t, uint32_t>, std::pair<int, float2*>> rope_tables;
    std::vector<float2*> retired_tables;   // replaced tables: kernels in flight may still read them; freed at close
    // Tensor maps already encoded for this device (the descriptor-set cache of the reference's
    // PipelineCache, cpp/src/pipeline_cache.cpp:217-305): a launch looks its maps up by
    // (pointer, shape, box) instead of encoding them again.
    std::vector<std::pair<grl::TmapKey, CUtensorMap>> tmaps;
    size_t tmap_next = 0;
    long long tmap_hits = 0, tmap_misses = 0;
    // Cycle budgets of the bounded device-side waits (grl_device_set_wait_limits).
    long long wait_limit_cycles = grl::kDefaultWaitLimitCycles;
    long long peer_wait_limit_cycles = grl::kDefaultPeerWaitLimitCycles;
    // Status word written by kernels with bounded waits; read back by grl_sync when dirty.
    int32_t* d_status = nullptr;   // device int32[4], followed by the arrival counters below
    bool status_dirty = false;
    int32_t* h_status = nullptr;   // pinned host int32[4]: the status word is copied here ahead of a wait
    // Arrival counters of the split-KV decode (one per (sequence, kv head), zero between launches: the
    // CTA that brings a counter to its final value resets it) and, last, the count of finished heads.
    static constexpr int kCounterSlots = 4096;
    static constexpr int kCounterInts = kCounterSlots + 1 + 2;   // + the prefill kernel's work and finished-CTA counters
    int32_t* d_counters = nullptr;   // = d_status + 4, int32[kCounterInts]
};

struct grl_event {
    cudaEvent_t ev = nullptr;
};

struct grl_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

namespace grl {

int set_error(int code, const char* fmt, ...);

// Peer inboxes of the cross-GPU merge, by value in kernel parameters (filled from grl_exchange_params).
constexpr int kMaxPeers = 16;
struct PeerExchange {
    float* inbox;                        // local: [2][world][n]
    unsigned int* flags;                 // local: [2][world][flag_slots]
    float* peer_inbox[kMaxPeers];        // the peers' inboxes mapped into this process
    unsigned int* peer_flags[kMaxPeers];
    unsigned int* seq;                   // local step counter
    int rank, world, flag_slots;
    long long wait_cycles;               // a missing peer ends in an error code after this many cycles, not in a hang
};
int fill_peer_exchange(grl_device* dev, const grl_exchange_params* p, PeerExchange* x);

// Cached cuTensorMapEncodeTiled for bf16 tensors (zero fill out of bounds, 256-byte L2 promotion).
int get_tensor_map(grl_device* dev, const TmapKey& key, CUtensorMap* out);

#ifdef __CUDACC__
// Low-latency inbox element: {value bits, step number} in one 8-byte word.  take3 reads three elements
// of one peer with the loads in flight together and repeats until all three carry step `e` (or the cycle
// limit passes: returns false).
__device__ __forceinline__ uint2 ld_pair_volatile(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ bool take3(const uint2* a, const uint2* b, const uint2* c, unsigned int e, long long t0,
                                      long long limit, float* va, float* vb, float* vc) {
    for (;;) {
        const uint2 x = ld_pair_volatile(a), y = ld_pair_volatile(b), z = ld_pair_volatile(c);
        if (x.y == e && y.y == e && z.y == e) {
            *va = __uint_as_float(x.x); *vb = __uint_as_float(y.x); *vc = __uint_as_float(z.x);
            return true;
        }
        if (clock64() - t0 > limit) return false;
    }
}
#endif
extern std::atomic<long long> g_launches;

#define GRL_CUDA(call)                                                                       \
    do {                                                                                     \
        cudaError_t _e = (call);                                                             \
        if (_e != cudaSuccess)                                                               \
            return grl::set_error(_e == cudaErrorMemoryAllocation ? GRL_ERR_OOM : GRL_ERR_CUDA, \
                                  "%s failed: %s", #call, cudaGetErrorString(_e));           \
    } while (0)

#define GRL_REQUIRE(cond, ...)                                              \
    do {                                                                    \
        if (!(cond)) return grl::set_error(GRL_ERR_INVALID, __VA_ARGS__);   \
    } while (0)

// Call after every kernel launch: counts it and turns a launch error into a status code.
#define GRL_LAUNCHED(name)                                                                    \
    do {                                                                                      \
        grl::g_launches.fetch_add(1, std::memory_order_relaxed);                              \
        cudaError_t _e = cudaGetLastError();                                                  \
        if (_e != cudaSuccess)                                                                \
            return grl::set_error(GRL_ERR_CUDA, "launch of %s failed: %s", name,              \
                                  cudaGetErrorString(_e));                                    \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int ordinal) {
        cudaGetDevice(&prev);
        if (prev != ordinal) cudaSetDevice(ordinal);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// inv_freq[i] = theta^(-2i/D) / scaling in double, for i < D/2 <= 128.
struct RopeFreq {
    double inv_freq[128];
};
RopeFreq make_rope_freq(int head_dim, float theta, float scaling);

// Device table of (cos, sin) for positions [0, >= n_pos) x pairs [0, D/2); cached per device.  Creating or
// growing a table allocates and launches, which a capturing stream does not allow: the call then fails and
// names the remedy (run the op once, or grl_rope_table_prepare, before the capture).
int get_rope_table(grl_device* dev, int n_pos, int head_dim, float theta, float scaling,
                   const float2** out);

#ifdef __CUDACC__
// cos/sin of pos * inv_freq with the product and the 2*pi reduction in double, so that the
// angle error stays near 1e-7 rad for positions up to 2^24 (a float product alone is off by
// up to pos * 2^-24 rad).
__device__ __forceinline__ void rope_sincos(int pos, double inv_freq, float* c, float* s) {
    double th = (double)pos * inv_freq;
    double k = rint(th * 0.15915494309189535);  // 1/(2*pi)
    double r = fma(-k, 6.283185307179586, th);
    r = fma(-k, 2.4492935982947064e-16, r);     // low part of 2*pi
    sincosf((float)r, s, c);
}

__device__ __forceinline__ float bf16_round(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}

template <typename T> __device__ __forceinline__ float load_as_float(const T* p);
template <> __device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat162float(*p);
}
// Where the packed value bytes of the quantised cache (GRL_FP8_INT4) live inside the value block of one
// (page, kv head), which holds page_tokens * D/2 bytes.  Byte j of a token packs elements 2j (low nibble) and 2j+1
// (high nibble) exactly as the reference packs them; only the ADDRESS of the byte is this library's choice.  Tokens
// are stored in pairs (2i, 2i+1), D bytes per pair, as D/4 words of [even token: bytes 2w, 2w+1 | odd token: bytes
// 2w, 2w+1]: one 32-bit word then holds the same four elements of two consecutive tokens, which is the pairing a
// tensor-core operand over the token axis needs, with no transpose.  The words of a pair are ordered [w % 8][w / 8]
// so that one load brings the same word of every scale group (32 elements = 8 words), and the eight pieces
// [w % 8] are XOR-swizzled by the pair index so that lanes reading the same piece of neighbouring pairs use
// different shared-memory banks.
__host__ __device__ __forceinline__ size_t quant_v_off(int token_in_page, int j, int D) {
    const int w = j >> 1, G = D >> 5;
    const int pw = ((w & 7) ^ ((token_in_page >> 1) & 7)) * G + (w >> 3);
    return (size_t)(token_in_page >> 1) * D + pw * 4 + (token_in_page & 1) * 2 + (j & 1);
}

template <typename T> __device__ __forceinline__ void store_from_float(T* p, float v);
template <> __device__ __forceinline__ void store_from_float<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_from_float<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
}
#endif

}  // namespace grl
