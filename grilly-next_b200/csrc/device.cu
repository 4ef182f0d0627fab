// Device, memory, stream, event and graph entry points of the C ABI, plus small element-wise
// kernels (cast, RoPE table).  See include/grilly_cuda.h for the reference pieces replaced.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <chrono>
#include <thread>

#include "common.cuh"

namespace grl {

static thread_local char t_err[512] = "";
std::atomic<long long> g_launches{0};

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
    return code;
}

RopeFreq make_rope_freq(int head_dim, float theta, float scaling) {
    RopeFreq f{};
    double sc = (scaling == 0.0f) ? 1.0 : (double)scaling;
    for (int i = 0; i < head_dim / 2 && i < 128; ++i)
        f.inv_freq[i] = pow((double)theta, -2.0 * (double)i / (double)head_dim) / sc;
    return f;
}

__global__ void rope_table_kernel(float2* table, int n_pos, int half, RopeFreq f) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_pos * half) return;
    int pos = idx / half, i = idx % half;
    float c, s;
    rope_sincos(pos, f.inv_freq[i], &c, &s);
    table[idx] = make_float2(c, s);
}

int get_rope_table(grl_device* dev, int n_pos, int head_dim, float theta, float scaling,
                   const float2** out) {
    uint32_t tb, sb;
    memcpy(&tb, &theta, 4);
    memcpy(&sb, &scaling, 4);
    auto key = std::make_tuple(head_dim, tb, sb);
    std::lock_guard<std::mutex> lock(dev->mu);
    auto it = dev->rope_tables.find(key);
    if (it != dev->rope_tables.end() && it->second.first >= n_pos) {
        *out = it->second.second;
        return GRL_OK;
    }
    // Row contents do not depend on the table's length: keep ONE table per (head_dim, theta, scaling), sized to
    // the next power of two, and replace it when a longer sequence arrives.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(dev->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
        return set_error(GRL_ERR_INVALID,
                         "the RoPE table for %d positions does not exist yet and cannot be built while the stream is "
                         "capturing: call grl_rope_table_prepare (or run the op once) before the capture", n_pos);
    int cap_pos = 256;
    while (cap_pos < n_pos) cap_pos <<= 1;
    float2* t = nullptr;
    int half = head_dim / 2;
    GRL_CUDA(cudaMalloc(&t, sizeof(float2) * (size_t)cap_pos * half));
    const size_t n = (size_t)cap_pos * half;
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, dev->stream>>>(t, cap_pos, half,
                                                                            make_rope_freq(head_dim, theta, scaling));
    GRL_LAUNCHED("rope_table_kernel");
    if (it != dev->rope_tables.end()) dev->retired_tables.push_back(it->second.second);
    dev->rope_tables[key] = std::make_pair(cap_pos, t);
    *out = t;
    return GRL_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int get_tensor_map(grl_device* dev, const TmapKey& key, CUtensorMap* out) {
    constexpr size_t kMaxCached = 64;
    std::lock_guard<std::mutex> lock(dev->mu);
    for (auto& e : dev->tmaps)
        if (memcmp(&e.first, &key, sizeof(TmapKey)) == 0) {
            *out = e.second;
            ++dev->tmap_hits;
            return GRL_OK;
        }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(GRL_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[3] = {key.dims[0], key.dims[1], key.dims[2]};
    cuuint64_t strides[2] = {key.strides[0], key.strides[1]};
    cuuint32_t box[3] = {key.box[0], key.box[1], key.box[2]};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, key.bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, key.rank, const_cast<void*>(key.ptr), dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    key.swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(GRL_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    ++dev->tmap_misses;
    if (dev->tmaps.size() < kMaxCached) {
        dev->tmaps.emplace_back(key, *out);
    } else {
        dev->tmaps[dev->tmap_next] = std::make_pair(key, *out);   // round robin
        dev->tmap_next = (dev->tmap_next + 1) % kMaxCached;
    }
    return GRL_OK;
}

template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ src, D* __restrict__ dst, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) store_from_float<D>(dst + i, load_as_float<S>(src + i));
}

// 8 elements per thread with 16/32-byte accesses; n8 = n / 8.
__global__ void cast_f32_bf16_vec8(const float4* __restrict__ src, uint4* __restrict__ dst, size_t n8) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n8; i += stride) {
        float4 a = src[2 * i], b = src[2 * i + 1];
        __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
        uint4 o;
        o.x = *reinterpret_cast<uint32_t*>(&p0);
        o.y = *reinterpret_cast<uint32_t*>(&p1);
        o.z = *reinterpret_cast<uint32_t*>(&p2);
        o.w = *reinterpret_cast<uint32_t*>(&p3);
        dst[i] = o;
    }
}

}  // namespace grl

using namespace grl;

extern "C" {

const char* grl_last_error(void) { return t_err; }

int64_t grl_launch_count(void) { return (int64_t)g_launches.load(); }

int grl_device_count(int* count) {
    GRL_REQUIRE(count, "count is NULL");
    cudaError_t e = cudaGetDeviceCount(count);
    if (e != cudaSuccess) {
        *count = 0;
        return set_error(GRL_ERR_CUDA, "cudaGetDeviceCount failed: %s", cudaGetErrorString(e));
    }
    return GRL_OK;
}

int grl_device_open(int ordinal, grl_device** out) {
    GRL_REQUIRE(out, "out is NULL");
    int n = 0;
    GRL_CUDA(cudaGetDeviceCount(&n));
    GRL_REQUIRE(ordinal >= 0 && ordinal < n, "device ordinal %d out of range (%d devices)", ordinal, n);
    GRL_CUDA(cudaSetDevice(ordinal));
    grl_device* d = new grl_device();
    d->ordinal = ordinal;
    cudaError_t e = cudaGetDeviceProperties(&d->prop, ordinal);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&d->own_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete d;
        return set_error(GRL_ERR_CUDA, "device open failed: %s", cudaGetErrorString(e));
    }
    d->stream = d->own_stream;
    const size_t status_bytes = (4 + grl_device::kCounterInts) * sizeof(int32_t);
    if (cudaMalloc(&d->d_status, status_bytes) != cudaSuccess ||
        cudaMemset(d->d_status, 0, status_bytes) != cudaSuccess ||
        cudaHostAlloc(&d->h_status, 4 * sizeof(int32_t), cudaHostAllocDefault) != cudaSuccess) {
        cudaFree(d->d_status);
        cudaStreamDestroy(d->own_stream);
        delete d;
        return set_error(GRL_ERR_OOM, "could not allocate the device status word");
    }
    if (d->prop.major != 10) {
        int maj = d->prop.major, min = d->prop.minor;
        cudaFree(d->d_status);
        cudaFreeHost(d->h_status);
        cudaStreamDestroy(d->own_stream);
        delete d;
        return set_error(GRL_ERR_UNSUPPORTED,
                         "this library is built for sm_100a only; device %d is sm_%d%d", ordinal, maj, min);
    }
    d->d_counters = d->d_status + 4;
    *out = d;
    return GRL_OK;
}

int grl_device_close(grl_device* dev) {
    if (!dev) return GRL_OK;
    DeviceGuard g(dev->ordinal);
    cudaStreamSynchronize(dev->stream);
    for (auto& kv : dev->rope_tables) cudaFree(kv.second.second);
    for (float2* t : dev->retired_tables) cudaFree(t);
    cudaFree(dev->d_status);
    cudaFreeHost(dev->h_status);
    cudaStreamDestroy(dev->own_stream);
    delete dev;
    return GRL_OK;
}

int grl_device_get_info(grl_device* dev, grl_device_info* info) {
    GRL_REQUIRE(dev && info, "NULL argument");
    memset(info, 0, sizeof(*info));
    strncpy(info->name, dev->prop.name, sizeof(info->name) - 1);
    info->ordinal = dev->ordinal;
    info->cc_major = dev->prop.major;
    info->cc_minor = dev->prop.minor;
    info->sm_count = dev->prop.multiProcessorCount;
    info->total_mem_bytes = (int64_t)dev->prop.totalGlobalMem;
    info->l2_bytes = dev->prop.l2CacheSize;
    info->smem_per_block_optin = (int64_t)dev->prop.sharedMemPerBlockOptin;
    return GRL_OK;
}

int grl_device_use_stream(grl_device* dev, void* cuda_stream) {
    GRL_REQUIRE(dev, "dev is NULL");
    dev->stream = cuda_stream ? (cudaStream_t)cuda_stream : dev->own_stream;
    return GRL_OK;
}

int grl_device_set_wait_limits(grl_device* dev, uint64_t barrier_wait_cycles, uint64_t peer_wait_cycles) {
    GRL_REQUIRE(dev, "dev is NULL");
    const uint64_t cap = 20000000000ull;   // ~10 s: a wait never becomes unbounded
    dev->wait_limit_cycles = barrier_wait_cycles ? (long long)(barrier_wait_cycles < cap ? barrier_wait_cycles : cap)
                                                 : kDefaultWaitLimitCycles;
    dev->peer_wait_limit_cycles = peer_wait_cycles ? (long long)(peer_wait_cycles < cap ? peer_wait_cycles : cap)
                                                   : kDefaultPeerWaitLimitCycles;
    return GRL_OK;
}

int grl_rope_table_prepare(grl_device* dev, int n_pos, int head_dim, float theta, float scaling) {
    GRL_REQUIRE(dev, "dev is NULL");
    GRL_REQUIRE(n_pos > 0 && head_dim > 0 && head_dim % 2 == 0 && head_dim <= 256 && theta > 0.f, "bad RoPE table shape");
    DeviceGuard g(dev->ordinal);
    const float2* t = nullptr;
    return get_rope_table(dev, n_pos, head_dim, theta, scaling == 0.f ? 1.f : scaling, &t);
}

int grl_tensor_map_cache_stats(grl_device* dev, int64_t* hits, int64_t* misses, int64_t* cached) {
    GRL_REQUIRE(dev, "dev is NULL");
    std::lock_guard<std::mutex> lock(dev->mu);
    if (hits) *hits = dev->tmap_hits;
    if (misses) *misses = dev->tmap_misses;
    if (cached) *cached = (int64_t)dev->tmaps.size();
    return GRL_OK;
}

int grl_malloc(grl_device* dev, size_t bytes, void** out) {
    GRL_REQUIRE(dev && out, "NULL argument");
    DeviceGuard g(dev->ordinal);
    *out = nullptr;
    if (bytes == 0) bytes = 256;
    GRL_CUDA(cudaMalloc(out, bytes));
    return GRL_OK;
}

int grl_free(grl_device* dev, void* ptr) {
    GRL_REQUIRE(dev, "dev is NULL");
    if (!ptr) return GRL_OK;
    DeviceGuard g(dev->ordinal);
    GRL_CUDA(cudaFree(ptr));
    {   // a later allocation may reuse the address with another shape: forget the maps built on it
        std::lock_guard<std::mutex> lock(dev->mu);
        for (size_t i = 0; i < dev->tmaps.size();) {
            if (dev->tmaps[i].first.ptr == ptr) { dev->tmaps[i] = dev->tmaps.back(); dev->tmaps.pop_back(); }
            else ++i;
        }
        if (dev->tmap_next >= dev->tmaps.size()) dev->tmap_next = 0;
    }
    return GRL_OK;
}

int grl_host_alloc(size_t bytes, void** out) {
    GRL_REQUIRE(out, "out is NULL");
    GRL_CUDA(cudaMallocHost(out, bytes ? bytes : 16));
    return GRL_OK;
}

int grl_host_free(void* ptr) {
    if (ptr) GRL_CUDA(cudaFreeHost(ptr));
    return GRL_OK;
}

int grl_memcpy_h2d(grl_device* dev, void* dst, const void* src_host, size_t bytes) {
    GRL_REQUIRE(dev && (bytes == 0 || (dst && src_host)), "NULL argument");
    DeviceGuard g(dev->ordinal);
    GRL_CUDA(cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, dev->stream));
    return GRL_OK;
}

int grl_memcpy_d2h(grl_device* dev, void* dst_host, const void* src, size_t bytes) {
    GRL_REQUIRE(dev && (bytes == 0 || (dst_host && src)), "NULL argument");
    DeviceGuard g(dev->ordinal);
    GRL_CUDA(cudaMemcpyAsync(dst_host, src, bytes, cudaMemcpyDeviceToHost, dev->stream));
    return GRL_OK;
}

int grl_memcpy_d2d(grl_device* dev, void* dst, const void* src, size_t bytes) {
    GRL_REQUIRE(dev && (bytes == 0 || (dst && src)), "NULL argument");
    DeviceGuard g(dev->ordinal);
    GRL_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, dev->stream));
    return GRL_OK;
}

int grl_memset(grl_device* dev, void* dst, int value, size_t bytes) {
    GRL_REQUIRE(dev && (bytes == 0 || dst), "NULL argument");
    DeviceGuard g(dev->ordinal);
    GRL_CUDA(cudaMemsetAsync(dst, value, bytes, dev->stream));
    return GRL_OK;
}

// A kernel with bounded waits leaves its failure in the device status word.  The word is copied to
// pinned host memory by the same stream AHEAD of the wait, so that one wait serves both.
static bool queue_status_copy(grl_device* dev) {
    if (!dev->status_dirty) return false;
    dev->status_dirty = false;
    return cudaMemcpyAsync(dev->h_status, dev->d_status, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, dev->stream) ==
           cudaSuccess;
}

static int report_kernel_status(grl_device* dev, bool copied) {
    if (!copied) return GRL_OK;
    const int32_t* st = dev->h_status;
    if (st[0] == 0) return GRL_OK;
    // a kernel that gave up may have left arrival counters half-way: clear them with the status
    GRL_CUDA(cudaMemsetAsync(dev->d_status, 0, (4 + grl_device::kCounterInts) * sizeof(int32_t), dev->stream));
    // [1] = kind << 28 | detail: 1 prefill (index of the mbarrier whose wait ran out; [3] = CTA),
    // 2 decode (mbarrier index; [2],[3] = CTA), 3 cross-GPU merge (peer that did not post; [2] = step, [3] = rank),
    // 4 append (a sequence without room; [2] = sequence, [3] = its length), 5 linear projection (mbarrier index)
    const int code = st[0] == GRL_ERR_TIMEOUT ? GRL_ERR_TIMEOUT : GRL_ERR_KERNEL;
    const unsigned int kind = (unsigned int)st[1] >> 28, detail = (unsigned int)st[1] & 0x0fffffffu;
    switch (kind) {
        case 1: return set_error(code, "prefill kernel: a wait ran out (mbarrier %u, CTA %d)", detail, st[3]);
        case 2: return set_error(code, "decode kernel: a wait ran out (mbarrier %u, CTA %d,%d)", detail, st[2], st[3]);
        case 3: return set_error(code, "cross-GPU merge on rank %d: peer %u did not post step %d within the wait limit",
                                 st[3], detail, st[2]);
        case 5: return set_error(code, "linear kernel: a wait ran out (mbarrier %u, CTA %d,%d)", detail, st[2], st[3]);
        case 4: return set_error(code, "kv append: sequence %d (length %d) has no room for the new tokens", st[2], st[3]);
        default: return set_error(code, "kernel reported failure %d (detail 0x%x, %d, %d)", st[0], st[1], st[2], st[3]);
    }
}

int grl_sync(grl_device* dev, uint64_t timeout_ns) {
    GRL_REQUIRE(dev, "dev is NULL");
    DeviceGuard g(dev->ordinal);
    const bool copied = queue_status_copy(dev);
    if (timeout_ns == 0) {
        GRL_CUDA(cudaStreamSynchronize(dev->stream));
        return report_kernel_status(dev, copied);
    }
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t e = cudaStreamQuery(dev->stream);
        if (e == cudaSuccess) return report_kernel_status(dev, copied);
        if (e != cudaErrorNotReady)
            return set_error(GRL_ERR_CUDA, "stream failed: %s", cudaGetErrorString(e));
        auto dt = std::chrono::steady_clock::now() - t0;
        const uint64_t ns = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(dt).count();
        if (ns > timeout_ns)
            return set_error(GRL_ERR_TIMEOUT, "stream did not finish within %llu ns",
                             (unsigned long long)timeout_ns);
        // a decode step is over in ~100 us and a sleep costs 50+ us of timer slack: poll first, sleep later
        if (ns > 500000) std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
}

int grl_event_create(grl_event** out) {
    GRL_REQUIRE(out, "out is NULL");
    grl_event* e = new grl_event();
    cudaError_t err = cudaEventCreate(&e->ev);
    if (err != cudaSuccess) {
        delete e;
        return set_error(GRL_ERR_CUDA, "cudaEventCreate failed: %s", cudaGetErrorString(err));
    }
    *out = e;
    return GRL_OK;
}

int grl_event_create_untimed(grl_event** out) {
    GRL_REQUIRE(out, "out is NULL");
    grl_event* e = new grl_event();
    cudaError_t err = cudaEventCreateWithFlags(&e->ev, cudaEventDisableTiming);
    if (err != cudaSuccess) {
        delete e;
        return set_error(GRL_ERR_CUDA, "cudaEventCreate failed: %s", cudaGetErrorString(err));
    }
    *out = e;
    return GRL_OK;
}

int grl_event_destroy(grl_event* ev) {
    if (ev) {
        cudaEventDestroy(ev->ev);
        delete ev;
    }
    return GRL_OK;
}

int grl_event_record(grl_device* dev, grl_event* ev) {
    GRL_REQUIRE(dev && ev, "NULL argument");
    DeviceGuard g(dev->ordinal);
    GRL_CUDA(cudaEventRecord(ev->ev, dev->stream));
    return GRL_OK;
}

int grl_event_wait(grl_device* dev, grl_event* ev) {
    GRL_REQUIRE(dev && ev, "NULL argument");
    DeviceGuard g(dev->ordinal);
    GRL_CUDA(cudaStreamWaitEvent(dev->stream, ev->ev, 0));
    return GRL_OK;
}

int grl_event_sync(grl_event* ev) {
    GRL_REQUIRE(ev, "ev is NULL");
    GRL_CUDA(cudaEventSynchronize(ev->ev));
    return GRL_OK;
}

int grl_event_elapsed_ms(grl_event* start, grl_event* stop, float* ms) {
    GRL_REQUIRE(start && stop && ms, "NULL argument");
    GRL_CUDA(cudaEventSynchronize(stop->ev));
    GRL_CUDA(cudaEventElapsedTime(ms, start->ev, stop->ev));
    return GRL_OK;
}

int grl_graph_begin(grl_device* dev) {
    GRL_REQUIRE(dev, "dev is NULL");
    DeviceGuard g(dev->ordinal);
    GRL_CUDA(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
    return GRL_OK;
}

int grl_graph_end(grl_device* dev, grl_graph** out) {
    GRL_REQUIRE(dev && out, "NULL argument");
    DeviceGuard g(dev->ordinal);
    grl_graph* gr = new grl_graph();
    cudaError_t e = cudaStreamEndCapture(dev->stream, &gr->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&gr->exec, gr->graph, 0);
    if (e != cudaSuccess) {
        if (gr->graph) cudaGraphDestroy(gr->graph);
        delete gr;
        return set_error(GRL_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    }
    *out = gr;
    return GRL_OK;
}

int grl_graph_launch(grl_device* dev, grl_graph* gr) {
    GRL_REQUIRE(dev && gr && gr->exec, "NULL argument");
    DeviceGuard g(dev->ordinal);
    GRL_CUDA(cudaGraphLaunch(gr->exec, dev->stream));
    // The replayed kernels may write the status word (bounded waits): the next grl_sync must read it.
    dev->status_dirty = true;
    return GRL_OK;
}

int grl_graph_destroy(grl_graph* gr) {
    if (gr) {
        if (gr->exec) cudaGraphExecDestroy(gr->exec);
        if (gr->graph) cudaGraphDestroy(gr->graph);
        delete gr;
    }
    return GRL_OK;
}

int grl_cast(grl_device* dev, const void* src, int src_dtype, void* dst, int dst_dtype, size_t n) {
    GRL_REQUIRE(dev && (n == 0 || (src && dst)), "NULL argument");
    if (n == 0) return GRL_OK;
    DeviceGuard g(dev->ordinal);
    int blocks = (int)((n + 255) / 256 < (size_t)dev->prop.multiProcessorCount * 16
                           ? (n + 255) / 256
                           : (size_t)dev->prop.multiProcessorCount * 16);
    if (src_dtype == GRL_F32 && dst_dtype == GRL_BF16) {
        if (n % 8 == 0 && ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0)) {
            cast_f32_bf16_vec8<<<blocks, 256, 0, dev->stream>>>((const float4*)src, (uint4*)dst, n / 8);
        } else {
            cast_kernel<float, __nv_bfloat16><<<blocks, 256, 0, dev->stream>>>(
                (const float*)src, (__nv_bfloat16*)dst, n);
        }
    } else if (src_dtype == GRL_BF16 && dst_dtype == GRL_F32) {
        cast_kernel<__nv_bfloat16, float><<<blocks, 256, 0, dev->stream>>>(
            (const __nv_bfloat16*)src, (float*)dst, n);
    } else if (src_dtype == dst_dtype && (src_dtype == GRL_F32 || src_dtype == GRL_BF16)) {
        GRL_CUDA(cudaMemcpyAsync(dst, src, n * (src_dtype == GRL_F32 ? 4 : 2), cudaMemcpyDeviceToDevice,
                                 dev->stream));
        return GRL_OK;
    } else {
        return set_error(GRL_ERR_INVALID, "unknown dtype pair %d -> %d", src_dtype, dst_dtype);
    }
    GRL_LAUNCHED("cast");
    return GRL_OK;
}

}  // extern "C"
