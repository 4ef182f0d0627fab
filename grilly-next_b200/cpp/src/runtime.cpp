// GrillyDevice, BufferPool, PipelineCache, CommandBatch over the CUDA C ABI.
#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>

#if defined(__AVX2__)
#include <immintrin.h>
#endif

#include "grilly/buffer_pool.h"
#include "grilly/command_batch.h"
#include "grilly/device.h"
#include "grilly/host_workers.h"
#include "grilly/pipeline_cache.h"

namespace grilly {

// ---------------------------------------------------------------- GrillyDevice
GrillyDevice::GrillyDevice() {
    int ordinal = 0;
    if (const char* e = std::getenv("GRILLY_GPU_INDEX")) ordinal = std::atoi(e);
    open(ordinal);
}
GrillyDevice::GrillyDevice(int ordinal) { open(ordinal); }

void GrillyDevice::open(int ordinal) {
    check(grl_device_open(ordinal, &dev_), "GrillyDevice: cannot open CUDA device");
    check(grl_device_get_info(dev_, &info_), "GrillyDevice: cannot query device");
    name_ = info_.name;
}

GrillyDevice::~GrillyDevice() {
    for (void* p : staging_)
        if (p) grl_host_free(p);
    if (up_) grl_device_close(up_);
    if (down_) grl_device_close(down_);
    if (dev_) grl_device_close(dev_);
}

grl_device* GrillyDevice::uploadQueue() {
    if (!up_) check(grl_device_open(info_.ordinal, &up_), "GrillyDevice: cannot open the upload queue");
    return up_;
}

grl_device* GrillyDevice::downloadQueue() {
    if (!down_) check(grl_device_open(info_.ordinal, &down_), "GrillyDevice: cannot open the download queue");
    return down_;
}

void GrillyDevice::quiesce() noexcept {
    if (up_) grl_sync(up_, 0);
    if (dev_) grl_sync(dev_, 0);
    if (down_) grl_sync(down_, 0);
}

void* GrillyDevice::pinnedStaging(int slot, size_t bytes) {
    if (slot < 0 || slot >= kStagingSlots) throw std::runtime_error("GrillyDevice::pinnedStaging: bad slot");
    if (stagingBytes_[slot] < bytes) {
        quiesce();      // an upload in flight may still read the old staging block
        if (staging_[slot]) grl_host_free(staging_[slot]);
        staging_[slot] = nullptr;
        stagingBytes_[slot] = 0;
        check(grl_host_alloc(bytes, &staging_[slot]), "GrillyDevice: pinned staging");
        stagingBytes_[slot] = bytes;
    }
    return staging_[slot];
}

// ---------------------------------------------------------------- HostWorkers
HostWorkers& HostWorkers::instance() {
    static HostWorkers pool;
    return pool;
}

HostWorkers::HostWorkers() {
    int n = int(std::thread::hardware_concurrency());
    if (n <= 0) n = 4;
    if (n > 32) n = 32;
    // one process per GPU: the processes of a node share the host's cores
    if (const char* e = std::getenv("LOCAL_WORLD_SIZE")) n = std::max(1, n / std::max(1, std::atoi(e)));
    if (const char* e = std::getenv("GRILLY_HOST_THREADS")) n = std::max(1, std::atoi(e));
    for (int i = 1; i < n; ++i) workers_.emplace_back([this, i] { loop(i); });
}

HostWorkers::~HostWorkers() {
    {
        std::lock_guard<std::mutex> lock(mu_);
        stop_ = true;
    }
    start_.notify_all();
    for (auto& t : workers_) t.join();
}

void HostWorkers::loop(int id) {
    uint64_t seen = 0;
    for (;;) {
        const std::function<void(int, int)>* job;
        {
            std::unique_lock<std::mutex> lock(mu_);
            start_.wait(lock, [&] { return stop_ || generation_ != seen; });
            if (stop_) return;
            seen = generation_;
            job = job_;
        }
        (*job)(id, threads());
        {
            std::lock_guard<std::mutex> lock(mu_);
            if (--pending_ == 0) done_.notify_one();
        }
    }
}

void HostWorkers::parallel(const std::function<void(int, int)>& fn) {
    {
        std::lock_guard<std::mutex> lock(mu_);
        job_ = &fn;
        pending_ = int(workers_.size());
        ++generation_;
    }
    start_.notify_all();
    fn(0, threads());
    std::unique_lock<std::mutex> lock(mu_);
    done_.wait(lock, [&] { return pending_ == 0; });
}

void convertF32ToBF16(const float* src, uint16_t* dst, size_t n) {
    auto scalar = [src, dst](size_t i0, size_t i1) {
        const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
        for (size_t i = i0; i < i1; ++i) {
            const uint32_t u = s[i];
            const uint32_t rounded = (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
            dst[i] = uint16_t((u & 0x7fffffffu) > 0x7f800000u ? 0x7fffu : rounded);
        }
    };
    auto range = [&](size_t i0, size_t i1) {
#if defined(__AVX2__)
        // 16 values per step; results leave with streaming stores (the destination is staging memory that
        // only the copy engine reads next, so it should not displace the source in the caches).
        size_t i = i0;
        while (i < i1 && (reinterpret_cast<uintptr_t>(dst + i) & 31u)) ++i;
        scalar(i0, i);
        const __m256i bias = _mm256_set1_epi32(0x7fff), one = _mm256_set1_epi32(1);
        const __m256i absmask = _mm256_set1_epi32(0x7fffffff), inf = _mm256_set1_epi32(0x7f800000);
        const __m256i qnan = _mm256_set1_epi32(0x7fff);
        for (; i + 16 <= i1; i += 16) {
            __m256i a = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(src + i));
            __m256i b = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(src + i + 8));
            auto round = [&](__m256i u) {
                const __m256i lsb = _mm256_and_si256(_mm256_srli_epi32(u, 16), one);
                const __m256i r = _mm256_srli_epi32(_mm256_add_epi32(_mm256_add_epi32(u, bias), lsb), 16);
                const __m256i isnan = _mm256_cmpgt_epi32(_mm256_and_si256(u, absmask), inf);
                return _mm256_blendv_epi8(r, qnan, isnan);
            };
            a = round(a);
            b = round(b);
            __m256i p = _mm256_packus_epi32(a, b);                  // lanes: a0-3 b0-3 | a4-7 b4-7
            p = _mm256_permute4x64_epi64(p, 0xD8);                  // a0-3 a4-7 b0-3 b4-7
            _mm256_stream_si256(reinterpret_cast<__m256i*>(dst + i), p);
        }
        _mm_sfence();
        scalar(i, i1);
#else
        scalar(i0, i1);
#endif
    };
    if (n < (1u << 16)) {
        range(0, n);
        return;
    }
    HostWorkers::instance().parallel([&](int part, int parts) {
        size_t per = (n + size_t(parts) - 1) / size_t(parts);
        per = (per + 63) / 64 * 64;
        const size_t i0 = std::min(n, per * size_t(part)), i1 = std::min(n, i0 + per);
        range(i0, i1);
    });
}

// ---------------------------------------------------------------- BufferPool
static constexpr size_t kMinBucket = 256;
static constexpr size_t kMaxBucket = 256ull << 20;
static constexpr size_t kMaxPerBucket = 32;

BufferPool::BufferPool(GrillyDevice& device) : device_(device) {}

BufferPool::~BufferPool() {
    for (auto& kv : free_)
        for (void* p : kv.second) grl_free(device_.handle(), p);
}

size_t BufferPool::bucketFor(size_t size) {
    if (size > kMaxBucket) return size;   // exact-size allocation above the largest bucket
    size_t b = kMinBucket;
    while (b < size) b <<= 1;
    return b;
}

GrillyBuffer BufferPool::acquire(size_t size) {
    GrillyBuffer buf;
    buf.size = size;
    buf.bucketSize = bucketFor(size ? size : 1);
    {
        std::lock_guard<std::mutex> lock(mu_);
        stats_.totalAcquired++;
        auto it = free_.find(buf.bucketSize);
        if (it != free_.end() && !it->second.empty()) {
            buf.dptr = it->second.back();
            it->second.pop_back();
            stats_.hits++;
            return buf;
        }
        stats_.misses++;
        stats_.allocations++;
    }
    check(grl_malloc(device_.handle(), buf.bucketSize, &buf.dptr), "BufferPool::acquire");
    return buf;
}

void BufferPool::release(GrillyBuffer& buf) {
    if (!buf.dptr) return;
    bool keep = false;
    {
        std::lock_guard<std::mutex> lock(mu_);
        stats_.totalReleased++;
        auto& v = free_[buf.bucketSize];
        if (buf.bucketSize <= kMaxBucket && v.size() < kMaxPerBucket) {
            v.push_back(buf.dptr);
            keep = true;
        }
    }
    if (!keep) {
        // a buffer may still be read by work in flight on the stream
        grl_sync(device_.handle(), 0);
        grl_free(device_.handle(), buf.dptr);
    }
    buf = GrillyBuffer{};
}

void BufferPool::upload(const GrillyBuffer& buf, const void* host, size_t bytes) {
    if (bytes > buf.bucketSize) throw std::runtime_error("BufferPool::upload: size exceeds the buffer");
    check(grl_memcpy_h2d(device_.handle(), buf.dptr, host, bytes), "BufferPool::upload");
}

void BufferPool::download(const GrillyBuffer& buf, void* host, size_t bytes) {
    if (bytes > buf.bucketSize) throw std::runtime_error("BufferPool::download: size exceeds the buffer");
    check(grl_memcpy_d2h(device_.handle(), host, buf.dptr, bytes), "BufferPool::download");
    check(grl_sync(device_.handle(), 0), "BufferPool::download");
}

PoolStats BufferPool::stats() const {
    std::lock_guard<std::mutex> lock(mu_);
    return stats_;
}

// ---------------------------------------------------------------- PipelineCache
bool PipelineCache::getOrCreate(const std::string& key) {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = map_.find(key);
    if (it != map_.end()) {
        lru_.splice(lru_.begin(), lru_, it->second);
        stats_.hits++;
        return true;
    }
    stats_.misses++;
    lru_.push_front(key);
    map_[key] = lru_.begin();
    if (map_.size() > capacity_) {
        map_.erase(lru_.back());
        lru_.pop_back();
        stats_.evictions++;
    }
    stats_.cachedSets = map_.size();
    return false;
}

CacheStats PipelineCache::cacheStats() const {
    CacheStats s;
    {
        std::lock_guard<std::mutex> lock(mu_);
        s = stats_;
    }
    // the tensor maps the library keeps per (pointer, shape, box): the descriptor sets of this build
    int64_t h = 0, m = 0, c = 0;
    if (grl_tensor_map_cache_stats(device_.handle(), &h, &m, &c) == GRL_OK) {
        s.tensorMapHits = uint64_t(h); s.tensorMapMisses = uint64_t(m); s.tensorMapsCached = uint64_t(c);
    }
    return s;
}

// ---------------------------------------------------------------- CommandBatch
void CommandBatch::begin() {
    if (recording_) throw std::runtime_error("CommandBatch::begin: already recording");
    recording_ = true;
}

void CommandBatch::submit() {
    recording_ = false;
    check(grl_sync(device_.handle(), timeoutNs_), "CommandBatch::submit");
}

void CommandBatch::submitNoWait() { recording_ = false; }

}  // namespace grilly
