// GrillyDevice, BufferPool, PipelineCache, CommandBatch over the CUDA C ABI.
#include <cstdlib>
#include <cstring>

#include "grilly/buffer_pool.h"
#include "grilly/command_batch.h"
#include "grilly/device.h"
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
    std::lock_guard<std::mutex> lock(mu_);
    return stats_;
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
