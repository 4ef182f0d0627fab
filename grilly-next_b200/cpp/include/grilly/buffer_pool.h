#pragma once
// cudaMalloc-backed bucket pool: HBM buffers instead of the reference's host-visible VMA
// buffers (cpp/include/grilly/buffer_pool.h:18-113).  Same interface: acquire / release /
// upload / download / stats, power-of-two buckets from 256 B to 256 MiB with at most 32 cached
// buffers per bucket (cpp/src/buffer_pool.cpp:64-82,128-175); larger requests are exact-size.
#include <cstddef>
#include <cstdint>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "grilly/device.h"

namespace grilly {

struct GrillyBuffer {
    void* dptr = nullptr;      // device pointer (HBM)
    size_t size = 0;           // requested bytes
    size_t bucketSize = 0;     // allocated bytes
    bool valid() const { return dptr != nullptr; }
};

struct PoolStats {
    uint64_t hits = 0, misses = 0, allocations = 0, totalAcquired = 0, totalReleased = 0;
};

class BufferPool {
public:
    explicit BufferPool(GrillyDevice& device);
    ~BufferPool();
    BufferPool(const BufferPool&) = delete;

    GrillyBuffer acquire(size_t size);
    void release(GrillyBuffer& buf);
    /// Host -> device copy through the context stream (asynchronous; ordered with launches).
    void upload(const GrillyBuffer& buf, const void* host, size_t bytes);
    /// Device -> host copy; returns after the data is in `host`.
    void download(const GrillyBuffer& buf, void* host, size_t bytes);
    PoolStats stats() const;
    GrillyDevice& device() { return device_; }

    static size_t bucketFor(size_t size);

private:
    GrillyDevice& device_;
    mutable std::mutex mu_;
    std::unordered_map<size_t, std::vector<void*>> free_;
    PoolStats stats_;
};

}  // namespace grilly
