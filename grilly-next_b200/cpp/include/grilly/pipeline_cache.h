#pragma once
// Kernel-plan registry.  In the reference, PipelineCache holds SPIR-V pipelines and an LRU of
// descriptor sets (cpp/include/grilly/pipeline_cache.h:35-115).  CUDA kernels are linked into
// the library, so what remains is the bookkeeping the bindings expose: named plans looked up
// per dispatch, with the same hits / misses / evictions / cachedSets counters.  The descriptor
// sets themselves have a counterpart inside the CUDA library: the tensor maps (TMA descriptors)
// of a launch are cached per (pointer, shape, box) and reported here beside the plan counters.
#include <cstdint>
#include <list>
#include <mutex>
#include <string>
#include <unordered_map>

#include "grilly/device.h"

namespace grilly {

struct CacheStats {
    uint64_t hits = 0, misses = 0, evictions = 0, cachedSets = 0;
    // encoded tensor maps kept by the CUDA library per (pointer, shape, box): grl_tensor_map_cache_stats
    uint64_t tensorMapHits = 0, tensorMapMisses = 0, tensorMapsCached = 0;
};

class PipelineCache {
public:
    explicit PipelineCache(GrillyDevice& device, size_t capacity = 256) : device_(device), capacity_(capacity) {}
    /// Records a lookup of plan `key` (op name + shape signature); returns true on a hit.
    bool getOrCreate(const std::string& key);
    bool hasShader(const std::string&) const { return true; }  // kernels are always present
    CacheStats cacheStats() const;
    GrillyDevice& device() { return device_; }

private:
    GrillyDevice& device_;
    size_t capacity_;
    mutable std::mutex mu_;
    std::list<std::string> lru_;
    std::unordered_map<std::string, std::list<std::string>::iterator> map_;
    CacheStats stats_;
};

}  // namespace grilly
