#pragma once
// Host-side helper threads of the op layer: a fixed pool that runs one parallel loop at a time.  Used
// to round float32 host tensors to bf16 while earlier chunks are already crossing the host link -- the
// reference's ops are synchronous host-pointer calls, so whatever the host can do in parallel with the
// copy engines shortens the call.
#include <condition_variable>
#include <cstddef>
#include <cstdint>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace grilly {

class HostWorkers {
public:
    /// Process-wide pool; threads = min(hardware threads, 32), overridden by GRILLY_HOST_THREADS.
    static HostWorkers& instance();
    ~HostWorkers();
    int threads() const { return int(workers_.size()) + 1; }
    /// Calls fn(part, parts) for part in [0, parts) on the pool and the calling thread; returns when all are done.
    void parallel(const std::function<void(int, int)>& fn);

private:
    HostWorkers();
    void loop(int id);
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable start_, done_;
    const std::function<void(int, int)>* job_ = nullptr;
    uint64_t generation_ = 0;
    int pending_ = 0;
    bool stop_ = false;
};

/// Round n float32 values to bf16 (round-to-nearest-even, NaN -> 0x7fff: what the device cast produces),
/// split over the pool.
void convertF32ToBF16(const float* src, uint16_t* dst, size_t n);

}  // namespace grilly
