#pragma once
// CUDA device context of the op layer.  Same role and accessors as the reference's Vulkan
// GrillyDevice (cpp/include/grilly/device.h:16-53): picks a GPU, owns the queue (here: a CUDA
// stream inside the C-ABI handle) and reports capabilities.
#include <cstddef>
#include <stdexcept>
#include <string>

#include "grilly_cuda.h"

namespace grilly {

/// Throws std::runtime_error carrying the C-ABI's message when rc != GRL_OK.
inline void check(int rc, const char* what) {
    if (rc != GRL_OK)
        throw std::runtime_error(std::string(what) + ": " + grl_last_error());
}

class GrillyDevice {
public:
    /// Opens the GPU named by the GRILLY_GPU_INDEX environment variable (default 0), the
    /// counterpart of VK_GPU_INDEX (cpp/src/device.cpp:408-414).
    GrillyDevice();
    explicit GrillyDevice(int ordinal);
    ~GrillyDevice();
    GrillyDevice(const GrillyDevice&) = delete;
    GrillyDevice& operator=(const GrillyDevice&) = delete;

    grl_device* handle() const { return dev_; }
    const std::string& deviceName() const { return name_; }
    bool hasCooperativeMatrix() const { return true; }  // tcgen05 tensor cores
    bool hasFloat16() const { return true; }
    int smCount() const { return info_.sm_count; }
    int ordinal() const { return info_.ordinal; }
    const grl_device_info& info() const { return info_; }
    /// Two more queues on the same GPU (opened on first use) for host->device and device->host copies
    /// that overlap the kernels of the main queue -- the transfer queues a Vulkan device offers next
    /// to its compute queue.  Order between queues is set with grl_event_record / grl_event_wait.
    grl_device* uploadQueue();
    grl_device* downloadQueue();
    /// Pinned host scratch kept for the life of the device (slot 0..5): staging for converted uploads.
    static constexpr int kStagingSlots = 6;
    void* pinnedStaging(int slot, size_t bytes);
    /// Waits (without limit, ignoring errors) for everything queued on the main, upload and download queues.
    /// Error paths call it before they hand buffers back to the pool: a buffer that a kernel or a copy in
    /// flight still touches must not be re-acquired, and a timed-out submit leaves work in flight.
    void quiesce() noexcept;

private:
    void open(int ordinal);
    grl_device* dev_ = nullptr;
    grl_device* up_ = nullptr;
    grl_device* down_ = nullptr;
    void* staging_[kStagingSlots] = {};
    size_t stagingBytes_[kStagingSlots] = {};
    grl_device_info info_{};
    std::string name_;
};

}  // namespace grilly
