#pragma once
// Stream wrapper with the reference's CommandBatch surface (cpp/include/grilly/command_batch.h:20-59):
// begin() / submit().  Recording is implicit (launches go straight to the stream); submit()
// waits for the stream with the reference's 2 s limit (cpp/src/command_batch.cpp:16,145-148)
// and throws std::runtime_error on timeout or on a failure reported by a kernel.
#include <cstdint>

#include "grilly/device.h"

namespace grilly {

class CommandBatch {
public:
    explicit CommandBatch(GrillyDevice& device) : device_(device) {}
    void begin();    // throws if already recording (command_batch.cpp:70-71)
    void barrier() {}  // stream order already serialises dependent launches
    void submit();   // wait (timeoutNs) and stop recording
    void submitNoWait();  // stop recording, leave the work in flight
    bool recording() const { return recording_; }
    void setTimeoutNs(uint64_t ns) { timeoutNs_ = ns; }
    GrillyDevice& device() { return device_; }

private:
    GrillyDevice& device_;
    bool recording_ = false;
    uint64_t timeoutNs_ = 2000000000ull;
};

}  // namespace grilly
