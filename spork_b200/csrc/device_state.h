// Per-device state shared by the kernels of this library: SM count, the device
// status word that bounded waits report into, and cached staging buffers of
// the host-buffer entry points.  One slot per device ordinal, created on first
// use with that device current, so that host threads driving different GPUs
// (one per GPU in the M-sharded runs) never share mutable state.
#pragma once

#include <cuda_runtime.h>

#include <mutex>
#include <stddef.h>
#include <stdint.h>

// CTA-pair (tcgen05 cta_group::2) kernels are the default GEMM path.
#ifndef SPORK_DEFAULT_CTA_GROUP
#define SPORK_DEFAULT_CTA_GROUP 2
#endif

namespace spork {

constexpr int kMaxDevices = 64;

struct DeviceState {
    int ordinal = -1;
    int sm_count = 0;
    int cc_major = 0;
    uint32_t* status_word = nullptr;  // device memory, zero = healthy
    // Counter pairs the CTAs of a stream-K launch meet at (device memory behind the status word): [0] counts
    // the warps that have zeroed their share, [1] the CTAs that have left; the last one to leave zeroes both.
    // Launches take the pairs in rotation, so launches that overlap (other streams) do not share one unless
    // more than kSkCounters are in flight.
    static constexpr int kSkCounters = 16;
    static constexpr int kSkCounterWord0 = 32;
    std::mutex sk_mutex;
    uint32_t sk_next = 0;
    // Staging buffers of the htod entry points (grown on demand, never shrunk).
    void* staging[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t staging_bytes[4] = {0, 0, 0, 0};
    // Copy-in / compute / copy-out streams and hand-over events of the pipelined host-buffer GEMM.
    static constexpr int kPipeChunks = 16;  // chunks of A plus chunks of B
    bool pipe_ready = false;
    cudaStream_t pipe_streams[3] = {nullptr, nullptr, nullptr};
    cudaEvent_t pipe_events[2 * kPipeChunks + 1] = {};
};

// State of the CURRENT device; creates it on first use.  Returns 0 or an error
// code (SPORK_ERR_NO_SM100 when the device is not compute capability 10.x).
int current_device_state(DeviceState** out);

// Create the pipeline streams and events of `dev` on first use; returns 0 or a cudaError_t.
int ensure_pipeline(DeviceState& dev);

// Hand a stream-K launch its pair of counters.
uint32_t* reserve_sk_counter(DeviceState& dev);

// After a launch gave up (its counters may be left non-zero): all counters back to zero.
void reset_sk_counters(DeviceState& dev, cudaStream_t stream);

// Grow staging buffer `slot` of `dev` to at least `bytes`; returns 0 or a cudaError_t.
int ensure_staging(DeviceState& dev, int slot, size_t bytes);

}  // namespace spork
