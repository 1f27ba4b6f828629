#include "device_state.h"

#include <mutex>

#include "../../include/spork_b200.h"

namespace spork {

static DeviceState g_states[kMaxDevices];
static std::mutex g_mutex;

int current_device_state(DeviceState** out)
{
    int ordinal = 0;
    cudaError_t e = cudaGetDevice(&ordinal);
    if (e != cudaSuccess) {
        return (int)e;
    }
    if (ordinal < 0 || ordinal >= kMaxDevices) {
        return SPORK_ERR_BAD_ARGUMENT;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState& s = g_states[ordinal];
    if (s.ordinal < 0) {
        int major = 0, sms = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, ordinal);
        if (e != cudaSuccess) {
            return (int)e;
        }
        if (major != 10) {
            return SPORK_ERR_NO_SM100;
        }
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal);
        if (e != cudaSuccess) {
            return (int)e;
        }
        // 256 bytes: [0] status word, [16..48) clock probe of the last GEMM launch (see gemm_sm100.cu),
        // [128..256) the stream-K counter pairs
        uint32_t* word = nullptr;
        e = cudaMalloc(&word, 256);
        if (e != cudaSuccess) {
            return (int)e;
        }
        e = cudaMemset(word, 0, 256);
        if (e != cudaSuccess) {
            cudaFree(word);
            return (int)e;
        }
        s.cc_major = major;
        s.sm_count = sms;
        s.status_word = word;
        s.ordinal = ordinal;
    }
    *out = &s;
    return 0;
}

uint32_t* reserve_sk_counter(DeviceState& dev)
{
    std::lock_guard<std::mutex> lock(dev.sk_mutex);
    const uint32_t slot = dev.sk_next++ % (uint32_t)DeviceState::kSkCounters;
    return dev.status_word + DeviceState::kSkCounterWord0 + 2 * slot;
}

void reset_sk_counters(DeviceState& dev, cudaStream_t stream)
{
    std::lock_guard<std::mutex> lock(dev.sk_mutex);
    cudaMemsetAsync(dev.status_word + DeviceState::kSkCounterWord0, 0,
                    sizeof(uint32_t) * 2 * DeviceState::kSkCounters, stream);
}

int ensure_staging(DeviceState& dev, int slot, size_t bytes)
{
    if (dev.staging_bytes[slot] >= bytes) {
        return 0;
    }
    if (dev.staging[slot]) {
        cudaFree(dev.staging[slot]);
        dev.staging[slot] = nullptr;
        dev.staging_bytes[slot] = 0;
    }
    const cudaError_t e = cudaMalloc(&dev.staging[slot], bytes);
    if (e != cudaSuccess) {
        return (int)e;
    }
    dev.staging_bytes[slot] = bytes;
    return 0;
}

int ensure_pipeline(DeviceState& dev)
{
    if (dev.pipe_ready) {
        return 0;
    }
    for (auto& st : dev.pipe_streams) {
        const cudaError_t e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            return (int)e;
        }
    }
    for (auto& ev : dev.pipe_events) {
        const cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (e != cudaSuccess) {
            return (int)e;
        }
    }
    dev.pipe_ready = true;
    return 0;
}

}  // namespace spork

extern "C" int spork_gemm_sm100_status(void* stream, uint32_t* detail)
{
    spork::DeviceState* dev = nullptr;
    const int rc = spork::current_device_state(&dev);
    if (rc) {
        return rc;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        return (int)e;
    }
    uint32_t word = 0;
    e = cudaMemcpyAsync(&word, dev->status_word, sizeof(word), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(s);
    }
    if (e != cudaSuccess) {
        return (int)e;
    }
    if (detail) {
        *detail = word;
    }
    if (word != 0) {
        cudaMemsetAsync(dev->status_word, 0, sizeof(word), s);
        spork::reset_sk_counters(*dev, s);
        cudaStreamSynchronize(s);
        // 0xC.......: a range check of the debug build; anything else: a bounded wait that ran out
        return (word >> 28) == 0xCu ? SPORK_ERR_DEVICE_CHECK : SPORK_ERR_DEVICE_TIMEOUT;
    }
    return 0;
}

extern "C" const char* spork_b200_version(void)
{
    return "spork_b200 0.1 sm_100a";
}
