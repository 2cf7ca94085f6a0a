// Internal helpers shared by every translation unit of libgpx: status plumbing, the
// thread-local error text, CUDA error checks that return instead of terminating, and the
// host clock.
#pragma once

#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <time.h>

#include "../../include/gpx.h"

namespace gpx {

void set_error(const char *fmt, ...) __attribute__((format(printf, 1, 2)));
const char *last_error();

inline uint64_t now_ns() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return uint64_t(ts.tv_sec) * 1000000000ull + uint64_t(ts.tv_nsec);
}

// The reference's CUDA_RETURN_STATUS prints and returns Fail (include/util/gpu_util.h:153-162);
// this one records the text for gpx_last_error and returns GPX_FAIL.
#define GPX_CUDA(call)                                                                      \
    do {                                                                                    \
        cudaError_t err__ = (call);                                                         \
        if (err__ != cudaSuccess) {                                                         \
            ::gpx::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(err__),     \
                             __FILE__, __LINE__);                                           \
            return GPX_FAIL;                                                                \
        }                                                                                   \
    } while (0)

#define GPX_TRY(call)                                                                       \
    do {                                                                                    \
        int st__ = (call);                                                                  \
        if (st__ != GPX_SUCC) return st__;                                                  \
    } while (0)

#define GPX_REQUIRE(cond, status, ...)                                                      \
    do {                                                                                    \
        if (!(cond)) {                                                                      \
            ::gpx::set_error(__VA_ARGS__);                                                  \
            return (status);                                                                \
        }                                                                                   \
    } while (0)

inline cudaStream_t as_stream(gpx_stream s) { return reinterpret_cast<cudaStream_t>(s); }

// Device properties cached by gpx_init for the current device.
struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    size_t total_mem = 0;
    int prio_least = 0;     // numerically largest = lowest priority
    int prio_greatest = 0;  // numerically smallest = highest priority
    char name[128] = {0};
};
const DeviceInfo &device_info();  // of the calling thread's current device (after gpx_init)

// Driver entry points resolved at run time (the library does not link libcuda, so it loads on
// a machine without a driver; compute calls then fail with a clear error).
typedef int (*cuStreamWriteValue32_t)(cudaStream_t, unsigned long long, uint32_t, unsigned);
cuStreamWriteValue32_t driver_stream_write32();
void *driver_entry(const char *name);

// Host-clock / device-%globaltimer correlation by bounded ping kernels.
struct ClockProbe {
    int *flag = nullptr;
    unsigned long long *seen = nullptr;
    int *dflag = nullptr;
    unsigned long long *dseen = nullptr;
    cudaStream_t stream = nullptr;
    int init();
    void destroy();
    int measure(int pings, uint64_t settle_ns, int64_t *host_minus_device, int64_t *spread);
};

}  // namespace gpx
