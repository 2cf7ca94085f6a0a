// The GPU* names of the reference's CUDA/HIP macro shim (include/util/gpu_util.h:12-162) on top
// of the libgpx C ABI, so client sources written against them compile without cuda.h.  Handles
// are opaque: a stream is a gpx_stream, a device pointer an integer wide enough for an address.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <string>
#include <sys/syscall.h>
#include <unistd.h>

#include "../../gpx.h"
#include "common.h"

#define util_gettid() ((pid_t)syscall(SYS_gettid))

typedef unsigned long long GPUdeviceptr;  // CUdeviceptr
typedef int GPUresult;                    // a gpx status: 0 = success
typedef gpx_stream GPUstream;
typedef int GPUdevice;
typedef void *GPUcontext;

#define GPU_SUCCESS 0
#define GPU_MEM_ATTACH_GLOBAL 1
#define CU_MEMHOSTALLOC_PORTABLE 1
#define GPUStreamDefault 0

inline const char *GPUGetErrorString(GPUresult) { return gpx_last_error(); }

// Streams.  Priorities follow the library's convention, which is also what the reference's
// clients end up passing: 0 = latency-critical, 1 = best-effort
// (src/common-clients/baseclient.cpp:57-61).
inline GPUresult GPUStreamCreate(GPUstream *s, unsigned /*flags*/) { return gpx_stream_create(s, 1); }
inline GPUresult GPUCtxGetStreamPriorityRange(int *least, int *greatest) {
    *least = 1;
    *greatest = 0;
    return GPU_SUCCESS;
}
inline GPUresult GPUStreamCreateWithPriority(GPUstream *s, unsigned /*flags*/, int priority) {
    return gpx_stream_create(s, priority ? 1 : 0);
}
inline GPUresult GPUStreamDestroy(GPUstream s) { return gpx_stream_destroy(s); }
inline GPUresult GPUStreamSynchronize(GPUstream s) { return gpx_stream_sync(s); }
inline GPUresult GPUStreamQuery(GPUstream s) { return gpx_stream_query(s); }

// Memory.
inline GPUresult GPUMemAlloc(GPUdeviceptr *p, size_t bytes) {
    void *d = nullptr;
    GPUresult r = gpx_malloc(&d, bytes);
    *p = (GPUdeviceptr)(uintptr_t)d;
    return r;
}
inline GPUresult GPUMemFree(GPUdeviceptr p) { return gpx_free((void *)(uintptr_t)p); }
template <typename T>
inline GPUresult GPUMemHostAlloc(T **h, size_t bytes, unsigned /*flags*/) {
    void *p = nullptr;
    GPUresult r = gpx_host_alloc(&p, bytes);
    *h = (T *)p;
    return r;
}
inline GPUresult GPUMemFreeHost(void *h) { return gpx_host_free(h); }
// Memory both sides can address (the reference uses managed memory for its test flag,
// src/tests/test-dnn-blp.cpp:18-22): pinned host memory, reachable from the device at the same
// address.
inline GPUresult GPUMallocManaged(GPUdeviceptr *p, size_t bytes, unsigned /*flags*/) {
    void *h = nullptr;
    GPUresult r = gpx_host_alloc(&h, bytes);
    *p = (GPUdeviceptr)(uintptr_t)h;
    return r;
}
inline GPUresult GPUMemset(GPUdeviceptr p, unsigned char v, size_t n) {
    GPUresult r = gpx_memset((void *)(uintptr_t)p, v, n, nullptr);
    return r == GPU_SUCCESS ? gpx_stream_sync(nullptr) : r;
}
inline GPUresult GPUMemsetAsync(GPUdeviceptr p, unsigned char v, size_t n, GPUstream s) {
    return gpx_memset((void *)(uintptr_t)p, v, n, s);
}
inline GPUresult GPUMemcpyHtoDAsync(GPUdeviceptr d, const void *h, size_t n, GPUstream s) {
    return gpx_memcpy_h2d((void *)(uintptr_t)d, h, n, s);
}
inline GPUresult GPUMemcpyDtoHAsync(void *h, GPUdeviceptr d, size_t n, GPUstream s) {
    return gpx_memcpy_d2h(h, (const void *)(uintptr_t)d, n, s);
}
inline GPUresult GPUMemcpyDtoDAsync(GPUdeviceptr dst, GPUdeviceptr src, size_t n, GPUstream s) {
    return gpx_memcpy_d2d((void *)(uintptr_t)dst, (const void *)(uintptr_t)src, n, s);
}
inline GPUresult GPUMemcpyHtoD(GPUdeviceptr d, const void *h, size_t n) {
    GPUresult r = gpx_memcpy_h2d((void *)(uintptr_t)d, h, n, nullptr);
    return r == GPU_SUCCESS ? gpx_stream_sync(nullptr) : r;
}
inline GPUresult GPUMemcpyDtoH(void *h, GPUdeviceptr d, size_t n) {
    GPUresult r = gpx_memcpy_d2h(h, (const void *)(uintptr_t)d, n, nullptr);
    return r == GPU_SUCCESS ? gpx_stream_sync(nullptr) : r;
}

// include/util/gpu_util.h:143-162.
#define ASSERT_CUDA_ERROR(cmd)                                                                     \
    {                                                                                              \
        GPUresult error__ = (cmd);                                                                 \
        if (error__ != GPU_SUCCESS) {                                                              \
            std::fprintf(stderr, "GPU error: %d %s at %s:%d\n", error__, GPUGetErrorString(error__), \
                         __FILE__, __LINE__);                                                      \
            std::exit(EXIT_FAILURE);                                                               \
        }                                                                                          \
    }

#define CUDA_RETURN_STATUS(cmd)                                                                    \
    {                                                                                              \
        GPUresult error__ = (cmd);                                                                 \
        if (error__ != GPU_SUCCESS) {                                                              \
            std::cout << "GPU error: " << error__ << " " << GPUGetErrorString(error__) << " at "  \
                      << __FILE__ << ":" << __LINE__ << std::endl;                                 \
            return Status::Fail;                                                                   \
        }                                                                                          \
    }

namespace foo {
namespace util {

// src/util/gpu_util.cpp:14-25: binds the calling thread to the GPU (idempotent).  The reference
// hard-codes device 0; GPX_DEVICE in the environment selects another one.
inline void init_cuda() {
    const char *e = std::getenv("GPX_DEVICE");
    ASSERT_CUDA_ERROR(gpx_init(e ? std::atoi(e) : 0));
}

}  // namespace util
}  // namespace foo
