// Runtime plumbing of libgpx: device binding, memory, streams, events, the preempt word and
// the bounded wait kernel.  Stands in for include/util/gpu_util.h (the GPU* macro shim),
// src/util/gpu_util.cpp, src/block.cu and the GDRCopy flag pool of
// src/cuda-clients/blpclient.cpp:30-76 in the reference.
#include "common.h"
#include "blp.cuh"
#include "word.h"

#include <atomic>
#include <mutex>
#include <pthread.h>
#include <sched.h>
#include <unistd.h>

namespace gpx {

static thread_local char tls_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
    va_end(ap);
}
const char *last_error() { return tls_error; }

static DeviceInfo g_devices[64];
static std::mutex g_dev_mutex;
static thread_local int tls_device = -1;
static thread_local int tls_priority_class = 1;

const DeviceInfo &device_info() {
    int d = tls_device;
    if (d < 0) {
        if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) d = 0;
    }
    return g_devices[d];
}

void *driver_entry(const char *name) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    return fn;
}

cuStreamWriteValue32_t driver_stream_write32() {
    static std::atomic<void *> cached{nullptr};
    void *p = cached.load(std::memory_order_acquire);
    if (!p) {
        p = driver_entry("cuStreamWriteValue32");
        cached.store(p, std::memory_order_release);
    }
    return reinterpret_cast<cuStreamWriteValue32_t>(p);
}

}  // namespace gpx

using namespace gpx;

__global__ void gpx_ping_kernel(const int *flag, unsigned long long *seen,
                                unsigned long long timeout_ns);

// ---- wait / no-op kernels -------------------------------------------------------------------

// One thread waits for *flag != 0, at most timeout_ns of %globaltimer; the outcome goes to
// *status so the host can tell a released wait from one that ran out.
__global__ void gpx_block_kernel(const int *flag, int *status, unsigned long long timeout_ns) {
    unsigned long long t0 = globaltimer_ns();
    int st = GPX_TIMEOUT;
    for (;;) {
        if (load_word(flag) != 0) {
            st = GPX_SUCC;
            break;
        }
        if (globaltimer_ns() - t0 > timeout_ns) break;
        __nanosleep(200);
    }
    if (status) *status = st;
}

__global__ void gpx_noop_kernel() {}

// Ping kernel for clock correlation: waits (bounded) for the mapped host flag, then stores the
// device time at which it saw it.
__global__ void gpx_ping_kernel(const int *flag, unsigned long long *seen,
                                unsigned long long timeout_ns) {
    unsigned long long t0 = globaltimer_ns();
    unsigned long long t = 0;
    for (;;) {
        if (load_word(flag) != 0) {
            t = globaltimer_ns();
            break;
        }
        if (globaltimer_ns() - t0 > timeout_ns) break;
    }
    *seen = t;
}

namespace gpx {

int ClockProbe::init() {
    GPX_CUDA(cudaHostAlloc((void **)&flag, 64, cudaHostAllocMapped));
    GPX_CUDA(cudaHostAlloc((void **)&seen, 64, cudaHostAllocMapped));
    GPX_CUDA(cudaHostGetDevicePointer((void **)&dflag, flag, 0));
    GPX_CUDA(cudaHostGetDevicePointer((void **)&dseen, seen, 0));
    GPX_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    return GPX_SUCC;
}

void ClockProbe::destroy() {
    if (stream) cudaStreamDestroy(stream);
    if (flag) cudaFreeHost(flag);
    if (seen) cudaFreeHost(seen);
    stream = nullptr;
    flag = nullptr;
    seen = nullptr;
}

// Each ping launches a one-thread kernel that polls a mapped host flag (bounded), lets it
// settle, stores the flag at host time th and reads back the device time at which the kernel
// saw it.  th - seen = (host - device) - transport latency, so the largest sample is the one
// with the least latency and under-estimates the true offset by that latency (about 1 us).
// The two clocks drift against each other by tens of ppm, so callers re-measure close to the
// events they want to place on the other clock.
int ClockProbe::measure(int pings, uint64_t settle_ns, int64_t *host_minus_device, int64_t *spread) {
    int64_t lo = INT64_MAX, hi = INT64_MIN;
    int good = 0;
    for (int i = 0; i < pings; ++i) {
        *flag = 0;
        *seen = 0;
        gpx_ping_kernel<<<1, 1, 0, stream>>>(dflag, dseen, 200000000ull);
        GPX_CUDA(cudaGetLastError());
        uint64_t t_wait = now_ns();
        while (now_ns() - t_wait < settle_ns) {
        }
        uint64_t th = now_ns();
        __atomic_store_n(flag, 1, __ATOMIC_SEQ_CST);
        GPX_CUDA(cudaStreamSynchronize(stream));
        if (*seen == 0) continue;
        int64_t off = (int64_t)th - (int64_t)*seen;
        if (off > hi) hi = off;
        if (off < lo) lo = off;
        ++good;
    }
    GPX_REQUIRE(good > 0, GPX_TIMEOUT, "clock ping never completed");
    *host_minus_device = hi;
    if (spread) *spread = hi - lo;
    return GPX_SUCC;
}

}  // namespace gpx

extern "C" {

int gpx_init(int device) {
    int n = 0;
    cudaError_t err = cudaGetDeviceCount(&n);
    if (err != cudaSuccess) {
        set_error("no CUDA device: %s", cudaGetErrorString(err));
        return GPX_FAIL;
    }
    GPX_REQUIRE(device >= 0 && device < n && device < 64, GPX_OUT_OF_RANGE,
                "device %d out of range (have %d)", device, n);
    GPX_CUDA(cudaSetDevice(device));
    GPX_CUDA(cudaFree(0));
    tls_device = device;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo &d = g_devices[device];
    if (d.device < 0) {
        cudaDeviceProp prop;
        GPX_CUDA(cudaGetDeviceProperties(&prop, device));
        d.sm_count = prop.multiProcessorCount;
        d.total_mem = prop.totalGlobalMem;
        snprintf(d.name, sizeof(d.name), "%s", prop.name);
        GPX_CUDA(cudaDeviceGetStreamPriorityRange(&d.prio_least, &d.prio_greatest));
        d.device = device;
    }
    return GPX_SUCC;
}

int gpx_device_count(int *count) {
    GPX_REQUIRE(count, GPX_FAIL, "count is NULL");
    cudaError_t err = cudaGetDeviceCount(count);
    if (err != cudaSuccess) {
        *count = 0;
        set_error("cudaGetDeviceCount: %s", cudaGetErrorString(err));
        return GPX_FAIL;
    }
    return GPX_SUCC;
}

int gpx_device_info(int *sm_count, size_t *total_mem, char *name, size_t name_cap) {
    const DeviceInfo &d = device_info();
    GPX_REQUIRE(d.device >= 0, GPX_FAIL, "gpx_init was not called on this thread's device");
    if (sm_count) *sm_count = d.sm_count;
    if (total_mem) *total_mem = d.total_mem;
    if (name && name_cap) snprintf(name, name_cap, "%s", d.name);
    return GPX_SUCC;
}

const char *gpx_strerror(int status) {
    switch (status) {
        case GPX_SUCC: return "Succ";
        case GPX_FAIL: return "Fail";
        case GPX_TIMEOUT: return "Timeout";
        case GPX_NOT_FOUND: return "NotFound";
        case GPX_OUT_OF_RANGE: return "OutOfRange";
        case GPX_FULL: return "Full";
        default: return "Unknown";
    }
}

const char *gpx_last_error(void) { return last_error(); }

int gpx_bind_core(int core_id) {
    long ncpu = sysconf(_SC_NPROCESSORS_ONLN);
    GPX_REQUIRE(ncpu > 0, GPX_FAIL, "no online cpus");
    cpu_set_t set;
    CPU_ZERO(&set);
    CPU_SET(core_id % ncpu, &set);
    int rc = pthread_setaffinity_np(pthread_self(), sizeof(set), &set);
    GPX_REQUIRE(rc == 0, GPX_FAIL, "pthread_setaffinity_np(%d) failed: %d", core_id, rc);
    return GPX_SUCC;
}

uint64_t gpx_host_now_ns(void) { return now_ns(); }

int gpx_malloc(void **dptr, size_t bytes) {
    GPX_REQUIRE(dptr, GPX_FAIL, "dptr is NULL");
    GPX_CUDA(cudaMalloc(dptr, bytes ? bytes : 1));
    return GPX_SUCC;
}
int gpx_free(void *dptr) {
    GPX_CUDA(cudaFree(dptr));
    return GPX_SUCC;
}
int gpx_host_alloc(void **hptr, size_t bytes) {
    GPX_REQUIRE(hptr, GPX_FAIL, "hptr is NULL");
    GPX_CUDA(cudaHostAlloc(hptr, bytes ? bytes : 1, cudaHostAllocPortable));
    return GPX_SUCC;
}
int gpx_host_free(void *hptr) {
    GPX_CUDA(cudaFreeHost(hptr));
    return GPX_SUCC;
}
int gpx_memcpy_h2d(void *dptr, const void *hptr, size_t bytes, gpx_stream s) {
    GPX_CUDA(cudaMemcpyAsync(dptr, hptr, bytes, cudaMemcpyHostToDevice, as_stream(s)));
    return GPX_SUCC;
}
int gpx_memcpy_d2h(void *hptr, const void *dptr, size_t bytes, gpx_stream s) {
    GPX_CUDA(cudaMemcpyAsync(hptr, dptr, bytes, cudaMemcpyDeviceToHost, as_stream(s)));
    return GPX_SUCC;
}
int gpx_memcpy_d2d(void *dst, const void *src, size_t bytes, gpx_stream s) {
    GPX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, as_stream(s)));
    return GPX_SUCC;
}
int gpx_memset(void *dptr, int byte, size_t bytes, gpx_stream s) {
    GPX_CUDA(cudaMemsetAsync(dptr, byte, bytes, as_stream(s)));
    return GPX_SUCC;
}

int gpx_set_priority(int priority) {
    GPX_REQUIRE(priority == 0 || priority == 1, GPX_OUT_OF_RANGE,
                "priority must be 0 (high) or 1 (low), got %d", priority);
    tls_priority_class = priority;
    return GPX_SUCC;
}

int gpx_stream_create(gpx_stream *s, int priority) {
    GPX_REQUIRE(s, GPX_FAIL, "stream out-pointer is NULL");
    if (priority < 0) priority = tls_priority_class;
    const DeviceInfo &d = device_info();
    GPX_REQUIRE(d.device >= 0, GPX_FAIL, "gpx_init was not called");
    int p = priority == 0 ? d.prio_greatest : d.prio_least;
    cudaStream_t st;
    GPX_CUDA(cudaStreamCreateWithPriority(&st, cudaStreamNonBlocking, p));
    *s = st;
    return GPX_SUCC;
}
int gpx_stream_destroy(gpx_stream s) {
    GPX_CUDA(cudaStreamDestroy(as_stream(s)));
    return GPX_SUCC;
}
int gpx_stream_sync(gpx_stream s) {
    GPX_CUDA(cudaStreamSynchronize(as_stream(s)));
    return GPX_SUCC;
}
int gpx_stream_query(gpx_stream s) {
    cudaError_t err = cudaStreamQuery(as_stream(s));
    if (err == cudaSuccess) return GPX_SUCC;
    if (err == cudaErrorNotReady) return GPX_TIMEOUT;
    set_error("cudaStreamQuery: %s", cudaGetErrorString(err));
    return GPX_FAIL;
}
int gpx_device_sync(void) {
    GPX_CUDA(cudaDeviceSynchronize());
    return GPX_SUCC;
}

int gpx_event_create(gpx_event *e) {
    GPX_REQUIRE(e, GPX_FAIL, "event out-pointer is NULL");
    cudaEvent_t ev;
    GPX_CUDA(cudaEventCreate(&ev));
    *e = ev;
    return GPX_SUCC;
}
int gpx_event_destroy(gpx_event e) {
    GPX_CUDA(cudaEventDestroy((cudaEvent_t)e));
    return GPX_SUCC;
}
int gpx_event_record(gpx_event e, gpx_stream s) {
    GPX_CUDA(cudaEventRecord((cudaEvent_t)e, as_stream(s)));
    return GPX_SUCC;
}
int gpx_event_sync(gpx_event e) {
    GPX_CUDA(cudaEventSynchronize((cudaEvent_t)e));
    return GPX_SUCC;
}
int gpx_event_elapsed_ms(gpx_event start, gpx_event stop, float *ms) {
    GPX_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return GPX_SUCC;
}

// ---- preempt word ---------------------------------------------------------------------------

int gpx_word_create(gpx_word **w, int transport) {
    GPX_REQUIRE(w, GPX_FAIL, "word out-pointer is NULL");
    GPX_REQUIRE(transport == GPX_WORD_MAPPED || transport == GPX_WORD_DEVICE, GPX_OUT_OF_RANGE,
                "unknown word transport %d", transport);
    gpx_word *p = new gpx_word();
    p->transport = transport;
    p->wstream = nullptr;
    GPX_CUDA(cudaGetDevice(&p->device));
    if (transport == GPX_WORD_MAPPED) {
        GPX_CUDA(cudaHostAlloc((void **)&p->host_alias, 64,
                               cudaHostAllocMapped | cudaHostAllocPortable));
        *p->host_alias = 0;
        GPX_CUDA(cudaHostGetDevicePointer((void **)&p->dptr, p->host_alias, 0));
    } else {
        GPX_REQUIRE(driver_stream_write32() != nullptr, GPX_FAIL,
                    "driver has no cuStreamWriteValue32");
        p->host_alias = new int(0);
        GPX_CUDA(cudaMalloc((void **)&p->dptr, 256));
        GPX_CUDA(cudaMemset(p->dptr, 0, 256));
        const DeviceInfo &d = device_info();
        GPX_CUDA(cudaStreamCreateWithPriority(&p->wstream, cudaStreamNonBlocking,
                                              d.prio_greatest));
    }
    *w = p;
    return GPX_SUCC;
}

int gpx_word_destroy(gpx_word *w) {
    if (!w) return GPX_SUCC;
    if (w->transport == GPX_WORD_MAPPED) {
        cudaFreeHost(w->host_alias);
    } else {
        cudaStreamSynchronize(w->wstream);
        cudaStreamDestroy(w->wstream);
        cudaFree(w->dptr);
        delete w->host_alias;
    }
    delete w;
    return GPX_SUCC;
}

static int word_store(gpx_word *w, int v) {
    GPX_REQUIRE(w, GPX_FAIL, "word is NULL");
    if (w->transport == GPX_WORD_MAPPED) {
        __atomic_store_n(w->host_alias, v, __ATOMIC_SEQ_CST);
        return GPX_SUCC;
    }
    __atomic_store_n(w->host_alias, v, __ATOMIC_SEQ_CST);
    int rc = driver_stream_write32()(w->wstream, (unsigned long long)(uintptr_t)w->dptr,
                                     (uint32_t)v, 0);
    GPX_REQUIRE(rc == 0, GPX_FAIL, "cuStreamWriteValue32 failed with %d", rc);
    return GPX_SUCC;
}

int gpx_word_raise(gpx_word *w) { return word_store(w, 1); }
int gpx_word_clear(gpx_word *w) { return word_store(w, 0); }

int gpx_word_dptr(gpx_word *w, void **dptr) {
    GPX_REQUIRE(w && dptr, GPX_FAIL, "NULL argument");
    *dptr = w->dptr;
    return GPX_SUCC;
}
int gpx_word_value(gpx_word *w, int *value) {
    GPX_REQUIRE(w && value, GPX_FAIL, "NULL argument");
    *value = __atomic_load_n(w->host_alias, __ATOMIC_SEQ_CST);
    return GPX_SUCC;
}

int gpx_block_launch(const void *flag_dptr, void *status_dptr, uint64_t timeout_ns,
                     gpx_stream s) {
    GPX_REQUIRE(flag_dptr, GPX_FAIL, "flag is NULL");
    // A wait longer than 2 s is refused: the GPU is shared and an unreleased wait would hold it.
    GPX_REQUIRE(timeout_ns <= 2000000000ull, GPX_OUT_OF_RANGE, "timeout above 2 s");
    gpx_block_kernel<<<1, 1, 0, as_stream(s)>>>((const int *)flag_dptr, (int *)status_dptr,
                                                (unsigned long long)timeout_ns);
    GPX_CUDA(cudaGetLastError());
    return GPX_SUCC;
}

int gpx_noop_launch(gpx_stream s) {
    gpx_noop_kernel<<<1, 1, 0, as_stream(s)>>>();
    GPX_CUDA(cudaGetLastError());
    return GPX_SUCC;
}

int gpx_clock_offset_ns(int64_t *host_minus_device, int64_t *uncertainty_ns) {
    GPX_REQUIRE(host_minus_device, GPX_FAIL, "NULL argument");
    ClockProbe probe;
    GPX_TRY(probe.init());
    int st = probe.measure(16, 200000, host_minus_device, uncertainty_ns);
    probe.destroy();
    return st;
}

}  // extern "C"
