// Preemption microbenchmark: raise the preempt word at uniformly random times inside a
// best-effort kernel, measure flag-to-drain latency on the device timeline, resume, and check
// that the final result is bit-identical to an uninterrupted run.
//
// This is the asserted, repeated form of the reference's manual preempt-and-resume test
// (src/tests/test-dnn-blp.cpp:36-43) applied to the two stand-alone best-effort kernels: the
// HBM-bound fp32 axpy and the tensor-bound bf16 GEMM.
#include "common.h"
#include "blp.cuh"
#include "word.h"

#include <algorithm>
#include <cmath>
#include <random>
#include <vector>

namespace gpx {

// Device-side copy of the counter-based generator of model.cu (same constants), used to fill
// operands that are too large to generate on the host in reasonable time.
__device__ __forceinline__ unsigned long long mix64_dev(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float uniform_dev(unsigned long long seed, unsigned long long stream,
                                             unsigned long long i, float lo, float hi) {
    unsigned long long h =
        mix64_dev(mix64_dev(seed * 0xD1342543DE82EF95ull + stream) ^ (i * 0x2545F4914F6CDD1Dull + 1));
    double u = (double)(h >> 11) * (1.0 / 9007199254740992.0);
    return (float)(lo + (hi - lo) * u);
}

__global__ void fill_uniform_f32_kernel(float *dst, size_t n, unsigned long long seed,
                                        unsigned long long stream, float lo, float hi) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        dst[i] = uniform_dev(seed, stream, i, lo, hi);
}

__global__ void fill_uniform_bf16_kernel(unsigned short *dst, size_t n, unsigned long long seed,
                                         unsigned long long stream, float lo, float hi) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        float f = uniform_dev(seed, stream, i, lo, hi);
        unsigned int u = __float_as_uint(f);
        u += 0x7fffu + ((u >> 16) & 1u);  // round to nearest even
        dst[i] = (unsigned short)(u >> 16);
    }
}

// Counts 32-bit words that differ between two buffers.
__global__ void count_diff_kernel(const unsigned int *a, const unsigned int *b, size_t n,
                                  unsigned long long *diff) {
    unsigned long long local = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        local += a[i] != b[i];
    if (local) atomicAdd(diff, local);
}

static void spin_ns(uint64_t ns) {
    uint64_t t0 = now_ns();
    while (now_ns() - t0 < ns) {
    }
}

struct BlpDevice {
    int *stop_index;              // +0
    int *executed;                // +4
    unsigned long long *trace;    // +64 .. +96
    unsigned char *base;
};

static int blp_reset(BlpDevice &b, cudaStream_t s) {
    struct Init {
        int stop, cursor;
        int pad[14];
        unsigned long long trace[4];
    } init;
    memset(&init, 0, sizeof(init));
    init.stop = -1;
    init.trace[0] = ~0ull;
    init.trace[2] = ~0ull;
    GPX_CUDA(cudaMemcpyAsync(b.base, &init, sizeof(init), cudaMemcpyHostToDevice, s));
    GPX_CUDA(cudaStreamSynchronize(s));
    return GPX_SUCC;
}

}  // namespace gpx

using namespace gpx;

extern "C" int gpx_fill_uniform(void *dptr, size_t n, int is_bf16, uint64_t seed, uint64_t stream,
                                float lo, float hi, gpx_stream s) {
    GPX_REQUIRE(dptr || n == 0, GPX_FAIL, "dptr is NULL");
    if (n == 0) return GPX_SUCC;
    const DeviceInfo &d = device_info();
    int grid = (d.sm_count > 0 ? d.sm_count : 148) * 8;
    if (is_bf16)
        fill_uniform_bf16_kernel<<<grid, 256, 0, as_stream(s)>>>((unsigned short *)dptr, n, seed,
                                                                 stream, lo, hi);
    else
        fill_uniform_f32_kernel<<<grid, 256, 0, as_stream(s)>>>((float *)dptr, n, seed, stream, lo, hi);
    GPX_CUDA(cudaGetLastError());
    return GPX_SUCC;
}

extern "C" int gpx_count_diff(const void *a, const void *b, size_t bytes, uint64_t *diff,
                              gpx_stream s) {
    GPX_REQUIRE(a && b && diff, GPX_FAIL, "NULL argument");
    GPX_REQUIRE(bytes % 4 == 0, GPX_OUT_OF_RANGE, "size must be a multiple of 4 bytes");
    unsigned long long *d = nullptr;
    GPX_CUDA(cudaMalloc((void **)&d, 8));
    GPX_CUDA(cudaMemsetAsync(d, 0, 8, as_stream(s)));
    const DeviceInfo &di = device_info();
    int grid = (di.sm_count > 0 ? di.sm_count : 148) * 8;
    count_diff_kernel<<<grid, 256, 0, as_stream(s)>>>((const unsigned int *)a, (const unsigned int *)b,
                                                     bytes / 4, d);
    cudaError_t err = cudaGetLastError();
    unsigned long long h = 0;
    if (err == cudaSuccess) err = cudaMemcpyAsync(&h, d, 8, cudaMemcpyDeviceToHost, as_stream(s));
    if (err == cudaSuccess) err = cudaStreamSynchronize(as_stream(s));
    cudaFree(d);
    GPX_CUDA(err);
    *diff = h;
    return GPX_SUCC;
}

extern "C" int gpx_preempt_microbench(int kind, size_t size, int triggers, uint64_t seed,
                                      int transport, double *drain_us, double *seen_us,
                                      gpx_microbench_summary *out) {
    GPX_REQUIRE(out, GPX_FAIL, "out is NULL");
    GPX_REQUIRE(kind == 0 || kind == 1, GPX_OUT_OF_RANGE, "kind must be 0 (axpy) or 1 (gemm)");
    GPX_REQUIRE(triggers >= 0 && triggers <= 100000, GPX_OUT_OF_RANGE, "bad trigger count");
    memset(out, 0, sizeof(*out));
    const float a = 1.0009765625f;
    cudaStream_t st;
    GPX_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    gpx_word *word = nullptr;
    GPX_TRY(gpx_word_create(&word, transport));
    BlpDevice blp{};
    GPX_CUDA(cudaMalloc((void **)&blp.base, 256));
    blp.stop_index = (int *)blp.base;
    blp.executed = (int *)(blp.base + 4);
    blp.trace = (unsigned long long *)(blp.base + 64);
    gpx_blp args{word->dptr, blp.stop_index, blp.executed, 9, blp.trace};

    // operands
    size_t out_bytes = 0;
    void *x = nullptr, *y = nullptr, *y0 = nullptr, *ref = nullptr, *ctx = nullptr;
    int M = 0;
    if (kind == 0) {
        out_bytes = size * sizeof(float);
        GPX_CUDA(cudaMalloc(&x, out_bytes));
        GPX_CUDA(cudaMalloc(&y, out_bytes));
        GPX_CUDA(cudaMalloc(&y0, out_bytes));
        GPX_CUDA(cudaMalloc(&ref, out_bytes));
        GPX_TRY(gpx_fill_uniform(x, size, 0, seed, 0, -1.f, 1.f, st));
        GPX_TRY(gpx_fill_uniform(y0, size, 0, seed, 1, -1.f, 1.f, st));
    } else {
        M = (int)size;
        size_t elems = (size_t)M * M;
        out_bytes = elems * 2;
        GPX_CUDA(cudaMalloc(&x, elems * 2));   // A
        GPX_CUDA(cudaMalloc(&y0, elems * 2));  // B
        GPX_CUDA(cudaMalloc(&y, out_bytes));   // C
        GPX_CUDA(cudaMalloc(&ref, out_bytes));
        size_t cb = 0;
        GPX_TRY(gpx_gemm_ctx_bytes(&cb));
        GPX_CUDA(cudaMalloc(&ctx, cb));
        GPX_TRY(gpx_fill_uniform(x, elems, 1, seed, 0, -1.f, 1.f, st));
        GPX_TRY(gpx_fill_uniform(y0, elems, 1, seed, 1, -1.f, 1.f, st));
    }
    auto prepare = [&]() -> int {
        if (kind == 0) {
            GPX_CUDA(cudaMemcpyAsync(y, y0, out_bytes, cudaMemcpyDeviceToDevice, st));
        } else {
            size_t cb = 0;
            gpx_gemm_ctx_bytes(&cb);
            GPX_CUDA(cudaMemsetAsync(ctx, 0, 8192, st));  // header + progress slots
            GPX_CUDA(cudaMemsetAsync(y, 0, out_bytes, st));
        }
        return blp_reset(blp, st);
    };
    auto launch = [&]() -> int {
        if (kind == 0) return gpx_axpy_f32(a, x, y, size, 0, &args, st);
        return gpx_gemm_bf16(x, y0, y, M, M, M, ctx, &args, st);
    };
    struct Snapshot {
        int stop, cursor;
        int pad[14];
        unsigned long long trace[4];
    } snap;
    auto read = [&]() -> int {
        GPX_CUDA(cudaMemcpyAsync(&snap, blp.base, sizeof(snap), cudaMemcpyDeviceToHost, st));
        GPX_CUDA(cudaStreamSynchronize(st));
        return GPX_SUCC;
    };

    // Uninterrupted reference run, timed with events after a warm-up.
    cudaEvent_t e0, e1;
    GPX_CUDA(cudaEventCreate(&e0));
    GPX_CUDA(cudaEventCreate(&e1));
    float kernel_ms = 0;
    for (int i = 0; i < 4; ++i) {
        GPX_TRY(prepare());
        GPX_CUDA(cudaEventRecord(e0, st));
        GPX_TRY(launch());
        GPX_CUDA(cudaEventRecord(e1, st));
        GPX_CUDA(cudaStreamSynchronize(st));
        GPX_CUDA(cudaEventElapsedTime(&kernel_ms, e0, e1));
    }
    GPX_TRY(read());
    GPX_REQUIRE(snap.stop == -1, GPX_FAIL, "uninterrupted run reported a stop point");
    GPX_CUDA(cudaMemcpyAsync(ref, y, out_bytes, cudaMemcpyDeviceToDevice, st));
    GPX_CUDA(cudaStreamSynchronize(st));
    out->kernel_ms = kernel_ms;

    // The host clock and %globaltimer drift apart by tens of ppm, so the offset is re-measured
    // right before every trigger.
    ClockProbe probe;
    GPX_TRY(probe.init());
    int64_t offset = 0, unc = 0;
    GPX_TRY(probe.measure(8, 100000, &offset, &unc));
    double unc_sum = 0;

    std::mt19937_64 rng(seed * 31 + 5);
    std::uniform_real_distribution<double> uni(0.0, 1.0);
    std::vector<double> drains, seens, raise_calls;
    double drain_after_return_max = 0;
    int mismatches = 0, preempted = 0, resumes_total = 0, late_starts = 0;
    for (int t = 0; t < triggers; ++t) {
        GPX_TRY(prepare());
        GPX_TRY(gpx_word_clear(word));
        if (transport == GPX_WORD_DEVICE) GPX_CUDA(cudaStreamSynchronize(word->wstream));
        uint64_t delay_ns = (uint64_t)(uni(rng) * kernel_ms * 1e6);
        GPX_TRY(probe.measure(3, 40000, &offset, &unc));
        unc_sum += (double)unc;
        GPX_TRY(launch());
        spin_ns(delay_ns);
        // Two host stamps around the raise.  The latency is counted from the first (before the
        // write is issued), so it includes the write's own way to the GPU and is an upper bound;
        // a host thread that is descheduled inside the call (seen once as a 0.9 ms "drain" among
        // 1000 triggers of 17 us) shows up as a long call, and the drain counted from the second
        // stamp tells such a host delay from a kernel that was slow to leave.
        uint64_t t_raise = now_ns();
        GPX_TRY(gpx_word_raise(word));
        uint64_t t_raised = now_ns();
        GPX_TRY(read());
        raise_calls.push_back((double)(t_raised - t_raise) / 1e3);
        // A launch that reached the GPU after the word was already up (a late launch on the host
        // side: the kernel then leaves at its entry check) has nothing to drain; its "latency" would
        // be the launch delay.  Such samples are counted, not mixed into the drain statistics.
        const bool started_late = snap.stop != -1 && snap.trace[0] != ~0ull &&
                                  (int64_t)snap.trace[0] + offset > (int64_t)t_raised + (int64_t)unc;
        if (started_late) ++late_starts;
        if (snap.stop != -1 && !started_late) {
            ++preempted;
            drain_after_return_max = std::max(
                drain_after_return_max, ((double)((int64_t)snap.trace[1] + offset) - (double)t_raised) / 1e3);
            // last CTA exit on the device clock, moved to the host clock
            double drain = ((double)((int64_t)snap.trace[1] + offset) - (double)t_raise) / 1e3;
            double seen = ((double)((int64_t)snap.trace[2] + offset) - (double)t_raise) / 1e3;
            drains.push_back(drain);
            seens.push_back(seen);
            if (drain_us && (int)drains.size() <= triggers) drain_us[drains.size() - 1] = drain;
            if (seen_us && (int)seens.size() <= triggers) seen_us[seens.size() - 1] = seen;
        }
        // resume until complete (the word is cleared only after the stream drained)
        int guard = 0;
        while (snap.stop != -1) {
            GPX_TRY(gpx_word_clear(word));
            if (transport == GPX_WORD_DEVICE) GPX_CUDA(cudaStreamSynchronize(word->wstream));
            int minus1 = -1;
            GPX_CUDA(cudaMemcpyAsync(blp.stop_index, &minus1, sizeof(int), cudaMemcpyHostToDevice, st));
            GPX_CUDA(cudaStreamSynchronize(st));
            GPX_TRY(launch());
            GPX_TRY(read());
            ++resumes_total;
            GPX_REQUIRE(++guard < 100, GPX_FAIL, "kernel never completed after 100 resumes");
        }
        uint64_t diff = 0;
        GPX_TRY(gpx_count_diff(y, ref, out_bytes, &diff, st));
        if (diff) ++mismatches;
        if (kind == 1) {
            int err = 0, cta = 0;
            GPX_TRY(gpx_gemm_status(ctx, &err, &cta));
            GPX_REQUIRE(err == 0, GPX_FAIL, "gemm reported error %d on cta %d", err, cta);
        }
    }
    auto pct = [](std::vector<double> v, double p) {
        if (v.empty()) return 0.0;
        std::sort(v.begin(), v.end());
        double pos = p * (v.size() - 1);
        size_t lo = (size_t)pos, hi = std::min(lo + 1, v.size() - 1);
        return v[lo] + (v[hi] - v[lo]) * (pos - lo);
    };
    out->clock_uncertainty_ns = triggers ? unc_sum / triggers : (double)unc;
    probe.destroy();
    out->triggers = triggers;
    out->preempted = preempted;
    out->resumes = resumes_total;
    out->mismatches = mismatches;
    out->drain_us_p50 = pct(drains, 0.5);
    out->drain_us_p99 = pct(drains, 0.99);
    out->drain_us_max = drains.empty() ? 0 : *std::max_element(drains.begin(), drains.end());
    double sum = 0;
    for (double d : drains) sum += d;
    out->drain_us_mean = drains.empty() ? 0 : sum / drains.size();
    out->seen_us_p50 = pct(seens, 0.5);
    out->seen_us_p99 = pct(seens, 0.99);
    out->raise_call_us_p50 = pct(raise_calls, 0.5);
    out->raise_call_us_max = raise_calls.empty() ? 0 : *std::max_element(raise_calls.begin(), raise_calls.end());
    out->drain_after_return_us_max = drain_after_return_max;
    out->late_starts = late_starts;

    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(x);
    cudaFree(y);
    cudaFree(y0);
    cudaFree(ref);
    if (ctx) cudaFree(ctx);
    cudaFree(blp.base);
    gpx_word_destroy(word);
    cudaStreamDestroy(st);
    return GPX_SUCC;
}
