// C entry points over the reference's own miniWeather translation unit
// (src/workloads/miniweather.cu, compiled unmodified next to this file into
// oracle/_ref/libminiweather_ref.so).  TEST INFRASTRUCTURE ONLY: the GPU parity test loads it to
// compare this repository's kernels and CPU oracle with what the reference computes.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstddef>

namespace SciComputeRaw {
// Globals and functions with external linkage defined by the reference source.
extern float *state;
extern float *state_tmp;
extern float dt;
void sci_init();
void perform_timestep(CUstream stream);
void reductions(double &mass, double &te);
void finalize();
}  // namespace SciComputeRaw

namespace {
// The reference fixes its grid at compile time (miniweather.cu:21-22).
constexpr int kNx = 3200, kNz = 1600, kHalo = 2, kVars = 4;
bool g_live = false;
}  // namespace

extern "C" {

int mwref_grid(int *nx, int *nz) {
    *nx = kNx;
    *nz = kNz;
    return 0;
}

// Executor::init for the scientific workload (src/executor.cpp:35-38).
int mwref_init(int device) {
    if (cudaSetDevice(device) != cudaSuccess) return 1;
    if (cudaFree(nullptr) != cudaSuccess) return 1;  // the driver-API calls below need the primary context
    if (g_live) SciComputeRaw::finalize();
    SciComputeRaw::sci_init();
    g_live = true;
    return cudaDeviceSynchronize() == cudaSuccess ? 0 : 2;
}

// Executor::execute (src/executor.cpp:131), n times on the default stream.
int mwref_steps(int n) {
    if (!g_live) return 1;
    for (int i = 0; i < n; ++i) SciComputeRaw::perform_timestep(nullptr);
    return cudaDeviceSynchronize() == cudaSuccess ? 0 : 2;
}

// Device time of n time steps in milliseconds (CUDA events on the default stream), < 0 on error.
float mwref_time_steps(int n) {
    if (!g_live) return -1.f;
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return -1.f;
    cudaEventRecord(a, nullptr);
    for (int i = 0; i < n; ++i) SciComputeRaw::perform_timestep(nullptr);
    cudaEventRecord(b, nullptr);
    float ms = -1.f;
    if (cudaEventSynchronize(b) == cudaSuccess) cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    return ms;
}

// which = 0: state, 1: state_tmp; `floats` must be 4 * (nz + 4) * (nx + 4).
int mwref_state(int which, float *host, size_t floats) {
    const size_t want = (size_t)kVars * (kNz + 2 * kHalo) * (kNx + 2 * kHalo);
    if (!g_live || floats != want) return 1;
    const float *src = which == 0 ? SciComputeRaw::state : SciComputeRaw::state_tmp;
    return cudaMemcpy(host, src, want * sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 2;
}

float mwref_dt() { return SciComputeRaw::dt; }

int mwref_reductions(double *mass, double *te) {
    if (!g_live) return 1;
    SciComputeRaw::reductions(*mass, *te);
    return 0;
}

int mwref_finalize() {
    if (g_live) SciComputeRaw::finalize();
    g_live = false;
    return 0;
}

}  // extern "C"
