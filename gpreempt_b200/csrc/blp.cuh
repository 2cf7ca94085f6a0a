// Device-side block-level-preemption protocol shared by every preemptible kernel.
//
// Semantics follow the persistent wrapper the reference generates around each kernel
// (scripts/compile/convert_to_blp.py:39-70): one elected thread per CTA reads the preempt
// word; while it is 0 the CTA claims the next logical tile with atomicAdd on the kernel's
// cursor; once it is non-zero the CTA records the kernel id as the stop point (first writer
// wins) and returns.  A tile that was claimed always completes, and a relaunch with the same
// cursor continues with the next unclaimed tile, so every tile runs exactly once.
#pragma once

#include <cstdint>
#include <cstdlib>

namespace gpx {

// Passed by value to kernels.  preempted == nullptr selects the static (non-preemptible)
// grid-stride schedule used for latency-critical executors.
struct BlpArgs {
    const int *preempted;
    int *stop_index;
    int *executed;
    int total_tiles;
    int kernel_id;
    unsigned long long *trace;  // {first start, last exit, first seen-raised, tiles run} or null
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ int load_word(const int *p) {
    // .relaxed.sys so the read is served by the point of coherence with host stores and
    // stream memory operations and is never cached in L1.
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Programmatic dependent launch.  The layer kernels of a model are launched with programmatic
// stream serialization: a kernel may become resident while its predecessor in the stream is
// still draining, so launch latency and the scheduling of its CTAs overlap the predecessor's
// tail (batch-1 forwards are ~90 kernels of a few microseconds each).  Every such kernel calls
// pdl_enter() before it touches global memory: it waits until the predecessor grid has completed
// and its writes are visible, then lets its own successor start launching.  In that order only
// one kernel ahead is ever parked on the GPU; releasing the successor first lets a whole chain of
// small kernels become resident and wait, which starves the one that can run (BERT batch 1 was
// 12 % slower that way).  Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
    pdl_wait();
    pdl_launch_dependents();
}

__device__ __forceinline__ void trace_begin(const BlpArgs &b) {
    if (b.trace) atomicMin(b.trace + 0, globaltimer_ns());
}
__device__ __forceinline__ void trace_end(const BlpArgs &b, int tiles_run) {
    if (b.trace) {
        atomicMax(b.trace + 1, globaltimer_ns());
        if (tiles_run) atomicAdd(b.trace + 3, (unsigned long long)tiles_run);
    }
}

// Called by ONE thread of the CTA.  Returns the claimed tile index, or -1 when the CTA must
// return (word raised, or no tiles left).  `iter` counts tiles this CTA has run so far and
// drives the static schedule.
__device__ __forceinline__ int blp_claim(const BlpArgs &b, int iter) {
    if (b.preempted == nullptr) {
        long long t = (long long)blockIdx.x + (long long)iter * gridDim.x;
        return t < b.total_tiles ? (int)t : -1;
    }
    if (load_word(b.preempted) != 0) {
        if (b.trace) atomicMin(b.trace + 2, globaltimer_ns());
        // Only a kernel with unclaimed tiles left is a stop point; a kernel whose cursor has
        // already passed the end has nothing to resume.
        int cur = *((volatile int *)b.executed);
        if (cur < b.total_tiles) atomicCAS(b.stop_index, -1, b.kernel_id);
        return -1;
    }
    int idx = atomicAdd(b.executed, 1);
    return idx < b.total_tiles ? idx : -1;
}

#if defined(__CUDACC__)
// Launch of a layer kernel with the programmatic-serialization attribute (GPX_PDL=0 turns it off).
inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("GPX_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_layer(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t s,
                                Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

}  // namespace gpx
