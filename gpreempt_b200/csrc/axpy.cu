// Preemptible fp32 axpy, the HBM-bound best-effort kernel of the preemption microbenchmark.
//
// y[i] = fma(a, x[i], y[i]).  Algorithmic traffic is 12 bytes per element (read x, read y,
// write y).  Persistent CTAs claim tiles of `tile_elems` elements through the block-level
// preemption protocol (scripts/compile/convert_to_blp.py:39-70 in the reference) and drain at
// a tile boundary once the preempt word is raised.  Every element belongs to exactly one
// tile and a tile is computed by one CTA in one pass, so a preempted-and-resumed run is
// bit-identical to an uninterrupted one.
#include "common.h"
#include "blp.cuh"

namespace gpx {

constexpr int kAxpyThreads = 256;
// Elements per tile.  24 KB of traffic per tile: with 8 resident CTAs per SM sharing ~46 GB/s a
// tile lasts about 4 us, which bounds the drain after the word is seen; bandwidth is unchanged
// against larger tiles because the poll and the claim of one CTA overlap the copies of the others.
constexpr size_t kAxpyDefaultTile = 2048;

// VEC float4 loads of x and of y are issued before the first use so each thread keeps
// 2*VEC 16-byte requests in flight.
template <int VEC>
__device__ __forceinline__ void axpy_tile_vec(float a, const float4 *__restrict__ x4,
                                              float4 *__restrict__ y4, size_t base4) {
    float4 xv[VEC], yv[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        size_t i = base4 + (size_t)v * kAxpyThreads + threadIdx.x;
        xv[v] = __ldcs(x4 + i);
        yv[v] = __ldcs(y4 + i);
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        size_t i = base4 + (size_t)v * kAxpyThreads + threadIdx.x;
        float4 r;
        r.x = fmaf(a, xv[v].x, yv[v].x);
        r.y = fmaf(a, xv[v].y, yv[v].y);
        r.z = fmaf(a, xv[v].z, yv[v].z);
        r.w = fmaf(a, xv[v].w, yv[v].w);
        __stcs(y4 + i, r);
    }
}

__global__ void __launch_bounds__(kAxpyThreads)
axpy_f32_kernel(float a, const float *__restrict__ x, float *__restrict__ y, size_t n,
                size_t tile_elems, BlpArgs blp) {
    __shared__ int s_tile;
    if (threadIdx.x == 0) trace_begin(blp);
    int iter = 0;
    const bool dynamic = blp.preempted != nullptr;
    for (;;) {
        int tile;
        if (dynamic) {
            if (threadIdx.x == 0) s_tile = blp_claim(blp, iter);
            __syncthreads();
            tile = s_tile;
        } else {
            tile = blp_claim(blp, iter);
        }
        if (tile < 0) break;
        size_t begin = (size_t)tile * tile_elems;
        size_t end = begin + tile_elems < n ? begin + tile_elems : n;
        size_t len = end - begin;
        // Tiles start on multiples of tile_elems (a multiple of 4 elements), so the float4
        // path is aligned whenever x and y are 16-byte aligned, which the entry point checks.
        const float4 *x4 = reinterpret_cast<const float4 *>(x + begin);
        float4 *y4 = reinterpret_cast<float4 *>(y + begin);
        size_t n4 = len / 4;
        size_t i4 = 0;
        constexpr int VEC = 4;
        for (; i4 + (size_t)VEC * kAxpyThreads <= n4; i4 += (size_t)VEC * kAxpyThreads)
            axpy_tile_vec<VEC>(a, x4, y4, i4);
        for (size_t i = i4 + threadIdx.x; i < n4; i += kAxpyThreads) {
            float4 xv = __ldcs(x4 + i), yv = __ldcs(y4 + i), r;
            r.x = fmaf(a, xv.x, yv.x);
            r.y = fmaf(a, xv.y, yv.y);
            r.z = fmaf(a, xv.z, yv.z);
            r.w = fmaf(a, xv.w, yv.w);
            __stcs(y4 + i, r);
        }
        for (size_t i = begin + n4 * 4 + threadIdx.x; i < end; i += kAxpyThreads)
            y[i] = fmaf(a, x[i], y[i]);
        ++iter;
        if (dynamic) __syncthreads();  // s_tile is rewritten by thread 0 in the next round
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

static int axpy_tile_count(size_t n, size_t tile_elems, size_t *tile_out, int *tiles) {
    if (tile_elems == 0) tile_elems = kAxpyDefaultTile;
    GPX_REQUIRE(tile_elems % 4 == 0, GPX_OUT_OF_RANGE, "tile_elems must be a multiple of 4");
    size_t t = (n + tile_elems - 1) / tile_elems;
    GPX_REQUIRE(t <= 0x7fffffffull, GPX_OUT_OF_RANGE, "too many tiles (%zu)", t);
    *tile_out = tile_elems;
    *tiles = (int)t;
    return GPX_SUCC;
}

}  // namespace gpx

using namespace gpx;

extern "C" {

int gpx_axpy_tiles(size_t n, size_t tile_elems, int *tiles) {
    GPX_REQUIRE(tiles, GPX_FAIL, "tiles is NULL");
    size_t te;
    return axpy_tile_count(n, tile_elems, &te, tiles);
}

int gpx_axpy_f32(float a, const void *x, void *y, size_t n, size_t tile_elems,
                 const gpx_blp *blp, gpx_stream s) {
    if (n == 0) return GPX_SUCC;
    GPX_REQUIRE(x && y, GPX_FAIL, "x or y is NULL");
    GPX_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0, GPX_FAIL,
                "x and y must be 16-byte aligned");
    size_t te;
    int tiles;
    GPX_TRY(axpy_tile_count(n, tile_elems, &te, &tiles));
    BlpArgs b{};
    b.total_tiles = tiles;
    if (blp) {
        b.preempted = (const int *)blp->preempted;
        b.stop_index = (int *)blp->stop_index;
        b.executed = (int *)blp->executed;
        b.kernel_id = blp->kernel_id;
        b.trace = (unsigned long long *)blp->trace;
        GPX_REQUIRE(!b.preempted || (b.stop_index && b.executed), GPX_FAIL,
                    "preemptible launch needs stop_index and executed");
    }
    static int max_ctas_per_sm = 0;
    if (!max_ctas_per_sm) {
        GPX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&max_ctas_per_sm, axpy_f32_kernel,
                                                               kAxpyThreads, 0));
        if (max_ctas_per_sm < 1) max_ctas_per_sm = 1;
    }
    const DeviceInfo &d = device_info();
    GPX_REQUIRE(d.device >= 0, GPX_FAIL, "gpx_init was not called");
    // Grid = resident CTAs over all SMs, like the reference's min(total_blocks, occupancy grid)
    // (src/model.cpp:373-385).
    long long grid = (long long)d.sm_count * max_ctas_per_sm;
    if (grid > tiles) grid = tiles;
    axpy_f32_kernel<<<(unsigned)grid, kAxpyThreads, 0, as_stream(s)>>>(
        a, (const float *)x, (float *)y, n, te, b);
    GPX_CUDA(cudaGetLastError());
    return GPX_SUCC;
}

}  // extern "C"
