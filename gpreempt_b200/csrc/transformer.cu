// Memory-bound transformer layers: embedding + LayerNorm, LayerNorm, multi-head attention.
//
// They stand in for the fused take/add/layer_norm, layer_norm and batch_matmul + softmax +
// batch_matmul kernels TVM generates for the reference's BERT workload
// (scripts/compile/compile-bert.py:33-91 traces the encoder; src/executor.cpp:157-162 replays
// the kernels).  Activations are [token][channel] matrices in the split-plane format of
// act_layout.h; all arithmetic is fp32 with a fixed reduction order, every kernel walks its
// tiles through the block-level preemption loop (scripts/compile/convert_to_blp.py:39-70), so a
// preempted and resumed run is bit-identical to an uninterrupted one.
#include "layers.cuh"

namespace gpx {

constexpr int kTfThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int sh = 16; sh >= 1; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
    return v;
}

// One warp normalises one row of H <= 1024 channels held in registers (up to four 8-channel
// vectors per lane): mean, then the variance of the deviations, then scale and shift.
constexpr int kLnMaxVec = 4;

__device__ __forceinline__ void layer_norm_row(float (&x)[kLnMaxVec][8], int nvec, int H, const float *gamma,
                                               const float *beta, float eps, int lane) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kLnMaxVec; ++i)
        if (i < nvec)
#pragma unroll
            for (int j = 0; j < 8; ++j) s += x[i][j];
    const float mean = warp_sum(s) / (float)H;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kLnMaxVec; ++i)
        if (i < nvec)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float d = x[i][j] - mean;
                ss += d * d;
            }
    const float rstd = rsqrtf(warp_sum(ss) / (float)H + eps);
#pragma unroll
    for (int i = 0; i < kLnMaxVec; ++i)
        if (i < nvec) {
            const int c0 = (lane + 32 * i) * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) x[i][j] = (x[i][j] - mean) * rstd * gamma[c0 + j] + beta[c0 + j];
        }
}

// Rows of a [rows][H] matrix, one warp per row, eight rows per tile.
__global__ void __launch_bounds__(kTfThreads)
layernorm_kernel(const __grid_constant__ LayerNormParams p, BlpArgs blp) {
    pdl_enter();
    __shared__ int s_tile;
    const bool dynamic = blp.preempted != nullptr;
    if (threadIdx.x == 0) trace_begin(blp);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int V = p.H / 8;
    int iter = 0;
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
        const int row = tile * (kTfThreads / 32) + wid;
        if (row < p.rows) {
            float x[kLnMaxVec][8];
            int nvec = 0;
#pragma unroll
            for (int i = 0; i < kLnMaxVec; ++i) {
                const int v = lane + 32 * i;
                if (v < V) {
                    nvec = i + 1;
                    if (p.ids) {
                        // embedding row: word + position (+ token type 0 where the model has that table)
                        const long long id = p.ids[row];
                        const int pos = row % p.S;
                        const float4 *w = reinterpret_cast<const float4 *>(p.word + (size_t)id * p.H + v * 8);
                        const float4 *q = reinterpret_cast<const float4 *>(p.pos + (size_t)pos * p.H + v * 8);
                        float4 a0 = w[0], a1 = w[1], b0 = q[0], b1 = q[1];
                        float4 c0 = make_float4(0.f, 0.f, 0.f, 0.f), c1 = c0;
                        if (p.type) {
                            const float4 *t = reinterpret_cast<const float4 *>(p.type + v * 8);
                            c0 = t[0];
                            c1 = t[1];
                        }
                        x[i][0] = a0.x + b0.x + c0.x;
                        x[i][1] = a0.y + b0.y + c0.y;
                        x[i][2] = a0.z + b0.z + c0.z;
                        x[i][3] = a0.w + b0.w + c0.w;
                        x[i][4] = a1.x + b1.x + c1.x;
                        x[i][5] = a1.y + b1.y + c1.y;
                        x[i][6] = a1.z + b1.z + c1.z;
                        x[i][7] = a1.w + b1.w + c1.w;
                    } else {
                        const size_t off = (size_t)row * p.H + v * 8;
                        planes_load8(p.in_hi, p.in_lo, off, p.fmt, x[i]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) x[i][j] = 0.f;
                }
            }
            layer_norm_row(x, nvec, p.H, p.gamma, p.beta, p.eps, lane);
#pragma unroll
            for (int i = 0; i < kLnMaxVec; ++i) {
                const int v = lane + 32 * i;
                if (v < V) {
                    const size_t off = (size_t)row * p.H + v * 8;
                    if (p.out_f32) {
                        float4 *o = reinterpret_cast<float4 *>(p.out_f32 + off);
                        o[0] = make_float4(x[i][0], x[i][1], x[i][2], x[i][3]);
                        o[1] = make_float4(x[i][4], x[i][5], x[i][6], x[i][7]);
                    } else {
                        planes_store8(p.out_hi, p.out_lo, off, p.fmt, x[i]);
                    }
                }
            }
        }
        ++iter;
        if (dynamic) __syncthreads();
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

cudaError_t layernorm_launch(const LayerNormParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    launch_layer(layernorm_kernel, grid, kTfThreads, 0, s, p, blp);
    return cudaGetLastError();
}

// ---- multi-head attention ---------------------------------------------------------------------

constexpr int kAttnThreads = 128;  // 32 queries x 4 key partitions
constexpr int kAttnKeys = 64;      // keys per shared-memory block
constexpr int kAttnDh = 64;        // head dimension
constexpr int kAttnLd = kAttnDh + 4;

// softmax(Q K^T / sqrt(d)) V for one (batch, head, block of 32 queries) per tile.  Four lanes
// share a query: lane `part` walks keys part, part+4, ... of every 64-key block with an online
// softmax (running maximum m, normaliser l, weighted sum o), the four partial results are merged
// in a fixed order by shuffles.
__global__ void __launch_bounds__(kAttnThreads)
attention_kernel(const __grid_constant__ AttnParams p, BlpArgs blp) {
    pdl_enter();
    __shared__ int s_tile;
    __shared__ __align__(16) float Ks[kAttnKeys][kAttnLd];
    __shared__ __align__(16) float Vs[kAttnKeys][kAttnLd];
    const bool dynamic = blp.preempted != nullptr;
    if (threadIdx.x == 0) trace_begin(blp);
    const int tid = threadIdx.x;
    const int qi = tid >> 2, part = tid & 3;
    const int qblocks = (p.S + 31) / 32;
    int iter = 0;
    for (;;) {
        int tile;
        if (dynamic) {
            if (tid == 0) s_tile = blp_claim(blp, iter);
            __syncthreads();
            tile = s_tile;
        } else {
            tile = blp_claim(blp, iter);
        }
        if (tile < 0) break;
        const int qb = tile % qblocks;
        const int head = (tile / qblocks) % p.heads;
        const int b = tile / (qblocks * p.heads);
        const int qrow = qb * 32 + qi;
        const bool qvalid = qrow < p.S;
        const size_t col = (size_t)head * kAttnDh;
        float q[kAttnDh], o[kAttnDh];
#pragma unroll
        for (int d = 0; d < kAttnDh; ++d) o[d] = 0.f;
        {
            const size_t off = ((size_t)b * p.S + (qvalid ? qrow : 0)) * p.ld + col;
#pragma unroll
            for (int v = 0; v < kAttnDh / 8; ++v) {
                float x[8];
                planes_load8(p.q_hi, p.q_lo, off + v * 8, p.fmt, x);
#pragma unroll
                for (int j = 0; j < 8; ++j) q[v * 8 + j] = x[j] * p.scale;
            }
        }
        float m = -INFINITY, l = 0.f;
        for (int k0 = 0; k0 < p.S; k0 += kAttnKeys) {
            // stage 64 keys and values of this head as fp32
            for (int e = tid; e < kAttnKeys * (kAttnDh / 8); e += kAttnThreads) {
                const int kr = e / (kAttnDh / 8), v = e % (kAttnDh / 8);
                float kx[8], vx[8];
                if (k0 + kr < p.S) {
                    const size_t off = ((size_t)b * p.S + k0 + kr) * p.ld + col + v * 8;
                    planes_load8(p.k_hi, p.k_lo, off, p.fmt, kx);
                    planes_load8(p.v_hi, p.v_lo, off, p.fmt, vx);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) kx[j] = vx[j] = 0.f;
                }
                *reinterpret_cast<float4 *>(&Ks[kr][v * 8]) = make_float4(kx[0], kx[1], kx[2], kx[3]);
                *reinterpret_cast<float4 *>(&Ks[kr][v * 8 + 4]) = make_float4(kx[4], kx[5], kx[6], kx[7]);
                *reinterpret_cast<float4 *>(&Vs[kr][v * 8]) = make_float4(vx[0], vx[1], vx[2], vx[3]);
                *reinterpret_cast<float4 *>(&Vs[kr][v * 8 + 4]) = make_float4(vx[4], vx[5], vx[6], vx[7]);
            }
            __syncthreads();
            for (int j = part; j < kAttnKeys; j += 4) {
                if (k0 + j >= p.S) break;
                float sc = 0.f;
#pragma unroll
                for (int d = 0; d < kAttnDh; d += 4) {
                    float4 kv = *reinterpret_cast<const float4 *>(&Ks[j][d]);
                    sc = fmaf(q[d], kv.x, sc);
                    sc = fmaf(q[d + 1], kv.y, sc);
                    sc = fmaf(q[d + 2], kv.z, sc);
                    sc = fmaf(q[d + 3], kv.w, sc);
                }
                if (sc > m) {
                    const float corr = __expf(m - sc);  // 0 on the first key (m = -inf)
                    l *= corr;
#pragma unroll
                    for (int d = 0; d < kAttnDh; ++d) o[d] *= corr;
                    m = sc;
                }
                const float w = __expf(sc - m);
                l += w;
#pragma unroll
                for (int d = 0; d < kAttnDh; d += 4) {
                    float4 vv = *reinterpret_cast<const float4 *>(&Vs[j][d]);
                    o[d] = fmaf(w, vv.x, o[d]);
                    o[d + 1] = fmaf(w, vv.y, o[d + 1]);
                    o[d + 2] = fmaf(w, vv.z, o[d + 2]);
                    o[d + 3] = fmaf(w, vv.w, o[d + 3]);
                }
            }
            __syncthreads();
        }
        // merge the four partitions of a query (lanes 4q .. 4q+3)
        float mm = m;
        mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 1));
        mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 2));
        const float corr = m == -INFINITY ? 0.f : __expf(m - mm);
        l *= corr;
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const float inv = 1.0f / l;
        float mine[16];
#pragma unroll
        for (int d = 0; d < kAttnDh; ++d) {
            float v = o[d] * corr;
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if ((d >> 4) == part) mine[d & 15] = v * inv;
        }
        if (qvalid) {
            const size_t off = ((size_t)b * p.S + qrow) * p.ld + col + part * 16;
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                float x[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] = mine[v * 8 + j];
                planes_store8(p.out_hi, p.out_lo, off + v * 8, p.fmt, x);
            }
        }
        ++iter;
    }
    if (tid == 0) trace_end(blp, iter);
}

cudaError_t attention_launch(const AttnParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    launch_layer(attention_kernel, grid, kAttnThreads, 0, s, p, blp);
    return cudaGetLastError();
}

}  // namespace gpx
