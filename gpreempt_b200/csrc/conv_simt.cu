// fp32 convolution / dense layer as an implicit GEMM on the CUDA cores (FFMA), with the
// bias + residual + ReLU epilogue fused and block-level preemption at output-tile granularity.
// It stands in for the TVM-generated fused conv2d / dense kernels the reference replays
// (src/executor.cpp:157-162); the preemption loop is the native form of
// scripts/compile/convert_to_blp.py:39-70.
//
// Exact fp32 arithmetic (one FFMA per multiply-add, K walked in increasing order inside one
// thread), so the result does not depend on which CTA runs a tile: preempt + resume is
// bit-identical to an uninterrupted run.
#include "layers.cuh"

namespace gpx {

constexpr int kConvThreads = 256;
constexpr int kConvBK = 16;

template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__(kConvThreads)
conv_simt_kernel(ConvParams p, BlpArgs blp) {
    constexpr int BK = kConvBK;
    static_assert((BM / TM) * (BN / TN) == kConvThreads, "thread layout");
    constexpr int SA = (BM * 4 + kConvThreads - 1) / kConvThreads;  // float4 slots of A per thread
    constexpr int SB = (BN * 4 + kConvThreads - 1) / kConvThreads;  // float4 slots of B per thread
    constexpr int EA = BM / 16;  // scalar A elements per thread on the generic path
    static_assert(EA <= SA * 4, "register staging too small");

    __shared__ __align__(16) float As[2][BK][BM + 4];
    __shared__ __align__(16) float Bs[2][BK][BN + 4];
    __shared__ int s_tile;

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);
    const int ty = tid / (BN / TN);
    const bool vecA = (p.Cin % BK == 0) && !p.in_nchw;
    const int nchunks = (p.K + BK - 1) / BK;
    const bool dynamic = blp.preempted != nullptr;

    if (tid == 0) trace_begin(blp);
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
        const int m0 = (tile % p.tiles_m) * BM;
        const int n0 = (tile / p.tiles_m) * BN;

        // Pixel coordinates of the A rows this thread stages; fixed for the whole tile.
        int row_n[SA], row_h[SA], row_w[SA];
#pragma unroll
        for (int j = 0; j < SA; ++j) {
            int r = vecA ? (tid + j * kConvThreads) / 4 : (tid % BM);
            int m = m0 + r;
            bool ok = (r < BM) && (m < p.M);
            int mm = ok ? m : 0;
            int wo = mm % p.Wo;
            int t = mm / p.Wo;
            int ho = t % p.Ho;
            row_n[j] = ok ? t / p.Ho : -1;
            row_h[j] = ho * p.stride - p.pad;
            row_w[j] = wo * p.stride - p.pad;
        }

        float ra[SA * 4];
        float4 rb[SB];

        auto load_chunk = [&](int c) {
            const int k0 = c * BK;
            if (vecA) {
                // A BK-wide chunk lies inside one filter tap because Cin % BK == 0.
                const int tap = k0 / p.Cin;
                const int ci0 = k0 - tap * p.Cin;
                const int fh = tap / p.kw;
                const int fw = tap - fh * p.kw;
#pragma unroll
                for (int j = 0; j < SA; ++j) {
                    int i = tid + j * kConvThreads;
                    int q = i & 3;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    int hi = row_h[j] + fh, wi = row_w[j] + fw;
                    if (i < BM * 4 && row_n[j] >= 0 && hi >= 0 && hi < p.H && wi >= 0 &&
                        wi < p.W) {
                        size_t off = (((size_t)row_n[j] * p.H + hi) * p.W + wi) * p.Cin + ci0 +
                                     q * 4;
                        v = *reinterpret_cast<const float4 *>(p.in + off);
                    }
                    ra[j * 4 + 0] = v.x;
                    ra[j * 4 + 1] = v.y;
                    ra[j * 4 + 2] = v.z;
                    ra[j * 4 + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int e = 0; e < EA; ++e) {
                    int kk = tid / BM + e * (kConvThreads / BM);
                    int k = k0 + kk;
                    float v = 0.f;
                    if (k < p.K && row_n[0] >= 0) {
                        int tap = k / p.Cin;
                        int ci = k - tap * p.Cin;
                        int fh = tap / p.kw;
                        int fw = tap - fh * p.kw;
                        int hi = row_h[0] + fh, wi = row_w[0] + fw;
                        if (hi >= 0 && hi < p.H && wi >= 0 && wi < p.W) {
                            size_t off =
                                p.in_nchw
                                    ? (((size_t)row_n[0] * p.Cin + ci) * p.H + hi) * p.W + wi
                                    : (((size_t)row_n[0] * p.H + hi) * p.W + wi) * p.Cin + ci;
                            v = p.in[off];
                        }
                    }
                    ra[e] = v;
                }
            }
#pragma unroll
            for (int j = 0; j < SB; ++j) {
                int i = tid + j * kConvThreads;
                int kk = i / (BN / 4);
                int c4 = i - kk * (BN / 4);
                int k = k0 + kk;
                int n = n0 + c4 * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < BN * 4 && k < p.K && n < p.Cout)
                    v = *reinterpret_cast<const float4 *>(p.w + (size_t)k * p.Cout + n);
                rb[j] = v;
            }
        };

        auto store_chunk = [&](int buf) {
            if (vecA) {
#pragma unroll
                for (int j = 0; j < SA; ++j) {
                    int i = tid + j * kConvThreads;
                    if (i < BM * 4) {
                        int r = i >> 2, q = i & 3;
                        As[buf][q * 4 + 0][r] = ra[j * 4 + 0];
                        As[buf][q * 4 + 1][r] = ra[j * 4 + 1];
                        As[buf][q * 4 + 2][r] = ra[j * 4 + 2];
                        As[buf][q * 4 + 3][r] = ra[j * 4 + 3];
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < EA; ++e) {
                    int kk = tid / BM + e * (kConvThreads / BM);
                    As[buf][kk][tid % BM] = ra[e];
                }
            }
#pragma unroll
            for (int j = 0; j < SB; ++j) {
                int i = tid + j * kConvThreads;
                if (i < BN * 4) {
                    int kk = i / (BN / 4);
                    int c4 = i - kk * (BN / 4);
                    *reinterpret_cast<float4 *>(&Bs[buf][kk][c4 * 4]) = rb[j];
                }
            }
        };

        float acc[TM][TN];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

        load_chunk(0);
        store_chunk(0);
        __syncthreads();
        for (int c = 0; c < nchunks; ++c) {
            const int buf = c & 1;
            if (c + 1 < nchunks) load_chunk(c + 1);
#pragma unroll
            for (int k = 0; k < BK; ++k) {
                float a[TM], b[TN];
#pragma unroll
                for (int i = 0; i < TM; ++i) a[i] = As[buf][k][ty * TM + i];
#pragma unroll
                for (int j = 0; j < TN; ++j) b[j] = Bs[buf][k][tx * TN + j];
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            }
            if (c + 1 < nchunks) store_chunk(buf ^ 1);
            __syncthreads();
        }

        // Epilogue: + bias, + residual, ReLU; NHWC rows are GEMM rows.
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            int m = m0 + ty * TM + i;
            if (m >= p.M) continue;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                int n = n0 + tx * TN + j;
                if (n >= p.Cout) continue;
                float v = acc[i][j];
                if (p.bias) v += p.bias[n];
                if (p.res) v += p.res[(size_t)m * p.Cout + n];
                if (p.relu) v = fmaxf(v, 0.f);
                p.out[(size_t)m * p.Cout + n] = v;
            }
        }
        ++iter;
    }
    if (tid == 0) trace_end(blp, iter);
}

static void tile_dims(int tile, int &bm, int &bn) {
    switch (tile) {
        case CONV_TILE_128: bm = 128; bn = 128; break;
        case CONV_TILE_64: bm = 64; bn = 64; break;
        default: bm = 32; bn = 32; break;
    }
}

void conv_set_tiles(ConvParams &p, int tile) {
    int bm, bn;
    tile_dims(tile, bm, bn);
    p.tiles_m = (p.M + bm - 1) / bm;
    p.tiles_n = (p.Cout + bn - 1) / bn;
}

int conv_pick_tile(const ConvParams &p, int sm_count) {
    // Largest tile that still yields about two waves of CTAs; small-M layers (batch 1, late
    // stages) fall through to the smallest tile to expose parallelism.
    for (int tile = CONV_TILE_128; tile <= CONV_TILE_32; ++tile) {
        int bm, bn;
        tile_dims(tile, bm, bn);
        long long tiles = (long long)((p.M + bm - 1) / bm) * ((p.Cout + bn - 1) / bn);
        if (tiles >= 2LL * sm_count || tile == CONV_TILE_32) return tile;
    }
    return CONV_TILE_32;
}

template <int BM, int BN, int TM, int TN>
static int occupancy() {
    static int v = 0;
    if (!v) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, conv_simt_kernel<BM, BN, TM, TN>,
                                                          kConvThreads, 0) != cudaSuccess ||
            v < 1)
            v = 1;
    }
    return v;
}

int conv_grid(const ConvParams &p, int tile, int sm_count, bool preemptible) {
    (void)preemptible;
    long long tiles = (long long)p.tiles_m * p.tiles_n;
    int occ = tile == CONV_TILE_128   ? occupancy<128, 128, 8, 8>()
              : tile == CONV_TILE_64 ? occupancy<64, 64, 4, 4>()
                                     : occupancy<32, 32, 2, 2>();
    // Persistent grid: min(total tiles, resident CTAs), as Model::add_block_preemption_param
    // sizes it in the reference (src/model.cpp:373-385).
    long long grid = (long long)sm_count * occ;
    if (grid > tiles) grid = tiles;
    if (grid < 1) grid = 1;
    return (int)grid;
}

cudaError_t conv_launch(const ConvParams &p, int tile, int grid, const BlpArgs &blp,
                        cudaStream_t s) {
    switch (tile) {
        case CONV_TILE_128:
            conv_simt_kernel<128, 128, 8, 8><<<grid, kConvThreads, 0, s>>>(p, blp);
            break;
        case CONV_TILE_64:
            conv_simt_kernel<64, 64, 4, 4><<<grid, kConvThreads, 0, s>>>(p, blp);
            break;
        default:
            conv_simt_kernel<32, 32, 2, 2><<<grid, kConvThreads, 0, s>>>(p, blp);
            break;
    }
    return cudaGetLastError();
}

// ---- pooling ------------------------------------------------------------------------------

constexpr int kPoolThreads = 256;

// Max / average pooling over NHWC, one float4 of channels per thread-iteration.  A tile is
// tile_elems consecutive output float4 vectors.
__global__ void __launch_bounds__(kPoolThreads) pool_kernel(PoolParams p, BlpArgs blp) {
    __shared__ int s_tile;
    const bool dynamic = blp.preempted != nullptr;
    if (threadIdx.x == 0) trace_begin(blp);
    const int C4 = p.C / 4;
    const long long total = (long long)p.N * p.Ho * p.Wo * C4;
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
        long long begin = (long long)tile * p.tile_elems;
        long long end = begin + p.tile_elems < total ? begin + p.tile_elems : total;
        for (long long e = begin + threadIdx.x; e < end; e += kPoolThreads) {
            int c4 = (int)(e % C4);
            long long t = e / C4;
            int wo = (int)(t % p.Wo);
            t /= p.Wo;
            int ho = (int)(t % p.Ho);
            int n = (int)(t / p.Ho);
            float4 acc = p.mode == 0 ? make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY)
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
            int cnt = 0;
            for (int fh = 0; fh < p.k; ++fh) {
                int hi = ho * p.stride - p.pad + fh;
                if (hi < 0 || hi >= p.H) continue;
                for (int fw = 0; fw < p.k; ++fw) {
                    int wi = wo * p.stride - p.pad + fw;
                    if (wi < 0 || wi >= p.W) continue;
                    float4 v = *reinterpret_cast<const float4 *>(
                        p.in + (((size_t)n * p.H + hi) * p.W + wi) * p.C + c4 * 4);
                    if (p.mode == 0) {
                        acc.x = fmaxf(acc.x, v.x);
                        acc.y = fmaxf(acc.y, v.y);
                        acc.z = fmaxf(acc.z, v.z);
                        acc.w = fmaxf(acc.w, v.w);
                    } else {
                        acc.x += v.x;
                        acc.y += v.y;
                        acc.z += v.z;
                        acc.w += v.w;
                    }
                    ++cnt;
                }
            }
            if (p.mode == 1) {
                float inv = 1.0f / (float)cnt;
                acc.x *= inv;
                acc.y *= inv;
                acc.z *= inv;
                acc.w *= inv;
            }
            *reinterpret_cast<float4 *>(p.out + (size_t)e * 4) = acc;
        }
        ++iter;
        if (dynamic) __syncthreads();
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

int pool_grid(const PoolParams &p, int sm_count) {
    long long grid = (long long)sm_count * 8;
    if (grid > p.total_tiles) grid = p.total_tiles;
    if (grid < 1) grid = 1;
    return (int)grid;
}

cudaError_t pool_launch(const PoolParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    pool_kernel<<<grid, kPoolThreads, 0, s>>>(p, blp);
    return cudaGetLastError();
}

}  // namespace gpx
