// Convolution / dense layer as an implicit GEMM on the CUDA cores (fp32 FFMA), pooling and
// sub-sampling; block-level preemption at output-tile granularity.
//
// These kernels cover what the tensor-core convolution does not: the stem (fp32 NCHW input with
// three channels), dense layers with a handful of rows, and the memory-bound layers.  They stand
// in for TVM-generated fused kernels the reference replays (src/executor.cpp:157-162); the
// preemption loop is the native form of scripts/compile/convert_to_blp.py:39-70.
//
// One FFMA per multiply-add with K walked in increasing order inside one thread, so the result
// does not depend on which CTA runs a tile: preempt + resume is bit-identical.
#include "layers.cuh"

namespace gpx {

constexpr int kConvThreads = 256;
constexpr int kConvBK = 16;

__device__ __forceinline__ float bf16_bits_to_f32(bf16_bits v) {
    return __uint_as_float((unsigned)v << 16);
}
__device__ __forceinline__ bf16_bits f32_to_bf16_bits(float f) {
    unsigned u = __float_as_uint(f);
    u += 0x7fffu + ((u >> 16) & 1u);  // round to nearest even (finite inputs)
    return (bf16_bits)(u >> 16);
}

__device__ __forceinline__ float view_load(const ActView &v, int n, int h, int w, int c) {
    if (v.f32) return v.f32[(((size_t)n * v.l.C + c) * v.l.H + h) * v.l.W + w];
    size_t off = (size_t)layout_row(v.l, n, h, w) * v.l.C + c;
    return planes_load1(v.hi, v.lo, off, v.l.fmt);
}

template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__(kConvThreads)
conv_simt_kernel(const __grid_constant__ ConvParams p, BlpArgs blp) {
    pdl_enter();
    constexpr int BK = kConvBK;
    static_assert((BM / TM) * (BN / TN) == kConvThreads, "thread layout");
    constexpr int SB = (BN * 4 + kConvThreads - 1) / kConvThreads;  // float4 slots of B per thread
    constexpr int EA = BM / 16;                                      // A elements per thread

    __shared__ __align__(16) float As[2][BK][BM + 4];
    __shared__ __align__(16) float Bs[2][BK][BN + 4];
    __shared__ int s_tile;

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);
    const int ty = tid / (BN / TN);
    const int nchunks = (p.K + BK - 1) / BK;
    const bool dynamic = blp.preempted != nullptr;
    const int H = p.in.l.H, W = p.in.l.W;

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

        // Output pixel of the A row this thread stages; fixed for the whole tile.
        int row_n, row_h, row_w;
        {
            int m = m0 + tid % BM;
            bool ok = m < p.M;
            int mm = ok ? m : 0;
            int wo = mm % p.Wo;
            int t = mm / p.Wo;
            int ho = t % p.Ho;
            row_n = ok ? t / p.Ho : -1;
            row_h = ho * p.stride - p.pad;
            row_w = wo * p.stride - p.pad_w;
        }

        float ra[EA];
        float4 rb[SB];

        auto load_chunk = [&](int c) {
            const int k0 = c * BK;
#pragma unroll
            for (int e = 0; e < EA; ++e) {
                int kk = tid / BM + e * (kConvThreads / BM);
                int k = k0 + kk;
                float v = 0.f;
                if (k < p.K && row_n >= 0) {
                    int tap = k / p.Cin;
                    int ci = k - tap * p.Cin;
                    int fh = tap / p.kw;
                    int fw = tap - fh * p.kw;
                    int hi = row_h + fh, wi = row_w + fw;
                    if (hi >= 0 && hi < H && wi >= 0 && wi < W) v = view_load(p.in, row_n, hi, wi, ci);
                }
                ra[e] = v;
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
#pragma unroll
            for (int e = 0; e < EA; ++e) {
                int kk = tid / BM + e * (kConvThreads / BM);
                As[buf][kk][tid % BM] = ra[e];
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

        // Epilogue: + bias, + residual, ReLU; rows go to the consumer's layout.
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            int m = m0 + ty * TM + i;
            if (m >= p.M) continue;
            int wo = m % p.Wo;
            int t = m / p.Wo;
            int ho = t % p.Ho;
            int n_img = t / p.Ho;
            size_t out_row = p.out_f32 ? (size_t)m : (size_t)layout_row(p.out, n_img, ho, wo);
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                int n = n0 + tx * TN + j;
                if (n >= p.Cout) continue;
                float v = acc[i][j];
                if (p.bias) v += p.bias[n];
                if (p.res.hi || p.res.f32) v += view_load(p.res, n_img, ho, wo, n);
                v = apply_act(v, p.relu);
                if (p.out_f32) {
                    p.out_f32[out_row * p.Cout + n] = v;
                } else {
                    // the row stride is the stored channel count, which may exceed Cout
                    planes_store1(p.out_hi, p.out_lo, out_row * p.out.C + n, p.out.fmt, v);
                }
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
    // Largest tile that still yields about two waves of CTAs; small-M layers fall through to
    // the smallest tile to expose parallelism.
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

int conv_grid(const ConvParams &p, int tile, int sm_count) {
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
            launch_layer(conv_simt_kernel<128, 128, 8, 8>, grid, kConvThreads, 0, s, p, blp);
            break;
        case CONV_TILE_64:
            launch_layer(conv_simt_kernel<64, 64, 4, 4>, grid, kConvThreads, 0, s, p, blp);
            break;
        default:
            launch_layer(conv_simt_kernel<32, 32, 2, 2>, grid, kConvThreads, 0, s, p, blp);
            break;
    }
    return cudaGetLastError();
}

// ---- pooling / sub-sampling ---------------------------------------------------------------

constexpr int kPoolThreads = 256;

// Eight channels of one input pixel as fp32: the sum of the planes, then the optional
// per-channel affine + activation of PoolParams.
__device__ __forceinline__ void pool_load8(const PoolParams &p, size_t off, int c0, float (&x)[8]) {
    planes_load8(p.in.hi, p.in.lo, off, p.in.l.fmt, x);
    if (p.scale) {
        const float4 *sc = reinterpret_cast<const float4 *>(p.scale + c0);
        const float4 *sh = reinterpret_cast<const float4 *>(p.shift + c0);
        float4 s0 = __ldg(sc), s1 = __ldg(sc + 1), h0 = __ldg(sh), h1 = __ldg(sh + 1);
        const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const float hv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = fmaf(x[j], sv[j], hv[j]);
        apply_act_n(x, p.act);
    }
}

__device__ __forceinline__ void pool_store8(const PoolParams &p, size_t off, const float (&x)[8]) {
    planes_store8(p.out_hi, p.out_lo, off, p.out.fmt, x);
}

// Max / average pooling, or a strided copy, over split-plane activations; eight channels (one
// 16-byte vector per plane) per thread-iteration.  A tile is tile_elems consecutive output
// vectors in (n, ho, wo, c/8) order.
// kMax3 selects the 3x3 max-pooling instance, which keeps nine taps in registers and so runs at a
// lower occupancy than the other modes want.
template <bool kMax3>
__global__ void __launch_bounds__(kPoolThreads)
pool_kernel(const __grid_constant__ PoolParams p, BlpArgs blp) {
    pdl_enter();
    __shared__ int s_tile;
    const bool dynamic = blp.preempted != nullptr;
    if (threadIdx.x == 0) trace_begin(blp);
    const int Cin = p.in.l.C, Cout = p.out.C;  // row strides
    const int C8 = p.channels / 8;
    const int Ho = p.out.H, Wo = p.out.W;
    const int H = p.in.l.H, W = p.in.l.W;
    const unsigned total = (unsigned)p.out.N * Ho * Wo * C8;  // < 2^31, checked when the model is built
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
        const unsigned begin = (unsigned)tile * p.tile_elems;
        const unsigned end = begin + p.tile_elems < total ? begin + p.tile_elems : total;
        if (p.mode == 1 && p.k * p.k >= 16) {
            // Large averaging window (global average pool): one warp per output vector, lanes
            // take taps lane, lane+32, ...; a fixed shuffle tree adds the lane sums, so the
            // result is the same on every run.
            const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
            for (unsigned e = begin + wid; e < end; e += kPoolThreads / 32) {
                int c8 = (int)(e % C8);
                unsigned t = e / C8;
                int wo = (int)(t % Wo);
                t /= Wo;
                int ho = (int)(t % Ho);
                int n = (int)(t / Ho);
                float acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                int cnt = 0;
                const bool readable = c8 * 8 < p.in_valid;
                for (int tap = lane; tap < p.k * p.k; tap += 32) {
                    int fh = tap / p.k, fw = tap - fh * p.k;
                    int hi = ho * p.stride - p.pad + fh, wi = wo * p.stride - p.pad + fw;
                    if (hi < 0 || hi >= H || wi < 0 || wi >= W) continue;
                    if (readable) {
                        float x[8];
                        pool_load8(p, (size_t)layout_row(p.in.l, n, hi, wi) * Cin + c8 * 8, c8 * 8, x);
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[j] += x[j];
                    }
                    ++cnt;
                }
#pragma unroll
                for (int sh = 16; sh >= 1; sh >>= 1) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], sh);
                    cnt += __shfl_xor_sync(0xffffffffu, cnt, sh);
                }
                if (lane == 0) {
                    float inv = 1.0f / (float)cnt;
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] *= inv;
                    pool_store8(p, (size_t)layout_row(p.out, n, ho, wo) * Cout + c8 * 8, acc);
                }
            }
            ++iter;
            if (dynamic) __syncthreads();
            continue;
        }
        for (unsigned e = begin + threadIdx.x; e < end; e += kPoolThreads) {
            int c8 = (int)(e % C8);
            unsigned t = e / C8;
            int wo = (int)(t % Wo);
            t /= Wo;
            int ho = (int)(t % Ho);
            int n = (int)(t / Ho);
            float acc[8];
            const bool readable = c8 * 8 < p.in_valid;
            if (kMax3 && readable) {
                // 3x3 max pooling: the nine taps are fetched before any is converted, so a thread
                // waits for memory once instead of nine times.
                uint4 ra[9], rb[9];
                bool ok[9];
                const int fmt = p.in.l.fmt;
#pragma unroll
                for (int t9 = 0; t9 < 9; ++t9) {
                    const int hi = ho * p.stride - p.pad + t9 / 3, wi = wo * p.stride - p.pad + t9 % 3;
                    ok[t9] = hi >= 0 && hi < H && wi >= 0 && wi < W;
                    ra[t9] = rb[t9] = make_uint4(0, 0, 0, 0);
                    if (ok[t9])
                        planes_fetch8(p.in.hi, p.in.lo, (size_t)layout_row(p.in.l, n, hi, wi) * Cin + c8 * 8, fmt,
                                      ra[t9], rb[t9]);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = -INFINITY;
#pragma unroll
                for (int t9 = 0; t9 < 9; ++t9) {
                    if (!ok[t9]) continue;
                    float x[8];
                    planes_decode8(ra[t9], rb[t9], fmt, x);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] = fmaxf(acc[j], x[j]);
                }
                pool_store8(p, (size_t)layout_row(p.out, n, ho, wo) * Cout + c8 * 8, acc);
                continue;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = (p.mode == 0 && readable) ? -INFINITY : 0.f;
            int cnt = 0;
            const int kk = p.mode == 2 ? 1 : p.k;
            for (int fh = 0; fh < kk; ++fh) {
                int hi = ho * p.stride - p.pad + fh;
                if (hi < 0 || hi >= H) continue;
                for (int fw = 0; fw < kk; ++fw) {
                    int wi = wo * p.stride - p.pad + fw;
                    if (wi < 0 || wi >= W) continue;
                    ++cnt;
                    if (!readable) continue;
                    float x[8];
                    pool_load8(p, (size_t)layout_row(p.in.l, n, hi, wi) * Cin + c8 * 8, c8 * 8, x);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (p.mode == 0)
                            acc[j] = fmaxf(acc[j], x[j]);
                        else
                            acc[j] += x[j];
                    }
                }
            }
            if (p.mode == 1 || p.mode == 3) {
                float inv = 1.0f / (float)(p.mode == 1 ? cnt : p.k * p.k);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] *= inv;
            }
            pool_store8(p, (size_t)layout_row(p.out, n, ho, wo) * Cout + c8 * 8, acc);
        }
        ++iter;
        if (dynamic) __syncthreads();
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

// Patch matrix for the tensor-core GEMM: one thread-iteration writes eight consecutive columns
// (one 16-byte vector per plane) of one row.
__global__ void __launch_bounds__(kPoolThreads)
im2col_kernel(const __grid_constant__ Im2colParams p, BlpArgs blp) {
    pdl_enter();
    __shared__ int s_tile;
    const bool dynamic = blp.preempted != nullptr;
    if (threadIdx.x == 0) trace_begin(blp);
    const int K8 = p.Kp / 8;
    const unsigned total = (unsigned)p.M * K8;
    const int H = p.in.l.H, W = p.in.l.W;
    // Column k of the patch matrix is filter tap (fh, fw) of channel ci; the decomposition and,
    // for an fp32 NCHW input, the element offset relative to the window origin are tabulated
    // once per CTA (K <= 1024).
    __shared__ int s_off[1024];
    __shared__ unsigned char s_fh[1024], s_fw[1024], s_ci[1024];
    for (int k = threadIdx.x; k < p.Kp && !p.planes_vec; k += kPoolThreads) {
        int tap = k / p.Cin;
        int ci = k - tap * p.Cin;
        int fh = tap / p.kw;
        int fw = tap - fh * p.kw;
        s_fh[k] = k < p.K ? (unsigned char)fh : 255;
        s_fw[k] = (unsigned char)fw;
        s_ci[k] = (unsigned char)ci;
        s_off[k] = (ci * H + fh) * W + fw;
    }
    __syncthreads();
    int iter = 0;
    if (p.s2d) {
        // Space-to-depth windows.  One thread-iteration gathers eight of the sixteen channels of one
        // 2x2 block (hb, wb'), splits them once and stores them into the up to four pixels
        // wb' - j (j = 0..3) whose window holds that block, at channel group j.  Blocks wb' >= Wo lie
        // past the padded image and are zero; they fill the tail groups of a row's last pixels.
        const int Wx = p.Wo + 3;
        const unsigned vectors = (unsigned)p.in.l.N * p.Ho * Wx * 2;
        // channel c of a block = (dy*2 + dx)*Cin + ci: the decomposition is tabulated once
        for (int c = threadIdx.x; c < 16; c += kPoolThreads) {
            const int q = c / p.Cin;
            s_fh[c] = q < 4 ? (unsigned char)q : 255;
            s_ci[c] = (unsigned char)(c - q * p.Cin);
        }
        for (;;) {
            int tile;
            __syncthreads();
            if (dynamic) {
                if (threadIdx.x == 0) s_tile = blp_claim(blp, iter);
                __syncthreads();
                tile = s_tile;
            } else {
                tile = blp_claim(blp, iter);
            }
            if (tile < 0) break;
            const unsigned begin = (unsigned)tile * p.tile_elems;
            const unsigned end = begin + p.tile_elems < vectors ? begin + p.tile_elems : vectors;
            for (unsigned e = begin + threadIdx.x; e < end; e += kPoolThreads) {
                const int half = (int)(e & 1);
                const unsigned b = e >> 1;
                const int wb = (int)(b % Wx);
                const unsigned t = b / Wx;
                const int hb = (int)(t % p.Ho), n = (int)(t / p.Ho);
                float x[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int c = half * 8 + u;
                    const int q = s_fh[c];
                    const int hi = 2 * hb + (q >> 1) - p.pad, wi = 2 * wb + (q & 1) - p.pad;
                    float v = 0.f;
                    if (q != 255 && hi >= 0 && hi < H && wi >= 0 && wi < W)
                        v = p.in.f32[(((size_t)n * p.Cin + s_ci[c]) * H + hi) * W + wi];
                    x[u] = v;
                }
                const size_t row0 = ((size_t)n * p.Ho + hb) * p.Wo;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int wp = wb - j;  // the pixel whose window has this block at position j
                    if (wp >= 0 && wp < p.Wo)
                        planes_store8(p.out_hi, p.out_lo, (row0 + wp) * 64 + j * 16 + half * 8, p.fmt, x);
                }
            }
            ++iter;
        }
        if (threadIdx.x == 0) trace_end(blp, iter);
        return;
    }
    if (p.planes_vec) {
        const int Cs = p.in.l.C;            // stored channels of the input
        const unsigned vectors = (unsigned)p.M * K8;
        const int c8_per_tap = Cs / 8;
        const int fmt = p.fmt;
        for (;;) {
            int tile;
            __syncthreads();
            if (dynamic) {
                if (threadIdx.x == 0) s_tile = blp_claim(blp, iter);
                __syncthreads();
                tile = s_tile;
            } else {
                tile = blp_claim(blp, iter);
            }
            if (tile < 0) break;
            const unsigned begin = (unsigned)tile * p.tile_elems;
            const unsigned end = begin + p.tile_elems < vectors ? begin + p.tile_elems : vectors;
            for (unsigned e = begin + threadIdx.x; e < end; e += kPoolThreads) {
                const int k8 = (int)(e % K8);
                const unsigned m = e / K8;
                const int wo = (int)(m % p.Wo);
                const unsigned t = m / p.Wo;
                const int ho = (int)(t % p.Ho), n = (int)(t / p.Ho);
                const int tap = k8 / c8_per_tap, c8 = k8 - tap * c8_per_tap;
                const int fh = tap / p.kw, fw = tap - fh * p.kw;
                const int hi = ho * p.stride - p.pad + fh, wi = wo * p.stride - p.pad_w + fw;
                uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
                if (fh < p.kh && hi >= 0 && hi < H && wi >= 0 && wi < W)
                    planes_fetch8(p.in.hi, p.in.lo, (size_t)layout_row(p.in.l, n, hi, wi) * Cs + c8 * 8, fmt, a, b);
                const size_t off = (size_t)m * p.Kp + k8 * 8;
                *reinterpret_cast<uint4 *>(p.out_hi + off) = a;
                if (fmt == PF_SPLIT) *reinterpret_cast<uint4 *>(p.out_lo + off) = b;
            }
            ++iter;
        }
        if (threadIdx.x == 0) trace_end(blp, iter);
        return;
    }
    if (p.win_w > 0) {
        // Row-window mode.  The window of the tile - Cin x kh input rows, (win_w-1)*stride + kw
        // wide, zeros outside the image - is staged with coalesced loads; a patch-matrix element
        // is then one table lookup and one shared-memory read, and the stores stay row-contiguous.
        __shared__ float s_win[kIm2colWindowFloats];
        const int win_cols = (p.win_w - 1) * p.stride + p.kw;
        const int seg = p.Cin * p.kh;  // window rows
        for (int k = threadIdx.x; k < p.Kp; k += kPoolThreads)
            s_off[k] = s_fh[k] == 255 ? -1 : ((int)s_ci[k] * p.kh + (int)s_fh[k]) * win_cols + (int)s_fw[k];
        for (;;) {
            int tile;
            __syncthreads();  // the table is complete / the previous window has been consumed
            if (dynamic) {
                if (threadIdx.x == 0) s_tile = blp_claim(blp, iter);
                __syncthreads();
                tile = s_tile;
            } else {
                tile = blp_claim(blp, iter);
            }
            if (tile < 0) break;
            const int chunk = tile % p.win_chunks;
            const int t = tile / p.win_chunks;
            const int ho = t % p.Ho, n = t / p.Ho;
            const int wo0 = chunk * p.win_w;
            const int nw = min(p.win_w, p.Wo - wo0);
            const int h0 = ho * p.stride - p.pad, w0 = wo0 * p.stride - p.pad;
            for (int e = threadIdx.x; e < seg * win_cols; e += kPoolThreads) {
                const int r = e / win_cols, c = e - r * win_cols;
                const int ci = r / p.kh, fh = r - ci * p.kh;
                const int hi = h0 + fh, wi = w0 + c;
                float v = 0.f;
                if (hi >= 0 && hi < H && wi >= 0 && wi < W)
                    v = p.in.f32[(((size_t)n * p.Cin + ci) * H + hi) * W + wi];
                s_win[e] = v;
            }
            __syncthreads();
            const size_t m0 = ((size_t)n * p.Ho + ho) * p.Wo + wo0;
            for (int e = threadIdx.x; e < nw * K8; e += kPoolThreads) {
                const int wl = e / K8, k8 = e - wl * K8;
                const int shift = wl * p.stride;
                float x[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int off = s_off[k8 * 8 + u];
                    x[u] = off < 0 ? 0.f : s_win[off + shift];
                }
                planes_store8(p.out_hi, p.out_lo, (m0 + wl) * p.Kp + k8 * 8, p.fmt, x);
            }
            ++iter;
        }
        if (threadIdx.x == 0) trace_end(blp, iter);
        return;
    }
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
        const unsigned begin = (unsigned)tile * p.tile_elems;
        const unsigned end = begin + p.tile_elems < total ? begin + p.tile_elems : total;
        for (unsigned e = begin + threadIdx.x; e < end; e += kPoolThreads) {
            int k8 = (int)(e % K8);
            int m = (int)(e / K8);
            int wo = m % p.Wo;
            int t = m / p.Wo;
            int ho = t % p.Ho;
            int n = t / p.Ho;
            const int h0 = ho * p.stride - p.pad, w0 = wo * p.stride - p.pad;
            const long long origin = ((long long)n * p.Cin * H + h0) * W + w0;
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                int k = k8 * 8 + u;
                float v = 0.f;
                int fh = s_fh[k];
                int hi = h0 + fh, wi = w0 + s_fw[k];
                if (fh != 255 && hi >= 0 && hi < H && wi >= 0 && wi < W)
                    v = p.in.f32 ? p.in.f32[origin + s_off[k]] : view_load(p.in, n, hi, wi, s_ci[k]);
                x[u] = v;
            }
            planes_store8(p.out_hi, p.out_lo, (size_t)m * p.Kp + k8 * 8, p.fmt, x);
        }
        ++iter;
        if (dynamic) __syncthreads();
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

cudaError_t im2col_launch(const Im2colParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    launch_layer(im2col_kernel, grid, kPoolThreads, 0, s, p, blp);
    return cudaGetLastError();
}

// Finishing pass of a split-K tensor-core convolution: one thread-iteration handles eight
// channels of one GEMM row.  The per-split sums are added in split order, so the result does
// not depend on which CTA produced which split or in which order they finished.
__global__ void __launch_bounds__(kPoolThreads)
splitk_finish_kernel(const __grid_constant__ SplitKParams p, BlpArgs blp) {
    pdl_enter();
    __shared__ int s_tile;
    const bool dynamic = blp.preempted != nullptr;
    if (threadIdx.x == 0) trace_begin(blp);
    const int C8 = p.cout_padded / 8;
    const unsigned total = (unsigned)p.m_rows * C8;
    const int img = p.in_hs * p.in_ws;
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
        const unsigned begin = (unsigned)tile * p.tile_elems;
        const unsigned end = begin + p.tile_elems < total ? begin + p.tile_elems : total;
        for (unsigned e = begin + threadIdx.x; e < end; e += kPoolThreads) {
            const int c8 = (int)(e % C8);
            const int vrow = (int)(e / C8);
            const int n_img = vrow / img;
            const int r = vrow - n_img * img;
            const int hs = r / p.in_ws;
            const int h = hs - p.in_off;
            const int w = r - hs * p.in_ws - p.in_off;
            if (h < 0 || h >= p.out.H || w < 0 || w >= p.out.W) continue;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = 0.f;
            for (int s = 0; s < p.k_splits; ++s) {
                const float4 *src = reinterpret_cast<const float4 *>(
                    p.partial + ((size_t)s * p.partial_rows + vrow) * p.partial_ld + c8 * 8);
                float4 a = src[0], b = src[1];
                f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
                f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
            }
            splitk_apply(p, n_img, h, w, c8 * 8, f);
        }
        ++iter;
        if (dynamic) __syncthreads();
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

__global__ void __launch_bounds__(kPoolThreads)
dense_rows_kernel(const __grid_constant__ DenseRowsParams p, BlpArgs blp) {
    pdl_enter();
    __shared__ int s_tile;
    __shared__ float s_part[kPoolThreads / 32][8];
    const bool dynamic = blp.preempted != nullptr;
    if (threadIdx.x == 0) trace_begin(blp);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    constexpr int kStep = kPoolThreads * 8;  // elements of one row the CTA reads per step (4 KB per plane)
    constexpr int kU = 4;
    int iter = 0;
    for (;;) {
        int tile;
        __syncthreads();
        if (dynamic) {
            if (threadIdx.x == 0) s_tile = blp_claim(blp, iter);
            __syncthreads();
            tile = s_tile;
        } else {
            tile = blp_claim(blp, iter);
        }
        if (tile < 0) break;
        // A tile is eight output columns, one after the other; the whole CTA walks one weight row
        // with consecutive threads on consecutive 16-byte vectors, so that DRAM sees long
        // contiguous reads (one warp per row opened a new DRAM page with every 512 bytes and
        // reached a quarter of the bandwidth).
        for (int c = 0; c < 8; ++c) {
            const int n = tile * 8 + c;
            if (n >= p.cout) break;
            float acc[8];
#pragma unroll
            for (int m = 0; m < 8; ++m) acc[m] = 0.f;
            const size_t w_row = (size_t)n * p.w_ld;
            for (int k0 = threadIdx.x * 8; k0 < p.K; k0 += kStep * kU) {
                uint4 wa[kU], wb[kU];
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    wa[u] = wb[u] = make_uint4(0, 0, 0, 0);
                    if (k0 + u * kStep < p.K) planes_fetch8(p.w_hi, p.w_lo, w_row + k0 + u * kStep, p.fmt, wa[u], wb[u]);
                }
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    if (k0 + u * kStep >= p.K) break;
                    float w[8];
                    planes_decode8(wa[u], wb[u], p.fmt, w);
#pragma unroll
                    for (int m = 0; m < 8; ++m) {
                        if (m < p.M) {
                            float a[8];
                            planes_load8(p.a_hi, p.a_lo, (size_t)m * p.a_ld + k0 + u * kStep, p.fmt, a);
#pragma unroll
                            for (int j = 0; j < 8; ++j) acc[m] = fmaf(a[j], w[j], acc[m]);
                        }
                    }
                }
            }
#pragma unroll
            for (int sh = 16; sh >= 1; sh >>= 1)
#pragma unroll
                for (int m = 0; m < 8; ++m) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], sh);
            __syncthreads();  // the previous column's partial sums have been consumed
            if (lane == 0)
#pragma unroll
                for (int m = 0; m < 8; ++m) s_part[wid][m] = acc[m];
            __syncthreads();
            if (threadIdx.x < p.M) {
                const int m = threadIdx.x;
                float v = 0.f;
#pragma unroll
                for (int w8 = 0; w8 < kPoolThreads / 32; ++w8) v += s_part[w8][m];  // fixed order
                v = apply_act(v + (p.bias ? p.bias[n] : 0.f), p.relu);
                if (p.out_f32)
                    p.out_f32[(size_t)m * p.cout + n] = v;
                else
                    planes_store1(p.out_hi, p.out_lo, (size_t)m * p.out_ld + n, p.fmt, v);
            }
        }
        ++iter;
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

cudaError_t dense_rows_launch(const DenseRowsParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    launch_layer(dense_rows_kernel, grid, kPoolThreads, 0, s, p, blp);
    return cudaGetLastError();
}

cudaError_t splitk_launch(const SplitKParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    launch_layer(splitk_finish_kernel, grid, kPoolThreads, 0, s, p, blp);
    return cudaGetLastError();
}

// Depthwise convolution: one thread-iteration produces eight channels of one output pixel,
// taps walked in (fh, fw) order with one FFMA each, so the result is independent of the tiling.
__global__ void __launch_bounds__(kPoolThreads)
dwconv_kernel(const __grid_constant__ DwConvParams p, BlpArgs blp) {
    pdl_enter();
    __shared__ int s_tile;
    const bool dynamic = blp.preempted != nullptr;
    if (threadIdx.x == 0) trace_begin(blp);
    const int C = p.out.C;
    const int C8 = C / 8;
    const int Ho = p.out.H, Wo = p.out.W;
    const int H = p.in.l.H, W = p.in.l.W;
    const unsigned total = (unsigned)p.out.N * Ho * Wo * C8;  // < 2^31, checked when the model is built
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
        const unsigned begin = (unsigned)tile * p.tile_elems;
        const unsigned end = begin + p.tile_elems < total ? begin + p.tile_elems : total;
        for (unsigned e = begin + threadIdx.x; e < end; e += kPoolThreads) {
            int c8 = (int)(e % C8);
            unsigned t = e / C8;
            int wo = (int)(t % Wo);
            t /= Wo;
            int ho = (int)(t % Ho);
            int n = (int)(t / Ho);
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int fh = 0; fh < p.k; ++fh) {
                int hi = ho * p.stride - p.pad + fh;
                if (hi < 0 || hi >= H) continue;
                for (int fw = 0; fw < p.k; ++fw) {
                    int wi = wo * p.stride - p.pad + fw;
                    if (wi < 0 || wi >= W) continue;
                    size_t off = (size_t)layout_row(p.in.l, n, hi, wi) * p.in.l.C + c8 * 8;
                    float x[8];
                    planes_load8(p.in.hi, p.in.lo, off, p.in.l.fmt, x);
                    const float4 *wv = reinterpret_cast<const float4 *>(p.w + (size_t)(fh * p.k + fw) * C + c8 * 8);
                    float4 w0 = wv[0], w1 = wv[1];
                    const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] = fmaf(x[j], wf[j], acc[j]);
                }
            }
            if (p.bias) {
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += p.bias[c8 * 8 + j];
            }
            apply_act_n(acc, p.act);
            planes_store8(p.out_hi, p.out_lo, (size_t)layout_row(p.out, n, ho, wo) * C + c8 * 8, p.out.fmt, acc);
        }
        ++iter;
        if (dynamic) __syncthreads();
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

cudaError_t dwconv_launch(const DwConvParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    launch_layer(dwconv_kernel, grid, kPoolThreads, 0, s, p, blp);
    return cudaGetLastError();
}

static bool pool_is_max3(const PoolParams &p) { return p.mode == 0 && p.k == 3 && !p.scale; }

int pool_grid(const PoolParams &p, int sm_count) {
    int per_sm = 8;
    if (pool_is_max3(p)) {
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pool_kernel<true>, kPoolThreads, 0);
        if (per_sm < 1) per_sm = 1;
    }
    long long grid = (long long)sm_count * per_sm;
    if (grid > p.total_tiles) grid = p.total_tiles;
    if (grid < 1) grid = 1;
    return (int)grid;
}

cudaError_t pool_launch(const PoolParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    if (pool_is_max3(p))
        launch_layer(pool_kernel<true>, grid, kPoolThreads, 0, s, p, blp);
    else
        launch_layer(pool_kernel<false>, grid, kPoolThreads, 0, s, p, blp);
    return cudaGetLastError();
}

}  // namespace gpx
