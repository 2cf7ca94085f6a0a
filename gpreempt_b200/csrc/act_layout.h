// Storage layout of an activation tensor in HBM.
//
// Activations between layers are kept as two bf16 planes (hi, lo) with x ~= hi + lo: 16 bits of
// mantissa, which is what the tensor-core convolution consumes directly (three bf16 products
// hi*hi + hi*lo + lo*hi stand in for one fp32 product).  Each plane is a row-major matrix
// [rows][C]: one row per stored pixel, channels contiguous, so every convolution is a GEMM over
// rows and a filter tap is a constant row shift.  Three row orders exist:
//   plain            row = (n*H + h)*W + w
//   padded           one zero pixel around every image: row = (n*(H+2) + h+1)*(W+2) + w+1
//                    (input of a 3x3 stride-1 convolution: a tap (fh,fw) is the row shift
//                    (fh-1)*(W+2) + (fw-1), and the zero border supplies the padding)
//   phased           the padded image split into its four (row parity, column parity) planes,
//                    plane-major (input of a 3x3 stride-2 convolution: tap (fh,fw) reads plane
//                    (fh&1, fw&1) shifted by (fh>>1, fw>>1), again a constant row shift)
// Border rows are zeroed once at allocation and never written.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define GPX_HD __host__ __device__ __forceinline__
#else
#define GPX_HD inline
#endif

namespace gpx {

enum ActOrder : int { ACT_PLAIN = 0, ACT_PADDED = 1, ACT_PHASED = 2 };

// Element format of the planes: two bf16 planes hi + lo (float32 models), or one plane of bf16
// or fp16 (the reduced-precision models).
enum PlaneFmt : int { PF_SPLIT = 0, PF_BF16 = 1, PF_F16 = 2 };

struct ActLayout {
    int N, H, W, C;  // logical shape
    int order;       // ActOrder
    int Hs, Ws;      // stored rows / columns per image (per phase plane when phased)
    int plane;       // rows of one phase plane (N*Hs*Ws); equals rows when not phased
    int rows;        // stored rows in total
    int fmt;         // PlaneFmt of the planes that hold the tensor
};

inline ActLayout make_layout(int N, int H, int W, int C, int order) {
    ActLayout l;
    l.N = N;
    l.H = H;
    l.W = W;
    l.C = C;
    l.order = order;
    l.fmt = PF_SPLIT;
    if (order == ACT_PLAIN) {
        l.Hs = H;
        l.Ws = W;
    } else if (order == ACT_PADDED) {
        l.Hs = H + 2;
        l.Ws = W + 2;
    } else {
        l.Hs = (H + 2) / 2;
        l.Ws = (W + 2) / 2;
    }
    l.plane = N * l.Hs * l.Ws;
    l.rows = order == ACT_PHASED ? 4 * l.plane : l.plane;
    return l;
}

// Stored row of logical pixel (n, h, w).
GPX_HD int layout_row(const ActLayout &l, int n, int h, int w) {
    if (l.order == ACT_PLAIN) return (n * l.Hs + h) * l.Ws + w;
    if (l.order == ACT_PADDED) return (n * l.Hs + h + 1) * l.Ws + w + 1;
    int hp = h + 1, wp = w + 1;
    int ph = ((hp & 1) << 1) | (wp & 1);
    return ph * l.plane + (n * l.Hs + (hp >> 1)) * l.Ws + (wp >> 1);
}

// Activation fused into a layer's epilogue.
enum ActKind : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_RELU6 = 3 };

#if defined(__CUDACC__)
__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == ACT_RELU) return fmaxf(v, 0.f);
    if (act == ACT_GELU) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));  // exact GELU
    if (act == ACT_RELU6) return fminf(fmaxf(v, 0.f), 6.f);
    return v;
}

// The same over a register array, with the (warp-uniform) choice made once outside the element
// loop: inside it the compiler would otherwise evaluate the erf of GELU for every element of every
// layer and select afterwards.
template <int N>
__device__ __forceinline__ void apply_act_n(float (&f)[N], int act) {
    if (act == ACT_RELU) {
#pragma unroll
        for (int j = 0; j < N; ++j) f[j] = fmaxf(f[j], 0.f);
    } else if (act == ACT_RELU6) {
#pragma unroll
        for (int j = 0; j < N; ++j) f[j] = fminf(fmaxf(f[j], 0.f), 6.f);
    } else if (act == ACT_GELU) {
#pragma unroll
        for (int j = 0; j < N; ++j) f[j] = 0.5f * f[j] * (1.0f + erff(f[j] * 0.70710678118654752440f));
    }
}
#endif

}  // namespace gpx
