// Element formats of activation / weight planes and the eight-channel load and store every
// memory-bound layer kernel uses.
//
// float32 models keep x as two bf16 planes (hi, lo), x ~= hi + lo.  The reduced-precision models
// (the fp16 / bf16 configurations layered on the reference's fp32-only graphs,
// scripts/compile/compile.py:27-31,66) keep one 16-bit plane: the lo pointer is null and the
// tensor-core kernel issues one product instead of three.  Arithmetic between loads and stores
// is fp32 in every format.
#pragma once

#include "act_layout.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace gpx {

typedef unsigned short plane_bits;

#if defined(__CUDACC__)

__device__ __forceinline__ plane_bits pf_bf16_bits(float f) {
    unsigned u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (plane_bits)((u >> 16) | 0x40);  // quiet NaN
    u += 0x7fffu + ((u >> 16) & 1u);  // round to nearest even
    return (plane_bits)(u >> 16);
}

// Two consecutive channels packed in one 32-bit word (low half = even channel).
__device__ __forceinline__ float2 pf_unpack2(unsigned w, int fmt) {
    if (fmt == PF_F16) {
        __half2 h = *reinterpret_cast<__half2 *>(&w);
        return __half22float2(h);
    }
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

__device__ __forceinline__ unsigned pf_pack2(float a, float b, int fmt) {
    if (fmt == PF_F16) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<unsigned *>(&h);
    }
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);  // one cvt.rn.bf16x2.f32
    return *reinterpret_cast<unsigned *>(&v);
}

__device__ __forceinline__ void planes_load8(const plane_bits *hi, const plane_bits *lo, size_t off, int fmt,
                                             float (&x)[8]) {
    const uint4 a = *reinterpret_cast<const uint4 *>(hi + off);
    const unsigned ah[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        float2 v = pf_unpack2(ah[q], fmt);
        x[2 * q] = v.x;
        x[2 * q + 1] = v.y;
    }
    if (fmt == PF_SPLIT) {
        const uint4 b = *reinterpret_cast<const uint4 *>(lo + off);
        const unsigned bl[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            x[2 * q] += __uint_as_float(bl[q] << 16);
            x[2 * q + 1] += __uint_as_float(bl[q] & 0xffff0000u);
        }
    }
}

// The two halves of planes_load8: raw 16-byte vectors first, so that a caller can have many
// loads in flight before it converts any of them.
__device__ __forceinline__ void planes_fetch8(const plane_bits *hi, const plane_bits *lo, size_t off, int fmt,
                                              uint4 &a, uint4 &b) {
    a = *reinterpret_cast<const uint4 *>(hi + off);
    if (fmt == PF_SPLIT) b = *reinterpret_cast<const uint4 *>(lo + off);
}
__device__ __forceinline__ void planes_decode8(const uint4 &a, const uint4 &b, int fmt, float (&x)[8]) {
    const unsigned ah[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        float2 v = pf_unpack2(ah[q], fmt);
        x[2 * q] = v.x;
        x[2 * q + 1] = v.y;
    }
    if (fmt == PF_SPLIT) {
        const unsigned bl[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            x[2 * q] += __uint_as_float(bl[q] << 16);
            x[2 * q + 1] += __uint_as_float(bl[q] & 0xffff0000u);
        }
    }
}

__device__ __forceinline__ void planes_store8(plane_bits *hi, plane_bits *lo, size_t off, int fmt,
                                              const float (&x)[8]) {
    unsigned h4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) h4[q] = pf_pack2(x[2 * q], x[2 * q + 1], fmt);
    *reinterpret_cast<uint4 *>(hi + off) = make_uint4(h4[0], h4[1], h4[2], h4[3]);
    if (fmt == PF_SPLIT) {
        unsigned l4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            l4[q] = pf_pack2(x[2 * q] - __uint_as_float(h4[q] << 16),
                             x[2 * q + 1] - __uint_as_float(h4[q] & 0xffff0000u), PF_SPLIT);
        *reinterpret_cast<uint4 *>(lo + off) = make_uint4(l4[0], l4[1], l4[2], l4[3]);
    }
}

// One channel (the CUDA-core convolution path).
__device__ __forceinline__ float planes_load1(const plane_bits *hi, const plane_bits *lo, size_t off, int fmt) {
    if (fmt == PF_F16) return __half2float(*reinterpret_cast<const __half *>(hi + off));
    float v = __uint_as_float((unsigned)hi[off] << 16);
    if (fmt == PF_SPLIT) v += __uint_as_float((unsigned)lo[off] << 16);
    return v;
}

__device__ __forceinline__ void planes_store1(plane_bits *hi, plane_bits *lo, size_t off, int fmt, float v) {
    if (fmt == PF_F16) {
        *reinterpret_cast<__half *>(hi + off) = __float2half_rn(v);
        return;
    }
    plane_bits h = pf_bf16_bits(v);
    hi[off] = h;
    if (fmt == PF_SPLIT) lo[off] = pf_bf16_bits(v - __uint_as_float((unsigned)h << 16));
}

#endif  // __CUDACC__

}  // namespace gpx
