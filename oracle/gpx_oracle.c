/*
 * CPU oracle for libgpx — TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the product (gpreempt_b200/, include/) may call, link or import this file; it is
 * used by tests/, by the smoke check and by the CPU-baseline leg of the benchmark as the
 * checker and the reported CPU figure.
 *
 * PARITY UNPINNED: the reference (thustorage/GPreempt) executes TVM-generated kernels that
 * are not part of its tree (model/ is git-ignored, .gitignore:2-3) and stores no expected
 * outputs anywhere (src/tests/test-dnn.cpp:38-41 only prints ten floats).  The arithmetic
 * lives in apache/tvm pinned at 513c2be0c3b853 (README.md:69-72), which is absent here.  This
 * file therefore restates the published layer definitions (direct convolution, pooling, GEMM)
 * in the reference's tensor conventions — NCHW activations, OIHW filters, fp32 storage
 * (scripts/compile/compile.py:27-31,66) — with fp64 accumulation, and is cross-checked in the
 * CPU test-suite against PyTorch's CPU operators on the same inputs.
 *
 * Build: make -C oracle   (gcc -O3 -fopenmp -shared)
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* y[i] = fma(a, x[i], y[i]) — the best-effort kernel of the preemption microbenchmark.
 * A single correctly-rounded fused multiply-add per element, so the GPU result must match
 * bit for bit. */
void orc_axpy_f32(float a, const float *x, float *y, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) y[i] = fmaf(a, x[i], y[i]);
}

/* Fused conv2d + bias + residual + ReLU, the unit TVM fuses into one kernel for the
 * reference (kernel names "fused_nn_conv2d_add_nn_relu", patch/tvm.patch:303-306).
 * in  [N][Cin][H][W], w [Cout][Cin][kh][kw], bias [Cout] or NULL, res [N][Cout][Ho][Wo] or
 * NULL, out [N][Cout][Ho][Wo].  Each output is accumulated in fp64 over (ci, fh, fw) in
 * increasing order and rounded to fp32 once. */
void orc_conv2d_nchw_hw(const float *in, const float *w, const float *bias, const float *res,
                        float *out, int N, int Cin, int H, int W, int Cout, int kh, int kw,
                        int stride, int pad_h, int pad_w, int relu);

void orc_conv2d_nchw(const float *in, const float *w, const float *bias, const float *res,
                     float *out, int N, int Cin, int H, int W, int Cout, int kh, int kw,
                     int stride, int pad, int relu) {
    orc_conv2d_nchw_hw(in, w, bias, res, out, N, Cin, H, W, Cout, kh, kw, stride, pad, pad, relu);
}

/* The same with separate vertical and horizontal padding (the 1x7 / 7x1 / 1x3 / 3x1 factorised
 * convolutions of Inception-v3 pad one direction only). */
void orc_conv2d_nchw_hw(const float *in, const float *w, const float *bias, const float *res,
                        float *out, int N, int Cin, int H, int W, int Cout, int kh, int kw,
                        int stride, int pad_h, int pad_w, int relu) {
    const int Ho = (H + 2 * pad_h - kh) / stride + 1;
    const int Wo = (W + 2 * pad_w - kw) / stride + 1;
#pragma omp parallel
    {
        double *acc = (double *)malloc(sizeof(double) * (size_t)Ho * Wo);
#pragma omp for collapse(2) schedule(dynamic, 1)
        for (int n = 0; n < N; ++n) {
            for (int co = 0; co < Cout; ++co) {
                for (int i = 0; i < Ho * Wo; ++i) acc[i] = 0.0;
                for (int ci = 0; ci < Cin; ++ci) {
                    const float *plane = in + ((size_t)n * Cin + ci) * H * W;
                    for (int fh = 0; fh < kh; ++fh) {
                        for (int fw = 0; fw < kw; ++fw) {
                            const double wv = w[(((size_t)co * Cin + ci) * kh + fh) * kw + fw];
                            /* valid output range for this tap */
                            int ho_lo = 0, wo_lo = 0;
                            while (ho_lo < Ho && ho_lo * stride - pad_h + fh < 0) ++ho_lo;
                            while (wo_lo < Wo && wo_lo * stride - pad_w + fw < 0) ++wo_lo;
                            int ho_hi = Ho, wo_hi = Wo;
                            while (ho_hi > ho_lo && (ho_hi - 1) * stride - pad_h + fh >= H) --ho_hi;
                            while (wo_hi > wo_lo && (wo_hi - 1) * stride - pad_w + fw >= W) --wo_hi;
                            for (int ho = ho_lo; ho < ho_hi; ++ho) {
                                const float *row = plane + (size_t)(ho * stride - pad_h + fh) * W;
                                double *arow = acc + (size_t)ho * Wo;
                                for (int wo = wo_lo; wo < wo_hi; ++wo)
                                    arow[wo] += wv * (double)row[wo * stride - pad_w + fw];
                            }
                        }
                    }
                }
                float *o = out + ((size_t)n * Cout + co) * Ho * Wo;
                const float *r = res ? res + ((size_t)n * Cout + co) * Ho * Wo : NULL;
                const double b = bias ? (double)bias[co] : 0.0;
                for (int i = 0; i < Ho * Wo; ++i) {
                    double v = acc[i] + b;
                    if (r) v += (double)r[i];
                    if (relu && v < 0.0) v = 0.0;
                    if (relu == 3 && v > 6.0) v = 6.0; /* ReLU6 */
                    o[i] = (float)v;
                }
            }
        }
        free(acc);
    }
}

/* Same layer with fp32 accumulation: the timed CPU baseline (no parity claim). */
void orc_conv2d_nchw_fast(const float *in, const float *w, const float *bias, const float *res,
                          float *out, int N, int Cin, int H, int W, int Cout, int kh, int kw,
                          int stride, int pad, int relu) {
    const int Ho = (H + 2 * pad - kh) / stride + 1;
    const int Wo = (W + 2 * pad - kw) / stride + 1;
#pragma omp parallel
    {
        float *acc = (float *)malloc(sizeof(float) * (size_t)Ho * Wo);
#pragma omp for collapse(2) schedule(dynamic, 1)
        for (int n = 0; n < N; ++n) {
            for (int co = 0; co < Cout; ++co) {
                const float b = bias ? bias[co] : 0.0f;
                for (int i = 0; i < Ho * Wo; ++i) acc[i] = b;
                for (int ci = 0; ci < Cin; ++ci) {
                    const float *plane = in + ((size_t)n * Cin + ci) * H * W;
                    for (int fh = 0; fh < kh; ++fh) {
                        for (int fw = 0; fw < kw; ++fw) {
                            const float wv = w[(((size_t)co * Cin + ci) * kh + fh) * kw + fw];
                            int ho_lo = 0, wo_lo = 0;
                            while (ho_lo < Ho && ho_lo * stride - pad + fh < 0) ++ho_lo;
                            while (wo_lo < Wo && wo_lo * stride - pad + fw < 0) ++wo_lo;
                            int ho_hi = Ho, wo_hi = Wo;
                            while (ho_hi > ho_lo && (ho_hi - 1) * stride - pad + fh >= H) --ho_hi;
                            while (wo_hi > wo_lo && (wo_hi - 1) * stride - pad + fw >= W) --wo_hi;
                            for (int ho = ho_lo; ho < ho_hi; ++ho) {
                                const float *row = plane + (size_t)(ho * stride - pad + fh) * W;
                                float *arow = acc + (size_t)ho * Wo;
                                if (stride == 1) {
                                    const float *src = row - pad + fw;
                                    for (int wo = wo_lo; wo < wo_hi; ++wo) arow[wo] += wv * src[wo];
                                } else {
                                    for (int wo = wo_lo; wo < wo_hi; ++wo)
                                        arow[wo] += wv * row[wo * stride - pad + fw];
                                }
                            }
                        }
                    }
                }
                float *o = out + ((size_t)n * Cout + co) * Ho * Wo;
                const float *r = res ? res + ((size_t)n * Cout + co) * Ho * Wo : NULL;
                for (int i = 0; i < Ho * Wo; ++i) {
                    float v = acc[i];
                    if (r) v += r[i];
                    if (relu && v < 0.0f) v = 0.0f;
                    if (relu == 3 && v > 6.0f) v = 6.0f;
                    o[i] = v;
                }
            }
        }
        free(acc);
    }
}

/* Depthwise convolution (groups == channels) + bias + activation (0 none, 1 ReLU, 3 ReLU6), the
 * building block of MobileNetV2.  in [N][C][H][W], w [C][1][kh][kw]; fp64 accumulation. */
void orc_dwconv2d_nchw(const float *in, const float *w, const float *bias, float *out, int N, int C,
                       int H, int W, int kh, int kw, int stride, int pad, int relu) {
    const int Ho = (H + 2 * pad - kh) / stride + 1;
    const int Wo = (W + 2 * pad - kw) / stride + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int c = 0; c < C; ++c) {
            const float *plane = in + ((size_t)n * C + c) * H * W;
            const float *f = w + (size_t)c * kh * kw;
            float *o = out + ((size_t)n * C + c) * Ho * Wo;
            for (int ho = 0; ho < Ho; ++ho) {
                for (int wo = 0; wo < Wo; ++wo) {
                    double acc = 0.0;
                    for (int fh = 0; fh < kh; ++fh) {
                        int hi = ho * stride - pad + fh;
                        if (hi < 0 || hi >= H) continue;
                        for (int fw = 0; fw < kw; ++fw) {
                            int wi = wo * stride - pad + fw;
                            if (wi < 0 || wi >= W) continue;
                            acc += (double)f[fh * kw + fw] * (double)plane[(size_t)hi * W + wi];
                        }
                    }
                    if (bias) acc += (double)bias[c];
                    if (relu && acc < 0.0) acc = 0.0;
                    if (relu == 3 && acc > 6.0) acc = 6.0;
                    o[(size_t)ho * Wo + wo] = (float)acc;
                }
            }
        }
    }
}

/* max (mode 0) / average over the valid taps (mode 1) / average with the whole window as divisor,
 * padding counted as zeros (mode 2, the default of torch.nn.functional.avg_pool2d) pooling, NCHW. */
void orc_pool2d_nchw(const float *in, float *out, int N, int C, int H, int W, int k, int stride,
                     int pad, int mode) {
    const int Ho = (H + 2 * pad - k) / stride + 1;
    const int Wo = (W + 2 * pad - k) / stride + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int c = 0; c < C; ++c) {
            const float *plane = in + ((size_t)n * C + c) * H * W;
            float *o = out + ((size_t)n * C + c) * Ho * Wo;
            for (int ho = 0; ho < Ho; ++ho) {
                for (int wo = 0; wo < Wo; ++wo) {
                    double acc = mode == 0 ? -INFINITY : 0.0;
                    int cnt = 0;
                    for (int fh = 0; fh < k; ++fh) {
                        int hi = ho * stride - pad + fh;
                        if (hi < 0 || hi >= H) continue;
                        for (int fw = 0; fw < k; ++fw) {
                            int wi = wo * stride - pad + fw;
                            if (wi < 0 || wi >= W) continue;
                            double v = plane[(size_t)hi * W + wi];
                            if (mode == 0)
                                acc = v > acc ? v : acc;
                            else
                                acc += v;
                            ++cnt;
                        }
                    }
                    if (mode == 1) acc /= (double)cnt;
                    if (mode == 2) acc /= (double)(k * k);
                    o[(size_t)ho * Wo + wo] = (float)acc;
                }
            }
        }
    }
}

/* ---- bf16 GEMM of the preemption microbenchmark ---------------------------------------- */

static inline float bf16_to_f32(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even fp32 -> bf16 */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

void orc_f32_to_bf16(const float *src, uint16_t *dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = f32_to_bf16(src[i]);
}
void orc_bf16_to_f32(const uint16_t *src, float *dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}

/* C[M][N] = A[M][K] * B[N][K]^T, bf16 inputs, fp64 accumulation; the exact (unrounded) sums
 * are returned as doubles so the caller chooses the output rounding and tolerance. */
void orc_gemm_bf16_nt(const uint16_t *A, const uint16_t *B, double *C, int M, int N, int K) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < M; ++i) {
        for (int j = 0; j < N; ++j) {
            const uint16_t *a = A + (size_t)i * K;
            const uint16_t *b = B + (size_t)j * K;
            double acc = 0.0;
            for (int k = 0; k < K; ++k) acc += (double)bf16_to_f32(a[k]) * (double)bf16_to_f32(b[k]);
            C[(size_t)i * N + j] = acc;
        }
    }
}

/* The same for a list of (row, col) samples of a large product. */
void orc_gemm_bf16_nt_samples(const uint16_t *A, const uint16_t *B, const int *rows,
                              const int *cols, int nsamples, double *out, int K) {
#pragma omp parallel for schedule(static)
    for (int s = 0; s < nsamples; ++s) {
        const uint16_t *a = A + (size_t)rows[s] * K;
        const uint16_t *b = B + (size_t)cols[s] * K;
        double acc = 0.0;
        for (int k = 0; k < K; ++k) acc += (double)bf16_to_f32(a[k]) * (double)bf16_to_f32(b[k]);
        out[s] = acc;
    }
}

/* fp32-accumulate blocked GEMM for the timed CPU baseline of the microbenchmark. */
void orc_gemm_bf16_nt_fast(const uint16_t *A, const uint16_t *B, float *C, int M, int N, int K) {
    float *Af = (float *)malloc(sizeof(float) * (size_t)M * K);
    float *Bf = (float *)malloc(sizeof(float) * (size_t)N * K);
    orc_bf16_to_f32(A, Af, (size_t)M * K);
    orc_bf16_to_f32(B, Bf, (size_t)N * K);
#pragma omp parallel for collapse(2) schedule(static)
    for (int i0 = 0; i0 < M; i0 += 4) {
        for (int j0 = 0; j0 < N; j0 += 4) {
            float acc[4][4] = {{0}};
            for (int k = 0; k < K; ++k)
                for (int i = 0; i < 4 && i0 + i < M; ++i)
                    for (int j = 0; j < 4 && j0 + j < N; ++j)
                        acc[i][j] += Af[(size_t)(i0 + i) * K + k] * Bf[(size_t)(j0 + j) * K + k];
            for (int i = 0; i < 4 && i0 + i < M; ++i)
                for (int j = 0; j < 4 && j0 + j < N; ++j) C[(size_t)(i0 + i) * N + j0 + j] = acc[i][j];
        }
    }
    free(Af);
    free(Bf);
}
