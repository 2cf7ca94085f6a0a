// Launch descriptors of the layer kernels.  One descriptor = one entry of the model's kernel
// list (KernelInfo in the reference, include/model.h:22-30).
#pragma once

#include "act_layout.h"
#include "blp.cuh"
#include "planes.cuh"

#include <cuda.h>
#include <cuda_runtime.h>

namespace gpx {

typedef unsigned short bf16_bits;

// A tensor as a layer kernel sees it: fp32 in canonical order (the graph input "data" is NCHW,
// "heads" is [N][C]) or two bf16 planes in one of the row orders of act_layout.h.
struct ActView {
    const float *f32;      // non-null: fp32 NCHW tensor (planes unused)
    const bf16_bits *hi;   // split planes
    const bf16_bits *lo;
    ActLayout l;
};

// ---- tensor-core convolution (cgemm_tcgen05.cu) ----------------------------------------------

// Finishing pass of a split-K convolution (splitk_finish_kernel, or the cluster reduction inside
// the convolution kernel): adds the per-split sums in split order, then bias, residual, activation.
struct SplitKParams {
    const float *partial;
    int k_splits, partial_rows, partial_ld;
    int m_rows, in_hs, in_ws, in_off;  // decode of a GEMM row, as in CgemmParams
    int relu;
    const float *bias;
    const bf16_bits *res_hi, *res_lo;
    ActLayout res;
    bf16_bits *out_hi, *out_lo;
    ActLayout out;
    float *out_f32;
    int cout_valid;
    int cout_padded;       // multiple of 8 covered by the partial sums
    int total_tiles;
    int tile_elems;        // (row, 8-channel group) pairs per tile
};

struct CgemmSlot {
    int next_iter;  // first iteration of this CTA's static schedule that is not complete
    int k_done;     // K blocks already accumulated for it (spill area valid if > 0)
    int grid;       // grid size the schedule was started with (0 = fresh)
    int pad;
};

struct CgemmParams {
    CUtensorMap a_hi, a_lo;  // activation planes [in.rows][Cin], box 128 rows x 64 channels
    CUtensorMap w_hi, w_lo;  // weight planes [Cout][taps*Cin], box BN rows x 64
    int taps;                // 1 or 9
    int cin;                 // input channels (multiple of 64)
    int cin_blocks;          // cin / 64
    int tap_shift[9];        // row shift of each tap
    int m_rows;              // GEMM rows to cover (stored rows of one input plane)
    int in_hs, in_ws;        // stored image dims of the input (decode of a GEMM row)
    int in_off;              // 1 when the input rows include a zero border, else 0
    int tiles_m, tiles_n;
    // Reciprocals of the divisors the epilogue decodes a tile and a row with (fast_div), and whether
    // GEMM row m is output row m (plain rows on both sides: no decode at all).
    float inv_k_splits, inv_tiles_n, inv_img, inv_in_ws;
    int identity_rows;
    int relu;
    const float *bias;       // [Cout] or null
    const bf16_bits *res_hi, *res_lo;  // residual planes or null
    ActLayout res;
    bf16_bits *out_hi, *out_lo;
    ActLayout out;
    float *out_f32;          // non-null: fp32 [pixel][cout_valid] output (graph heads) instead of planes
    int cout_valid;          // real output channels (the last column tile may be partly padding)
    int fmt;                 // PlaneFmt of operands, residual and output: PF_SPLIT issues three
                             // products per K step (hi*hi, hi*lo, lo*hi), the others one
    // Residual by tensor core (1x1 stride-1 convolutions on plain rows, no split K): res_kb = BN/64
    // extra K blocks per tile whose A operand is the residual tile and whose W operand is the
    // identity; res_hi/res_lo are then null and the epilogue adds nothing.
    CUtensorMap r_hi, r_lo, ident;
    int res_kb;
    int drop_on_stop;        // 1: a tile interrupted by the word is recomputed from K block 0 after the
                             // resume instead of being saved (no spill on the way out)
    int packed;              // 1 (two-plane operands, dual plan): hi*hi and hi*lo issued as one product of
                             // width 2*BN against the adjacent W_hi / W_lo tiles
    int dual;                // 1: two accumulators per tile in two TMEM buffers (short K ranges and
                             // single-plane operands), 0: four accumulators in one buffer
    int k_splits;            // >= 1: the K range is cut into this many tiles per output block
    int kb_per_split;        // K blocks per split (the last split may be shorter)
    float *partial;          // k_splits > 1: fp32 workspace [split][partial_rows][partial_ld]
    int partial_rows, partial_ld;
    // Cluster reduction (non-preemptible launches only): the k_splits CTAs of one output block form
    // a thread-block cluster, leave their partial tiles in shared memory and each finishes a share
    // of the rows, reading its peers' tiles through distributed shared memory in split order - the
    // additions of splitk_finish_kernel without the workspace round trip and the second launch.
    int cluster_reduce;
    SplitKParams fin;        // what the finishing pass needs (bias, residual, activation, output)
    CgemmSlot *slots;        // one per CTA of this kernel
    float *spill;            // [grid][128*BN] fp32, shared by the kernels of one executor
    int *error;              // {code, kernel*1000+cta}
};

cudaError_t cgemm_prepare(int device);
cudaError_t cgemm_launch(const CgemmParams &p, int bn, int grid, const BlpArgs &blp, cudaStream_t s);
int cgemm_max_cluster(int bn, int cluster);  // CTAs of clusters of this size that can be resident at once
size_t cgemm_spill_floats_per_cta();
int cgemm_threads();

// ---- CUDA-core convolution / dense (conv_simt.cu) --------------------------------------------

// out[M = N*Ho*Wo][Cout] = im2col(in)[M][K] * w[K][Cout], K = kh*kw*Cin ordered (kh, kw, ci),
// then + bias, + residual, ReLU.  Used where the tensor-core kernel does not apply: the stem
// (3 input channels, fp32 NCHW input), dense layers with a handful of rows, odd channel counts.
struct ConvParams {
    ActView in;
    const float *w;     // [K][Cout] fp32
    const float *bias;  // [Cout] or null
    ActView res;        // residual (hi == null && f32 == null: none)
    float *out_f32;     // fp32 [M][Cout] output (graph heads), or null
    bf16_bits *out_hi, *out_lo;
    ActLayout out;
    int Cin, Ho, Wo, Cout;
    int kh, kw, stride, pad;  // pad: vertical padding
    int pad_w;                // horizontal padding (one-sided filters pad one direction only)
    int M, K;
    int relu;
    int tiles_m, tiles_n;
};

struct PoolParams {
    ActView in;
    bf16_bits *out_hi, *out_lo;
    ActLayout out;
    int k, stride, pad;
    int mode;         // 0 = max, 1 = average over valid taps, 2 = copy of the tap (0,0) (subsample),
                      // 3 = average with the whole window as divisor (padding counts as zeros)
    int total_tiles;
    int tile_elems;   // output 8-channel vectors per tile
    // The output may be a channel slice of a wider tensor and the input a channel prefix of one:
    // `channels` are produced (out.C and in.l.C are only the row strides); of those the first
    // `in_valid` are read from the input, the rest are written as zeros.
    int channels;
    int in_valid;
    // Optional per-channel affine + activation applied to every input value as it is loaded
    // (a batch norm that precedes its consumer, as in DenseNet): x -> act(x * scale + shift).
    const float *scale, *shift;
    int act;
};

// Second half of a split-K tensor-core convolution: adds the per-split fp32 partial sums in
// split order, then bias, residual and ReLU, and stores the result like the one-pass epilogue.
#if defined(__CUDACC__)
// Tail of the finishing pass for eight channels (col0 .. col0+7) of output pixel (n_img, h, w):
// f holds the sum of the splits.  One definition for both places that finish a split-K tile, so
// they produce the same bits.
__device__ __forceinline__ void splitk_apply(const SplitKParams &p, int n_img, int h, int w, int col0, float (&f)[8]) {
    if (p.bias) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += p.bias[col0 + j];  // bias buffers are padded
    }
    if (p.res_hi) {
        size_t off = (size_t)layout_row(p.res, n_img, h, w) * p.res.C + col0;
        float r[8];
        planes_load8(p.res_hi, p.res_lo, off, p.res.fmt, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += r[j];
    }
    apply_act_n(f, p.relu);
    if (p.out_f32) {
        size_t off = ((size_t)(n_img * p.out.H + h) * p.out.W + w) * p.cout_valid;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (col0 + j < p.cout_valid) p.out_f32[off + col0 + j] = f[j];
        return;
    }
    planes_store8(p.out_hi, p.out_lo, (size_t)layout_row(p.out, n_img, h, w) * p.out.C + col0, p.out.fmt, f);
}
#endif
cudaError_t splitk_launch(const SplitKParams &p, int grid, const BlpArgs &blp, cudaStream_t s);

// Dense layer on at most eight rows (batch <= 8 classifiers: VGG's 25088 -> 4096 -> 4096 -> 1000,
// ResNet's 2048 -> 1000): a matrix-vector product streams the weights once and is bound by HBM,
// where a 128-row tensor-core tile would idle.  One warp per output column; every lane walks the K
// range in steps of 256 with eight elements per step, fp32 FMAs in a fixed order, a fixed shuffle
// tree adds the lanes: the result does not depend on the grid.
struct DenseRowsParams {
    const bf16_bits *a_hi, *a_lo;  // input rows, planes
    const bf16_bits *w_hi, *w_lo;  // weight planes [Cout][w_ld]
    const float *bias;
    bf16_bits *out_hi, *out_lo;    // output planes (row stride out_ld) or
    float *out_f32;                // fp32 [M][cout] (graph heads)
    int M, K, cout;
    int a_ld, w_ld, out_ld;
    int relu, fmt;
    int total_tiles;               // eight output columns per tile
};
cudaError_t dense_rows_launch(const DenseRowsParams &p, int grid, const BlpArgs &blp, cudaStream_t s);

// Patch matrix of a convolution whose input has too few channels for the tensor-core kernel
// (the stem): row m = output pixel, column k = (fh, fw, ci), zero-padded to a multiple of 64
// columns, written as hi/lo planes so a 1x1 tensor-core GEMM can consume it.
struct Im2colParams {
    ActView in;             // fp32 NCHW or split planes
    bf16_bits *out_hi, *out_lo;
    int Cin, Ho, Wo;
    int kh, kw, stride, pad;
    int K, Kp;              // real and padded row length
    int M;
    int fmt;                // PlaneFmt of the patch matrix
    int total_tiles;
    int tile_elems;         // 8-column vectors per tile
    // Row-window mode (fp32 NCHW input): a tile is `win_w` consecutive output pixels of one
    // output row; the input window they read is staged in shared memory with coalesced loads.
    int win_w;              // 0 = off
    int win_chunks;         // ceil(Wo / win_w)
    // Space-to-depth window mode: the output is [N][Ho][Wo][64]; channel j*16 + (dy*2+dx)*Cin + ci
    // of block (hb, wb) is input pixel (2*hb+dy-pad, 2*(wb+j)+dx-pad), j = 0..3, zero elsewhere;
    // kh, kw, stride, K are unused.
    int s2d;
    // Plane mode (the input is an activation in planes with a multiple of eight stored channels):
    // eight consecutive columns are eight channels of one tap, so a thread-iteration copies one
    // 16-byte vector per plane, or writes zeros where the tap falls outside the image.
    int planes_vec;
    int pad_w;              // horizontal padding (plane mode; `pad` is the vertical one)
};
constexpr int kIm2colWindowFloats = 4096;
cudaError_t im2col_launch(const Im2colParams &p, int grid, const BlpArgs &blp, cudaStream_t s);

// LayerNorm over the channels of a [rows][H] matrix (H <= 1024, multiple of 8).  With `ids` set
// the input row is the sum of the word, position and token-type embeddings instead of planes.
struct LayerNormParams {
    const bf16_bits *in_hi, *in_lo;
    const long long *ids;                   // [rows] token ids or null
    const float *word, *pos, *type;         // embedding tables (ids != null)
    const float *gamma, *beta;
    bf16_bits *out_hi, *out_lo;
    float *out_f32;                         // non-null: fp32 output (graph heads)
    int rows, H, S;
    int fmt;                                // PlaneFmt of the input and output planes
    float eps;
    int total_tiles;
};
cudaError_t layernorm_launch(const LayerNormParams &p, int grid, const BlpArgs &blp, cudaStream_t s);

// Multi-head self-attention over [B*S][ld] matrices of queries, keys and values (head h owns
// columns h*64 .. h*64+63); no mask.
struct AttnParams {
    const bf16_bits *q_hi, *q_lo, *k_hi, *k_lo, *v_hi, *v_lo;
    bf16_bits *out_hi, *out_lo;
    int B, S, heads, ld;
    int fmt;                // PlaneFmt of all four matrices
    float scale;
    int total_tiles;
    // Tensor-core path (single-plane formats, attention_tcgen05.cu): TMA maps of Q and K
    // ([B*S][ld], boxes of 128 rows x 64 columns) and of the transposed values
    // ([B*heads*64][S], boxes of 64 x 64), the transposed-value scratch and the error word.
    CUtensorMap tq, tk, tvt;
    bf16_bits *vt;
    int *error;
    // One slot per CTA (this executor's): next_iter holds, plus one, the tile the CTA gave up when
    // the word went up inside it; the relaunched CTA recomputes that tile before it claims new ones.
    CgemmSlot *slots;
};
cudaError_t attention_launch(const AttnParams &p, int grid, const BlpArgs &blp, cudaStream_t s);
cudaError_t attention_tc_prepare();
cudaError_t attention_tc_launch(const AttnParams &p, int grid, const BlpArgs &blp, cudaStream_t s);
cudaError_t transpose_v_launch(const AttnParams &p, int grid, const BlpArgs &blp, cudaStream_t s);

// Depthwise k x k convolution + bias + activation over split-plane activations; the filter is
// stored [kh*kw][C] so that eight channels of one tap are one 32-byte load.
struct DwConvParams {
    ActView in;
    const float *w;      // [k*k][C stored]
    const float *bias;   // [C] (zero-padded to the stored channel count)
    bf16_bits *out_hi, *out_lo;
    ActLayout out;
    int k, stride, pad, act;
    int total_tiles;
    int tile_elems;      // output 8-channel vectors per tile
};
cudaError_t dwconv_launch(const DwConvParams &p, int grid, const BlpArgs &blp, cudaStream_t s);

enum ConvTile { CONV_TILE_128 = 0, CONV_TILE_64 = 1, CONV_TILE_32 = 2 };

int conv_pick_tile(const ConvParams &p, int sm_count);
void conv_set_tiles(ConvParams &p, int tile);
int conv_grid(const ConvParams &p, int tile, int sm_count);
cudaError_t conv_launch(const ConvParams &p, int tile, int grid, const BlpArgs &blp, cudaStream_t s);
cudaError_t pool_launch(const PoolParams &p, int grid, const BlpArgs &blp, cudaStream_t s);
int pool_grid(const PoolParams &p, int sm_count);

}  // namespace gpx
