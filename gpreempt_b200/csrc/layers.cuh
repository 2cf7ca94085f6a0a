// Launch descriptors of the layer kernels.  One descriptor = one entry of the model's kernel
// list (KernelInfo in the reference, include/model.h:22-30).
#pragma once

#include "blp.cuh"
#include <cuda_runtime.h>

namespace gpx {

// Convolution / dense layer as an implicit GEMM: out[M = N*Ho*Wo][Cout] = im2col(in)[M][K] *
// w[K][Cout], K = kh*kw*Cin ordered (kh, kw, ci), followed by + bias, + residual, ReLU.
struct ConvParams {
    const float *in;    // NHWC, or NCHW when in_nchw (the graph input "data")
    const float *w;     // [K][Cout]
    const float *bias;  // [Cout] or null
    const float *res;   // NHWC residual with the output's shape, or null
    float *out;         // NHWC
    int N, H, W, Cin;
    int Ho, Wo, Cout;
    int kh, kw, stride, pad;
    int M, K;
    int relu;
    int in_nchw;
    int tiles_m, tiles_n;
};

struct PoolParams {
    const float *in;  // NHWC
    float *out;       // NHWC
    int N, H, W, C;
    int Ho, Wo;
    int k, stride, pad;
    int mode;         // 0 = max, 1 = average over valid taps (global average uses k = H)
    int total_tiles;
    int tile_elems;   // output float4 vectors per tile
};

// Tile shapes the SIMT convolution is instantiated for.
enum ConvTile { CONV_TILE_128 = 0, CONV_TILE_64 = 1, CONV_TILE_32 = 2 };

int conv_pick_tile(const ConvParams &p, int sm_count);
void conv_set_tiles(ConvParams &p, int tile);
int conv_grid(const ConvParams &p, int tile, int sm_count, bool preemptible);
cudaError_t conv_launch(const ConvParams &p, int tile, int grid, const BlpArgs &blp,
                        cudaStream_t s);
cudaError_t pool_launch(const PoolParams &p, int grid, const BlpArgs &blp, cudaStream_t s);
int pool_grid(const PoolParams &p, int sm_count);

}  // namespace gpx
