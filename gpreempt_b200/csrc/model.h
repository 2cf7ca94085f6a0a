// Graph, storages and kernel list of one model instance: the native counterpart of
// foo::Model (include/model.h:32-93, src/model.cpp) in the reference.  The reference parses a
// TVM graph JSON and binds generated kernels from a cubin; here the graph is built in and every
// node maps to hand-written kernels linked into the library.
#pragma once

#include "common.h"
#include "layers.cuh"
#include "stencil.h"
#include "graphwl.h"

#include <string>
#include <unordered_map>
#include <vector>

namespace gpx {

// StorageInfo of the reference (include/model.h:13-18) plus layout knowledge.
struct Storage {
    enum Kind {
        InputF32,  // graph input, fp32 NCHW on the device as given by the client
        OutputF32, // graph output, fp32 [N][C]
        ActSplit,  // intermediate activation: hi/lo bf16 planes in the row order of `layout`
        InputI64,  // graph input of token ids, int64 [N][S]
        Table,     // fp32 parameter matrix used as is (embedding tables)
        Weight,    // canonical OIHW fp32; device copies: fp32 [kh][kw][Cin][Cout] and, for the
                   // tensor-core kernel, hi/lo bf16 planes [Cout][kh*kw*Cin]
        Vec        // bias
    };
    std::string name;
    std::string stype = "float32";
    Kind kind = InputF32;
    int rank = 0;
    int64_t dims[4] = {0, 0, 0, 0};  // canonical dims (NCHW / OIHW / [N][C] / [C])
    size_t bytes = 0;                // canonical size in bytes (what get/set move)
    float *dptr = nullptr;           // fp32 device buffer (InputF32, OutputF32, Weight, Vec)
    bf16_bits *hi = nullptr;         // split planes (ActSplit: activation; Weight: tensor-core copy)
    bf16_bits *lo = nullptr;
    size_t plane_elems = 0;
    ActLayout layout{};              // ActSplit only
    bool is_param = false;
    bool hidden = false;             // internal scratch tensor, not listed
    bool wants_split = false;        // Weight: a tensor-core kernel consumes it
    int split_k = 0;                 // Weight: row length of the split planes (K padded to 64)
    int fan_in = 0;
    int cs = 0;                      // ActSplit: stored channels (logical channels padded to 64), 0 = dims[1]
    int cin_pad = 0, cout_pad = 0;   // Weight: padded channel counts of the tensor-core planes
    bool depthwise = false;          // Weight: [C][1][kh][kw] filter of a depthwise convolution
    bool s2d = false;                // Weight: tensor-core planes in the space-to-depth order of the stem
    float init_mean = 0.f, init_std = 0.f;  // seeded initialiser; std 0 = He-normal / 0.01 default
    bool token_major = false;        // activations of sequence models: canonical [N][S][C]
    int parent = -1;                 // ActSplit: this tensor is a channel slice of that storage
    int ch_off = 0;                  //   starting at this stored channel (concatenation by placement)
};

// Buffer: a tensor other nodes write slices of (the running concatenation of a dense block).
// Affine: per-channel scale + shift + activation of the first in_c channels of its input.
enum class Op { Input, Conv, MaxPool, AvgPool, LayerNorm, Attention, DwConv, Buffer, Affine };

struct Node {
    std::string name;
    Op op = Op::Input;
    std::vector<int> inputs;
    int storage = -1;
    int weight = -1, bias = -1;
    int N = 0, H = 0, W = 0, C = 0;  // output shape
    int k = 0, stride = 1, pad = 0;
    int kw = 0;      // filter width when it differs from the height `k` (0 = square)
    int pad_w = -1;  // horizontal padding when it differs from the vertical `pad` (-1 = same)
    bool count_pad = false;  // average pooling that divides by the whole window (padding counts as zeros)
    int act = 0;  // ActKind applied after bias and residual
    int residual = -1;
    bool tensor_core = false;  // decided by finalize_model
    int sub_storage = -1;      // stride-2 1x1: compact copy of the sub-sampled input;
                               // few-channel input: patch matrix
    bool via_im2col = false;
    bool via_s2d = false;      // 7x7 stride-2 stem on few channels: space-to-depth window tensor + four-tap GEMM
    int tables[3] = {-1, -1, -1};  // LayerNorm fed by embeddings: word, position, token-type tables
    int heads = 0;                 // Attention
    int Cs = 0;                    // stored output channels (C padded to 64 when the model pads)
    int in_c = 0;                  // channels of the input that are read (0 = all): a prefix of a Buffer
    int scale = -1, shift = -1;    // Affine, or a pooling node that normalises its input: Vec storages
};

enum class KernelType { ConvSimt, Cgemm, Pool, Im2col, SplitK, LayerNorm, Attention, DwConv, AttentionTc, TransposeV, Stencil, DenseRows, GraphWl };

struct Kernel {
    std::string name;
    int node = -1;
    KernelType type = KernelType::ConvSimt;
    ConvParams conv{};
    PoolParams pool{};
    CgemmParams cgemm{};
    Im2colParams im2col{};
    SplitKParams splitk{};
    LayerNormParams ln{};
    AttnParams attn{};
    DwConvParams dw{};
    StencilParams stencil{};
    DenseRowsParams dense{};
    GraphWlParams graphwl{};
    int tile = 0;  // ConvSimt: ConvTile; Cgemm: BN
    bool fused_into_prev = false;  // SplitK: a non-preemptible executor's convolution kernel finishes the tile itself
    int grid = 1;
    int threads = 256;
    int total_tiles = 0;
    double flops = 0, bytes = 0;
};

int make_tmap_2d_bf16(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols,
                      uint32_t box_rows, uint32_t box_cols);

}  // namespace gpx

struct gpx_model {
    std::string name;
    int batch = 1;
    int device = 0;
    int sm_count = 0;
    std::vector<gpx::Storage> storages;
    std::unordered_map<std::string, size_t> storage_idx;
    std::vector<gpx::Node> nodes;
    std::vector<gpx::Kernel> kernels;
    int head_node = -1;
    int max_cgemm_grid = 0;
    size_t max_partial_floats = 0;  // split-K workspace an executor must provide
    bool pad_channels = false;      // store activations with channels padded to a multiple of 64
    std::vector<void *> scratch;         // device buffers owned by the model besides the storages
    gpx::bf16_bits *identity = nullptr;  // 128 x 128 identity matrix in the plane format
    int fmt = 0;                    // PlaneFmt of activations and tensor-core weights (dtype option)
    // miniWeather (stencil.h): no graph nodes, no "data"/"heads"; one execute is one time step.
    bool sci = false;
    int sci_nx = 0, sci_nz = 0;
    float sci_dt = 0.f, sci_dx = 0.f, sci_dz = 0.f;
    std::vector<float> sci_hy_dens_cell, sci_hy_dens_theta_cell;  // host copies for the reductions
    std::vector<float> sci_initial;                               // initial state, to start over
    // Graph analytics (graphwl.h): `sci` is set as well (no graph nodes, no "data"/"heads"); one
    // execute is one run of the algorithm to its fixed point.
    int graph_algo = -1;
    uint64_t graph_vertices = 0, graph_edges = 0;
    int graph_iterations = 0;     // live iterations of the run that sized the kernel list
    int *graph_active = nullptr;  // device: iteration flags (owned through `scratch`)

    int add_storage(const gpx::Storage &s);
    int find(const std::string &name) const;
};

namespace gpx {

int build_builtin_graph(gpx_model &m, const std::string &name, const gpx_model_opts &opts);
// Model directories (artifacts.cu): mod.json + host.json (+ mod.params).
bool model_dir_exists(const std::string &dir);
int build_graph_from_dir(gpx_model &m, const std::string &dir, const gpx_model_opts &opts);
int check_host_json(const gpx_model &m, const std::string &dir);
int finalize_model(gpx_model &m);
void normal_fill(float *dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std);
void uniform_fill(float *dst, size_t n, uint64_t seed, uint64_t stream, float lo, float hi);

}  // namespace gpx
