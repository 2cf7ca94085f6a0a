// Graph, storages and kernel list of one model instance: the native counterpart of
// foo::Model (include/model.h:32-93, src/model.cpp) in the reference.  The reference parses a
// TVM graph JSON and binds generated kernels from a cubin; here the graph is built in (or read
// from a graph JSON written by gpx_model_export_json) and every node maps to a hand-written
// kernel linked into the library.
#pragma once

#include "common.h"
#include "layers.cuh"

#include <string>
#include <unordered_map>
#include <vector>

namespace gpx {

// StorageInfo of the reference (include/model.h:13-18) plus layout knowledge.
struct Storage {
    enum Kind {
        ActCanonical,  // device layout == canonical layout (graph input NCHW, 2-D outputs)
        ActNHWC,       // device NHWC, canonical NCHW
        Weight,        // device [kh][kw][Cin][Cout], canonical OIHW
        Vec            // bias and other 1-D parameters
    };
    std::string name;
    std::string stype = "float32";
    Kind kind = ActCanonical;
    int rank = 0;
    int64_t dims[4] = {0, 0, 0, 0};  // canonical dims
    size_t bytes = 0;
    float *dptr = nullptr;
    bool is_param = false;
    int fan_in = 0;  // for the seeded initialiser
};

enum class Op { Input, Conv, MaxPool, AvgPool };

struct Node {
    std::string name;
    Op op = Op::Input;
    std::vector<int> inputs;  // node ids: data input, then residual if any
    int storage = -1;         // output storage index
    int weight = -1, bias = -1;
    int N = 0, H = 0, W = 0, C = 0;  // output shape (logical NHWC)
    int k = 0, stride = 1, pad = 0;
    bool relu = false;
    int residual = -1;  // node id
};

struct Kernel {
    std::string name;
    int node = -1;
    bool is_conv = true;
    ConvParams conv{};
    PoolParams pool{};
    int tile = 0;
    int grid = 1;
    int total_tiles = 0;
    double flops = 0, bytes = 0;  // algorithmic work of the layer
};

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

    int add_storage(const gpx::Storage &s);
    int find(const std::string &name) const;
};

namespace gpx {

int build_builtin_graph(gpx_model &m, const std::string &name, const gpx_model_opts &opts);
int finalize_model(gpx_model &m);  // allocate storages, derive the kernel list
void normal_fill(float *dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std);
void uniform_fill(float *dst, size_t n, uint64_t seed, uint64_t stream, float lo, float hi);

}  // namespace gpx
