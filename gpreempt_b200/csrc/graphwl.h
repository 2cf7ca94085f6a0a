// Graph-analytics best-effort workloads of the reference: breadth-first search, single-source
// shortest paths, connected components and PageRank on a graph held whole in GPU memory
// (src/workloads/graphcompute.cu, the block-level-preemptible variant graphcompute.tr.cu; the task
// config config/Z.json runs them under a latency-critical DNN).  The graph comes from files in the
// EMOGI "bel" layout the reference reads (read_graph, graphcompute.cu:15-45): <prefix>.col holds the
// row offsets, <prefix>.dst the neighbour ids, <prefix>.val the edge weights of sssp.
//
// The reference drives each algorithm from the host: one or two kernels per iteration, then a copy
// of a `changed` byte and a stream synchronisation, until nothing changed.  Here one `execute` is a
// fixed kernel list - an initialisation kernel and one group of kernels per iteration - and
// convergence is tracked on the device: iteration i runs only if iteration i-1 raised its flag, the
// kernels of the iterations behind the last live one return at once.  The length of the list is
// found when the model is opened, by running the algorithm once.  For that to be exact the
// iterations are race-free: every kernel reads values only an earlier kernel wrote (the reference's
// kernels read distances and component ids other warps are lowering in the same launch, so its
// iteration count depends on timing; the fixed points are the same).  Connected components use
// hooking with shortcuts instead of the reference's plain label propagation, for the same fixed
// point in a handful of iterations.
#pragma once

#include <cuda_runtime.h>
#include <string>

#include "blp.cuh"

struct gpx_model;
struct gpx_model_opts;

namespace gpx {

enum GraphAlgo { GW_BFS = 0, GW_SSSP = 1, GW_CC = 2, GW_PAGERANK = 3 };
enum GraphPhase {
    GW_INIT = 0,    // start of a request: result arrays, frontier and iteration flags
    GW_EDGES = 1,   // walks the edge lists of a tile of vertices (a warp takes one list at a time)
    GW_VERTICES = 2 // per-vertex pass after the edge pass (sssp: update; cc: shortcut)
};

constexpr int kGwThreads = 256;
constexpr int kGwEdgeTileVertsMax = 256;  // vertices per tile of an edge pass at most (32 per warp)
constexpr int kGwVertexTileVerts = 1024;  // vertices per tile of a per-vertex pass
constexpr int kGwMaxIters = 16384;        // iteration flags a graph workload has: no run may need more rounds
constexpr unsigned kGwInfinity = 0xFFFFFFFFu;  // MYINFINITY, include/workloads/graphcompute.h:14

struct GraphWlParams {
    int algo;
    int phase;
    int iter;             // iteration index; the BFS level
    int tile_verts;       // edge passes: vertices per tile, a multiple of 8 (one warp takes an eighth of them in turn)
    unsigned n;           // vertices
    unsigned src;         // bfs, sssp: source vertex (0, graphcompute.cu:181,344)
    const unsigned long long *row;  // [n + 1] edge offsets (pagerank: of the in-edge lists)
    const unsigned *adj;            // neighbour ids (pagerank: in-neighbours)
    const unsigned *wgt;            // sssp: edge weights
    const unsigned *outdeg;         // pagerank: out-degree of every vertex
    unsigned *a;          // bfs: label; sssp: cost; cc: comp; pagerank: value (float)
    unsigned *b;          // sssp: new cost; cc: offered ids; pagerank: residual (float)
    unsigned *d0, *d1;    // pagerank: delta, read from d<iter & 1>, written to the other
    unsigned char *f0;    // sssp: label (the frontier)
    int *active;          // [kGwMaxIters + 1]: active[i] != 0 <=> iteration i has work
    float alpha, tol;     // pagerank (0.85, 0.001: include/workloads/graphcompute.h:85-86)
};

cudaError_t graphwl_launch(const GraphWlParams &p, int grid, const BlpArgs &blp, cudaStream_t s);
int graphwl_grid(const GraphWlParams &p, int total_tiles, int sm_count);

// "bfs:<prefix>", "sssp:<prefix>", "cc:<prefix>", "pagerank:<prefix>".
bool is_graph_workload(const std::string &name);
int build_graph_workload(gpx_model &m, const std::string &name, const gpx_model_opts &opts);

}  // namespace gpx
