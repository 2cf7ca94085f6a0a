// C entry points over the reference's own graph-analytics translation unit
// (src/workloads/graphcompute.cu, compiled unmodified next to this file into
// oracle/_ref/libgraphcompute_ref.so).  TEST INFRASTRUCTURE ONLY: the GPU parity test loads it to
// compare this repository's kernels and CPU oracle with what the reference computes.
//
// The reference keeps its result arrays in private members and has no call that returns them;
// this file reads them by seeing the class declarations with `private` and `protected` spelt `public` (the
// standard and CUDA headers are included before that, so only the reference's header is affected).
#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <chrono>
#include <cstddef>
#include <cstring>
#include <string>
#include <sys/syscall.h>
#include <glog/logging.h>

#define private public
#define protected public
#include "workloads/graphcompute.h"
#undef protected
#undef private

namespace {
GraphComputeRaw::GraphCompute *g_graph = nullptr;
int g_algo = -1;  // 0 bfs, 1 sssp, 2 cc, 3 pagerank
}  // namespace

extern "C" {

int gcref_close() {
    delete g_graph;
    g_graph = nullptr;
    g_algo = -1;
    return 0;
}

// Executor::init for a graph workload (src/executor.cpp:24-34) with the dataset prefix given whole.
int gcref_open(int device, const char *algo, const char *prefix) {
    if (cudaSetDevice(device) != cudaSuccess) return 1;
    if (cudaFree(nullptr) != cudaSuccess) return 1;  // the driver-API calls of the reference need the primary context
    gcref_close();
    const std::string a(algo), p(prefix);
    try {
        if (a == "bfs") {
            g_graph = new GraphComputeRaw::bfs::BFS(p);
            g_algo = 0;
        } else if (a == "sssp") {
            g_graph = new GraphComputeRaw::sssp::SSSP(p);
            g_algo = 1;
        } else if (a == "cc") {
            g_graph = new GraphComputeRaw::cc::CC(p);
            g_algo = 2;
        } else if (a == "pagerank") {
            g_graph = new GraphComputeRaw::pagerank::PageRank(p);
            g_algo = 3;
        } else {
            return 3;
        }
    } catch (...) {
        return 4;
    }
    return cudaDeviceSynchronize() == cudaSuccess ? 0 : 2;
}

unsigned long long gcref_vertices() { return g_graph ? g_graph->vertex_count : 0; }

// Executor::execute (src/executor.cpp:129), n times on the default stream; `compute` synchronises
// the stream every iteration itself.  Returns the host time of the n runs in milliseconds, < 0 on
// error.
double gcref_compute(int n) {
    if (!g_graph) return -1.0;
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < n; ++i) g_graph->compute(nullptr);
    if (cudaDeviceSynchronize() != cudaSuccess) return -2.0;
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
}

// The result of the latest run: bfs uint32 label, sssp uint32 cost, cc uint64 comp, pagerank float
// value; `bytes` must be the size of that array.
int gcref_result(void *out, size_t bytes) {
    if (!g_graph) return 1;
    const size_t n = g_graph->vertex_count;
    const void *src = nullptr;
    size_t need = 0;
    if (g_algo == 0) {
        src = static_cast<GraphComputeRaw::bfs::BFS *>(g_graph)->label_d;
        need = n * sizeof(uint32_t);
    } else if (g_algo == 1) {
        src = static_cast<GraphComputeRaw::sssp::SSSP *>(g_graph)->costList_d;
        need = n * sizeof(uint32_t);
    } else if (g_algo == 2) {
        src = static_cast<GraphComputeRaw::cc::CC *>(g_graph)->comp_d;
        need = n * sizeof(unsigned long long);
    } else {
        src = static_cast<GraphComputeRaw::pagerank::PageRank *>(g_graph)->value_d;
        need = n * sizeof(float);
    }
    if (bytes != need) return 2;
    return cudaMemcpy(out, src, need, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 3;
}

}  // extern "C"
