// The reference's graph-analytics smoke tests (src/tests/test-graph.cpp:7-47 and
// src/tests/test-graph-blp.cpp) through the executor interface: load the dataset, run the algorithm
// twice and print the time of the second run - and, beyond the reference, write the result to a
// file, then preempt a BLPExecutor's run, resume it and require the same result bytes.
//
//   test_graph <cc|bfs|pagerank|sssp> <prefix of the .col/.dst/.val files> <result file>
#include "executor.h"  // found in include/gpx, as the reference's sources find theirs in include/

#include <chrono>
#include <cstdio>
#include <cstring>
#include <vector>

static const char *result_name(const std::string &algo) {
    if (algo == "bfs") return "label";
    if (algo == "sssp") return "cost";
    if (algo == "cc") return "comp";
    return "value";
}

static Status fetch(foo::Executor &ex, const std::string &algo, std::vector<char> &out, GPUstream stream) {
    size_t idx;
    Status st = ex.get_model()->find_storage_idx(result_name(algo), idx);
    if (st != Status::Succ) return st;
    out.resize(ex.get_model()->get_storage_size(idx));
    st = ex.get_model()->get(idx, out.data(), out.size(), stream);
    GPUStreamSynchronize(stream);
    return st;
}

int main(int argc, char **argv) {
    if (argc < 4) {
        printf("usage: test_graph <cc|bfs|pagerank|sssp> <prefix> <result file>\n");
        return 2;
    }
    const std::string algo = argv[1], prefix = argv[2];
    foo::util::init_cuda();
    GPUstream stream;
    GPUStreamCreate(&stream, 0);

    foo::BaseExecutor base;
    CHECK_STATUS(base.set_graph_path(prefix));
    auto t2 = std::chrono::high_resolution_clock::now();
    CHECK_STATUS(base.init(algo));
    auto t3 = std::chrono::high_resolution_clock::now();
    CHECK_STATUS(base.execute(stream));
    GPUStreamSynchronize(stream);
    auto t4 = std::chrono::high_resolution_clock::now();
    CHECK_STATUS(base.execute(stream));
    GPUStreamSynchronize(stream);
    auto t5 = std::chrono::high_resolution_clock::now();
    printf("%s Init: %ldus\n", algo.c_str(), (long)std::chrono::duration_cast<std::chrono::microseconds>(t3 - t2).count());
    printf("%s Compute: %ldus\n", algo.c_str(), (long)std::chrono::duration_cast<std::chrono::microseconds>(t5 - t4).count());
    (void)t4;
    ASSERT(base.get_data_size("data") == 0);  // src/executor.cpp:87-97
    std::vector<char> want, got;
    CHECK_STATUS(fetch(base, algo, want, stream));
    FILE *fp = fopen(argv[3], "wb");
    ASSERT(fp && fwrite(want.data(), 1, want.size(), fp) == want.size());
    fclose(fp);

    foo::BLPExecutor blp;
    CHECK_STATUS(blp.set_graph_path(prefix));
    CHECK_STATUS(blp.init(algo));
    GPUdeviceptr flag;
    ASSERT_CUDA_ERROR(GPUMallocManaged(&flag, 4, GPU_MEM_ATTACH_GLOBAL));
    *(volatile int *)flag = 0;
    blp.dpStop = flag;
    CHECK_STATUS(blp.execute(stream));
    blp.running = true;
    *(volatile int *)flag = 1;
    GPUStreamSynchronize(stream);  // drained
    int stops = 0;
    for (int round = 0; round < 256; ++round) {
        *(volatile int *)flag = 0;
        CHECK_STATUS(blp.resume(stream));  // BLPExecutor::resume, src/executor.cpp:280-298
        if (blp.stop_index() < 0) break;   // nothing had been stopped: the run is complete
        ++stops;
        if (round < 4) *(volatile int *)flag = 1;  // stop what was just relaunched, a few times
        GPUStreamSynchronize(stream);
    }
    GPUStreamSynchronize(stream);
    CHECK_STATUS(fetch(blp, algo, got, stream));
    const bool same = got.size() == want.size() && memcmp(got.data(), want.data(), want.size()) == 0;
    printf("preempted and resumed %d time(s): result %s\n", stops, same ? "identical" : "DIFFERS");
    if (!same) return 1;
    printf("PASS\n");
    base.clear();
    blp.clear();
    return 0;
}
