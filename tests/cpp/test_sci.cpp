// The reference's scientific smoke test (src/tests/test-sci.cpp:6-24) through the executor
// interface: initialise miniWeather, take the reductions, run one time step, print the relative
// change of mass and total energy - and, beyond the reference, preempt a BLPExecutor's time step,
// resume it and require the same state reductions as the uninterrupted run.
//
//   test_sci [workload]      (default miniweather)
#include "executor.h"  // found in include/gpx, as the reference's sources find theirs in include/

#include <cmath>
#include <cstdio>

int main(int argc, char **argv) {
    const std::string workload = argc > 1 ? argv[1] : "miniweather";
    foo::util::init_cuda();
    GPUstream stream;
    GPUStreamCreate(&stream, 0);

    foo::BaseExecutor base;
    CHECK_STATUS(base.init(workload));
    ASSERT(base.get_data_size("data") == 0);  // src/executor.cpp:87-97
    float dummy = 0.f;
    CHECK_STATUS(base.set_input("data", &dummy, sizeof(dummy), stream));  // accepted and ignored
    double mass0, te0, mass, te;
    CHECK_STATUS(base.get_model()->reductions(mass0, te0));
    CHECK_STATUS(base.execute(stream));
    GPUStreamSynchronize(stream);
    CHECK_STATUS(base.get_model()->reductions(mass, te));
    printf("d_mass: %le\n", (mass - mass0) / mass0);
    printf("d_te:   %le\n", (te - te0) / te0);
    ASSERT(std::fabs((mass - mass0) / mass0) < 1e-9);
    ASSERT(std::fabs((te - te0) / te0) < 1e-4);

    foo::BLPExecutor blp;
    CHECK_STATUS(blp.init(workload));
    GPUdeviceptr flag;
    ASSERT_CUDA_ERROR(GPUMallocManaged(&flag, 4, GPU_MEM_ATTACH_GLOBAL));
    *(volatile int *)flag = 0;
    blp.dpStop = flag;
    CHECK_STATUS(blp.execute(stream));
    blp.running = true;
    *(volatile int *)flag = 1;
    GPUStreamSynchronize(stream);  // drained
    int stops = 0;
    for (int round = 0; round < 64; ++round) {
        *(volatile int *)flag = 0;
        // resume reads the stop point itself (BLPExecutor::resume, src/executor.cpp:280-298)
        CHECK_STATUS(blp.resume(stream));
        if (blp.stop_index() < 0) break;  // nothing had been stopped: the time step is complete
        ++stops;
        if (round < 3) *(volatile int *)flag = 1;  // stop what was just relaunched, a few times
        GPUStreamSynchronize(stream);
    }
    GPUStreamSynchronize(stream);
    double bm, bt;
    CHECK_STATUS(blp.get_model()->reductions(bm, bt));
    printf("preempted and resumed %d time(s): mass %s, energy %s\n", stops, bm == mass ? "identical" : "DIFFERS",
           bt == te ? "identical" : "DIFFERS");
    if (bm != mass || bt != te) return 1;
    printf("PASS\n");
    base.clear();
    blp.clear();
    return 0;
}
