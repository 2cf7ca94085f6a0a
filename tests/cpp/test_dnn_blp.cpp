// Execute, raise the flag, drain, clear, resume: the sequence of the reference's manual test
// (src/tests/test-dnn-blp.cpp:13-52) written against the reference's class names through the
// include/gpx shim, with the comparison the reference leaves to the eye done here: the resumed
// output must equal an uninterrupted BaseExecutor run bit for bit.
//
//   test_dnn_blp <model> [batch] [delay_us] [out.bin]
#include "executor.h"  // found in include/gpx, as the reference's sources find theirs in include/

#include <chrono>
#include <cstdio>
#include <cstring>
#include <vector>

int main(int argc, char **argv) {
    if (argc < 2) {
        printf("Usage: %s <model> [batch] [delay_us] [out.bin]\n", argv[0]);
        return 1;
    }
    const std::string model_name = argv[1];
    const int batch = argc > 2 ? atoi(argv[2]) : 1;
    const int delay_us = argc > 3 ? atoi(argv[3]) : 0;
    foo::util::init_cuda();
    GPUstream stream;
    GPUStreamCreate(&stream, 0);

    std::vector<float> want;
    size_t input_size = 0, output_size = 0;
    std::vector<float> input;
    {
        foo::BaseExecutor base;
        base.set_options(batch);
        CHECK_STATUS(base.init(model_name));
        input_size = base.get_data_size("data");
        output_size = base.get_data_size("heads");
        input.assign(input_size / sizeof(float), 10.0f);  // the reference's all-10.0 input
        CHECK_STATUS(base.set_input("data", input.data(), input_size, stream));
        CHECK_STATUS(base.execute(stream));
        GPUStreamSynchronize(stream);
        want.resize(output_size / sizeof(float));
        CHECK_STATUS(base.get_output("heads", want, stream));
        GPUStreamSynchronize(stream);
        base.clear();
    }

    foo::BLPExecutor executor;
    executor.set_options(batch);
    GPUdeviceptr p1;
    CHECK_STATUS(executor.init(model_name));
    ASSERT_CUDA_ERROR(GPUMallocManaged(&p1, 4, GPU_MEM_ATTACH_GLOBAL));
    *(volatile int *)p1 = 0;
    executor.dpStop = p1;
    ASSERT(executor.get_data_size("data") == input_size);
    ASSERT(executor.get_data_size("nosuch") == 0);
    CHECK_STATUS(executor.set_input("data", input.data(), input_size, stream));
    GPUStreamSynchronize(stream);
    auto t0 = std::chrono::high_resolution_clock::now();
    CHECK_STATUS(executor.execute(stream));
    executor.running = true;
    if (delay_us > 0) usleep(delay_us);
    *(volatile int *)p1 = 1;
    GPUStreamSynchronize(stream);
    *(volatile int *)p1 = 0;
    int resumes = 0;
    for (;;) {
        CHECK_STATUS(executor.resume(stream));
        GPUStreamSynchronize(stream);
        if (executor.stop_index() == -1) break;
        ++resumes;
        ASSERT(resumes < 4);
    }
    auto t1 = std::chrono::high_resolution_clock::now();
    std::vector<float> output(output_size / sizeof(float));
    CHECK_STATUS(executor.get_output("heads", output, stream));
    GPUStreamSynchronize(stream);
    printf("Time: %ldus\n", (long)std::chrono::duration_cast<std::chrono::microseconds>(t1 - t0).count());
    printf("Resumed: %d\n", resumes);
    for (size_t i = 0; i < 10 && i < output.size(); i++) printf("%f\n", output[i]);
    if (argc > 4) {
        FILE *fp = fopen(argv[4], "wb");
        ASSERT(fp != nullptr);
        fwrite(output.data(), sizeof(float), output.size(), fp);
        fclose(fp);
    }
    const bool same = memcmp(output.data(), want.data(), output_size) == 0;
    printf("%s\n", same ? "PASS resumed output is bit-identical" : "FAIL resumed output differs");
    executor.clear();
    GPUMemFreeHost((void *)(uintptr_t)p1);
    GPUStreamDestroy(stream);
    return same ? 0 : 2;
}
