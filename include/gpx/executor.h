// foo::Executor, foo::BaseExecutor and foo::BLPExecutor with the reference's public interface
// (include/executor.h:14-84, src/executor.cpp:18-342) over the libgpx C ABI.  Header-only, so a
// client source of the reference compiles against it and links libgpx.so.
//
// Differences a port has to know:
//  * `init(workload)` opens a graph the library knows by that name (the reference's aliases
//    "vgg", "resnet152", "densenet", "bert", "inception" included) or, when MODEL_PATH/<workload>
//    holds a mod.json, that directory; parameters come from MODEL_PATH/<workload>/mod.params if
//    it exists, else from the seeded generator (set_seed).  MODEL_PATH is read from the macro of
//    that name, if defined, or from the environment.
//  * batch size, storage format and sequence length are options (set_options) because the
//    reference compiles one graph per shape.
//  * a failed call returns its Status; nothing here terminates the process.
#pragma once

#include <atomic>
#include <cstdlib>
#include <memory>
#include <string>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

#include "model.h"

namespace foo {

class Executor {
public:
    // Executor::set_graph_path, src/executor.cpp:18-21: the dataset of the graph-analytics
    // workloads ("cc", "bfs", "pagerank", "sssp"), called before init as the clients do
    // (src/cuda-clients/blpclient.cpp:115-117).  A relative path is taken under the directory named by
    // the environment variable GPX_GRAPH_BASE_PATH (GRAPH_BASE_PATH in the reference).
    Status set_graph_path(const std::string &path) {
        graph_path = path;
        return Status::Succ;
    }

    void set_options(int batch, const std::string &dtype = "", int seq_len = 0) {
        batch_ = batch;
        dtype_ = dtype;
        seq_len_ = seq_len;
    }
    void set_seed(uint64_t seed) { seed_ = seed; }

    // Executor::load_model / load_param, src/executor.cpp:110-117.
    virtual Status load_model(std::string model_path) {
        model = std::make_shared<Model>();
        model->set_options(batch_, dtype_, seq_len_);
        return model->load_model(model_path);
    }
    virtual Status load_param(std::string model_path) {
        return model->load_param((model_path + "/mod.params").c_str());
    }

    // Executor::init, src/executor.cpp:23-45.
    virtual Status init(std::string workload) { return init_kind(workload, GPX_EXEC_BASE); }

    // Executor::execute, src/executor.cpp:119-134.
    virtual Status execute(GPUstream stream) { return (Status)gpx_exec_execute(exec_, stream); }

    // Executor::launch_kernel, src/executor.cpp:136-164.
    virtual Status launch_kernel(size_t kernel_offset, GPUstream stream = 0) {
        return (Status)gpx_exec_launch_kernel(exec_, kernel_offset, stream);
    }

    // src/executor.cpp:47-85.
    virtual Status set_input(const std::string &key, void *value, size_t len, GPUstream stream) {
        // the scientific workload has no request data: Succ, as src/executor.cpp:47-60
        if (model && model->is_scientific()) return Status::Succ;
        size_t idx;
        if (model->find_storage_idx(key, idx) != Status::Succ) return Status::NotFound;
        return model->set(idx, value, len, stream);
    }
    virtual Status set_input(const std::string &key, std::vector<float> &value, GPUstream stream) {
        return set_input(key, value.data(), value.size() * sizeof(float), stream);
    }
    virtual Status get_output(const std::string &key, void *value, size_t len, GPUstream stream) {
        if (model && model->is_scientific()) return Status::Succ;  // src/executor.cpp:64-80
        size_t idx;
        if (model->find_storage_idx(key, idx) != Status::Succ) return Status::NotFound;
        return model->get(idx, value, len, stream);
    }
    virtual Status get_output(const std::string &key, std::vector<float> &value, GPUstream stream) {
        return get_output(key, value.data(), value.size() * sizeof(float), stream);
    }
    // src/executor.cpp:87-97: 0 for a name the model does not have.
    virtual size_t get_data_size(const std::string &key) {
        size_t idx;
        if (!model || model->find_storage_idx(key, idx) != Status::Succ) return 0;
        return model->get_storage_size(idx);
    }

    // Executor::clear, src/executor.cpp:99-108.
    virtual void clear() {
        if (exec_) gpx_exec_destroy(exec_);
        exec_ = nullptr;
        if (model) model->clear();
    }
    size_t get_kernel_num() const { return model ? model->get_kernel_num() : 0; }
    // Executor::capture_graph, src/executor.cpp:176-196.
    virtual void capture_graph(GPUstream stream) {
        if (gpx_exec_capture_graph(exec_, stream) == GPX_SUCC) use_cuda_graph = true;
    }
    virtual ~Executor() {
        if (exec_) gpx_exec_destroy(exec_);
    }

    gpx_exec *handle() const { return exec_; }
    std::shared_ptr<Model> get_model() const { return model; }

protected:
    static std::string model_root() {
#ifdef MODEL_PATH
        return MODEL_PATH;
#else
        const char *e = std::getenv("MODEL_PATH");
        return e ? e : "";
#endif
    }
    static bool exists(const std::string &path) {
        struct stat st;
        return ::stat(path.c_str(), &st) == 0;
    }

    Status init_kind(const std::string &workload, int kind) {
        if (workload == "cc" || workload == "bfs" || workload == "pagerank" || workload == "sssp") {
            // src/executor.cpp:24-34
            type = "graph";
            Status st = load_model(workload + ":" + graph_path);
            if (st != Status::Succ) return st;
            return (Status)gpx_exec_create(model->handle(), kind, &exec_);
        }
        type = "dnn";
        const std::string root = model_root();
        const std::string dir = root.empty() ? "" : root + "/" + workload;
        const bool from_dir = !dir.empty() && exists(dir + "/mod.json");
        Status st = load_model(from_dir ? dir : workload);
        if (st != Status::Succ) return st;
        if (!dir.empty() && exists(dir + "/mod.params"))
            st = load_param(dir);
        else
            st = model->init_random(seed_);
        if (st != Status::Succ) return st;
        return (Status)gpx_exec_create(model->handle(), kind, &exec_);
    }

    std::shared_ptr<Model> model;
    std::string type;
    bool use_cuda_graph = false;
    std::string graph_path;
    gpx_exec *exec_ = nullptr;
    int batch_ = 1, seq_len_ = 0;
    std::string dtype_;
    uint64_t seed_ = 1;
};

class BaseExecutor : public Executor {
public:
    BaseExecutor() {}
    virtual ~BaseExecutor() {}
};

class BLPExecutor : public Executor {
public:
    BLPExecutor() : dpStop(0), running(false) {}
    virtual ~BLPExecutor() {}

    // BLPExecutor::init, src/executor.cpp:300-342: the stop index and the per-kernel tile cursors
    // are the executor's; the preempt flag `dpStop` is the caller's and may be set afterwards.
    virtual Status init(std::string workload) override {
        stopIndex = -1;
        return init_kind(workload, GPX_EXEC_BLP);
    }

    // BLPExecutor::execute, src/executor.cpp:211-232: zeroes the cursors, then launches everything.
    virtual Status execute(GPUstream stream) override {
        Status st = bind_word();
        if (st != Status::Succ) return st;
        return (Status)gpx_exec_execute(exec_, stream);
    }
    virtual Status launch_kernel(size_t kernel_offset, GPUstream stream = 0) override {
        Status st = bind_word();
        if (st != Status::Succ) return st;
        return (Status)gpx_exec_launch_kernel(exec_, kernel_offset, stream);
    }
    virtual void capture_graph(GPUstream stream) override {
        if (bind_word() != Status::Succ) return;
        Executor::capture_graph(stream);
    }

    // BLPExecutor::getStopPoint, src/executor.cpp:269-278: waits for the stream, reads the index of
    // the first kernel that stopped early (-1: none) and re-arms it.
    Status getStopPoint(GPUstream stream) { return (Status)gpx_exec_stop_point(exec_, stream, &stopIndex); }

    // BLPExecutor::resume, src/executor.cpp:280-298: nothing to do unless `running` was set by the
    // caller after execute; otherwise relaunches kernels stop..N-1 with their saved cursors.
    Status resume(GPUstream stream) {
        if (!running) return Status::Succ;
        Status st = bind_word();
        if (st != Status::Succ) return st;
        return (Status)gpx_exec_resume(exec_, stream, &stopIndex);
    }
    int stop_index() const { return stopIndex; }

    void set_lc_be_tasks(std::atomic<int> &lc_tasks, std::atomic<int> &be_tasks) {
        this->lc_tasks = &lc_tasks;
        this->be_tasks = &be_tasks;
    }

public:
    GPUdeviceptr dpStop;  // allocated by the user to share among all clients (include/executor.h:75)
    std::atomic<bool> running;

private:
    Status bind_word() {
        if (dpStop == bound_) return Status::Succ;
        if (dpStop == 0) return Status::Fail;
        int st = gpx_exec_set_word_dptr(exec_, (const void *)(uintptr_t)dpStop);
        if (st == GPX_SUCC) bound_ = dpStop;
        return (Status)st;
    }
    GPUdeviceptr bound_ = 0;
    int stopIndex = -1;
    std::atomic<int> *lc_tasks = nullptr;
    std::atomic<int> *be_tasks = nullptr;
};

}  // namespace foo
