// foo::Model with the reference's public interface (include/model.h:13-93) over the libgpx C ABI.
// Header-only.  Where the reference parses TVM artefacts and binds kernels of a cubin, this class
// opens a graph the library knows (or a directory holding mod.json) and the kernels are the
// library's own.
#pragma once

#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "util/common.h"
#include "util/gpu_util.h"

namespace foo {

using namespace foo::util;

// include/model.h:13-18.
class StorageInfo {
public:
    std::string name;
    size_t size;
    std::string stype;
};

// include/model.h:21-30 (no function handle or argument arrays: kernels are linked into the
// library); tiles, flops and bytes are what gpx_model_kernel_info adds.
class KernelInfo {
public:
    std::string name;
    uint32_t launch_params[6];  // gridDims & blockDims
    int total_tiles = 0;
    double flops = 0, bytes = 0;
};

class Model {
public:
    Model() {}
    // The reference's three paths (mod.json, host.json, mod.cubin) name one directory; the model
    // is opened from `device_json`'s directory when that holds a mod.json, else by graph name.
    Model(const std::string &device_json, const std::string &host_json, const std::string &cuda_module) {
        load_model(device_json, host_json, cuda_module);
    }
    ~Model() { clear(); }
    Model(const Model &) = delete;
    Model &operator=(const Model &) = delete;

    // Options the reference has no place for (its graphs are compiled for one shape).
    void set_options(int batch, const std::string &dtype = "", int seq_len = 0) {
        batch_ = batch;
        dtype_ = dtype;
        seq_len_ = seq_len;
    }

    // Model::load_model, src/model.cpp:79-125.
    Status load_model(const std::string &device_json, const std::string & /*host_json*/ = "",
                      const std::string & /*cuda_module*/ = "") {
        clear();
        std::string name = device_json;
        const std::string tail = "/mod.json";
        if (name.size() > tail.size() && name.compare(name.size() - tail.size(), tail.size(), tail) == 0)
            name.erase(name.size() - tail.size());
        gpx_model_opts o{};
        o.batch = batch_;
        o.dtype = dtype_.empty() ? nullptr : dtype_.c_str();
        o.seq_len = seq_len_;
        int st = gpx_model_open(name.c_str(), &o, &m_);
        if (st != GPX_SUCC) return (Status)st;
        return refresh();
    }

    // Model::load_param, src/model.cpp:263-282.
    Status load_param(const char *param_file_path) { return (Status)gpx_model_load_params(m_, param_file_path); }
    // Seeded synthetic parameters (no trained weights travel with this library).
    Status init_random(uint64_t seed) { return (Status)gpx_model_init_random(m_, seed); }

    bool is_loaded() { return m_ != nullptr; }
    size_t get_kernel_num() const { return kernel_infos.size(); }
    size_t get_storage_num() const { return storage_infos.size(); }
    size_t get_storage_size(size_t idx) { return storage_infos[idx].size; }
    StorageInfo &get_storage_info(size_t idx) { return storage_infos[idx]; }
    KernelInfo &get_kernel_info(size_t idx) { return kernel_infos[idx]; }

    // Model::get / Model::set, src/model.cpp:288-321 (`len < size` is rejected).
    Status get(size_t idx, void *out, size_t len, GPUstream stream) {
        if (idx >= storage_infos.size()) return Status::OutOfRange;
        return get(storage_infos[idx].name, out, len, stream);
    }
    Status get(const std::string &key, void *out, size_t len, GPUstream stream) {
        return (Status)gpx_model_get(m_, key.c_str(), out, len, stream);
    }
    Status set(size_t idx, void *value, size_t len, GPUstream stream) {
        if (idx >= storage_infos.size()) return Status::OutOfRange;
        return set(storage_infos[idx].name, value, len, stream);
    }
    Status set(const std::string &key, void *value, size_t len, GPUstream stream) {
        return (Status)gpx_model_set(m_, key.c_str(), value, len, stream);
    }

    // src/model.cpp:69-77.
    static size_t get_stype_size(std::string &stype) {
        if (stype == "float32" || stype == "int32") return 4;
        if (stype == "int64") return 8;
        if (stype == "uint1" || stype == "byte" || stype == "int8" || stype == "uint8") return 1;
        if (stype == "float16" || stype == "bfloat16") return 2;
        return 0;
    }

    // Model::find_storage_idx, src/model.cpp:347-356.
    Status find_storage_idx(const std::string &name, size_t &idx) {
        return (Status)gpx_model_find(m_, name.c_str(), &idx);
    }

    // Model::clear, src/model.cpp:238-260.
    Status clear() {
        if (m_) gpx_model_close(m_);
        m_ = nullptr;
        storage_infos.clear();
        kernel_infos.clear();
        return Status::Succ;
    }

    // "miniweather" (the reference's sciCompute workload, src/executor.cpp:14): a simulation state
    // instead of "data" / "heads".
    // The graph-analytics workloads (graphCompute, src/executor.cpp:13) have none either.
    bool is_scientific() {
        size_t idx;
        if (!m_ || gpx_model_find(m_, "data", &idx) == GPX_SUCC) return false;
        return gpx_model_find(m_, "state", &idx) == GPX_SUCC || is_graph();
    }
    bool is_graph() { return m_ && gpx_model_graph_info(m_, nullptr, nullptr, nullptr, nullptr, nullptr) == GPX_SUCC; }
    // reductions(mass, te), src/workloads/miniweather.cu:650-677.
    Status reductions(double &mass, double &te) { return (Status)gpx_model_reductions(m_, &mass, &te); }

    gpx_model *handle() const { return m_; }

private:
    Status refresh() {
        size_t n = 0;
        gpx_model_storage_num(m_, &n);
        storage_infos.resize(n);
        for (size_t i = 0; i < n; ++i) {
            char name[256], stype[32];
            size_t bytes = 0;
            int is_param = 0;
            int st = gpx_model_storage_info(m_, i, name, sizeof(name), &bytes, stype, sizeof(stype), &is_param);
            if (st != GPX_SUCC) return (Status)st;
            storage_infos[i].name = name;
            storage_infos[i].size = bytes;
            storage_infos[i].stype = stype;
        }
        gpx_model_kernel_num(m_, &n);
        kernel_infos.resize(n);
        for (size_t i = 0; i < n; ++i) {
            char name[256];
            KernelInfo &k = kernel_infos[i];
            int st = gpx_model_kernel_info(m_, i, name, sizeof(name), k.launch_params, &k.total_tiles, &k.flops, &k.bytes);
            if (st != GPX_SUCC) return (Status)st;
            k.name = name;
        }
        return Status::Succ;
    }

    gpx_model *m_ = nullptr;
    int batch_ = 1, seq_len_ = 0;
    std::string dtype_;
    std::vector<StorageInfo> storage_infos;
    std::vector<KernelInfo> kernel_infos;
};

typedef std::unordered_map<std::string, std::vector<float>> ModelParam;

// ModelParamParser::parse_from_file, src/model.cpp:15-55: "TVM_MODEL_PARAMS\0", u64 count, then
// per tensor a NUL-terminated name, u64 n and n floats.  Returns nullptr on a malformed file.
class ModelParamParser {
public:
    static ModelParam *parse_from_file(const char *param_file) {
        FILE *fp = std::fopen(param_file, "rb");
        if (!fp) return nullptr;
        ModelParam *params = new ModelParam();
        bool ok = false;
        do {
            char magic[17];
            if (std::fread(magic, 1, 17, fp) != 17 || std::memcmp(magic, "TVM_MODEL_PARAMS", 17) != 0) break;
            uint64_t count = 0;
            if (std::fread(&count, 8, 1, fp) != 1 || count == 0) break;
            uint64_t i = 0;
            for (; i < count; ++i) {
                std::string key;
                int c;
                while ((c = std::fgetc(fp)) != EOF && c != 0) key.push_back((char)c);
                uint64_t n = 0;
                if (c == EOF || std::fread(&n, 8, 1, fp) != 1 || n == 0 || n > (1ull << 34)) break;
                std::vector<float> v(n);
                if (std::fread(v.data(), 4, n, fp) != n) break;
                (*params)[key] = std::move(v);
            }
            ok = i == count;
        } while (false);
        std::fclose(fp);
        if (!ok) {
            delete params;
            return nullptr;
        }
        return params;
    }
};

}  // namespace foo
