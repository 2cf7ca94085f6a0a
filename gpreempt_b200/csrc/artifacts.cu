// Model directories in the reference's file formats: mod.json (TVM graph JSON), host.json
// (kernel list per fused function) and mod.params, as Model::load_from_json and
// ModelParamParser read them (src/model.cpp:15-55, 128-235; producer patch/tvm.patch:296-329).
//
// The reference's mod.json names a generated function per node and nothing else; what the
// function computes is baked into the generated mod.cu.  Here the kernels are the library's own,
// so a node carries its operator and hyper-parameters in `attrs` next to `func_name`
// (gpx_conv2d, gpx_max_pool2d, ...).  gpx_model_export_dir writes such a directory from any
// opened model; gpx_model_open(<directory>) rebuilds the graph from it.  A mod.json without those
// attributes (one written by TVM) is rejected with a message naming what is missing: its
// arithmetic cannot be recovered from the JSON alone.
#include "graph_builder.h"
#include "json.h"

#include <cerrno>
#include <fstream>
#include <sstream>
#include <sys/stat.h>

using namespace gpx;

namespace gpx {

static const char *func_name_of(const Node &n) {
    switch (n.op) {
        case Op::Conv: return "gpx_conv2d";
        case Op::DwConv: return "gpx_depthwise_conv2d";
        case Op::MaxPool: return "gpx_max_pool2d";
        case Op::AvgPool: return "gpx_avg_pool2d";
        case Op::LayerNorm: return "gpx_layer_norm";
        case Op::Attention: return "gpx_attention";
        case Op::Affine: return "gpx_affine";
        default: return "";
    }
}

static const char *kernel_type_name(KernelType t) {
    switch (t) {
        case KernelType::ConvSimt: return "conv_simt_kernel";
        case KernelType::Cgemm: return "cgemm_tcgen05_kernel";
        case KernelType::Pool: return "pool_kernel";
        case KernelType::Im2col: return "im2col_kernel";
        case KernelType::SplitK: return "splitk_finish_kernel";
        case KernelType::LayerNorm: return "layernorm_kernel";
        case KernelType::Attention: return "attention_kernel";
        case KernelType::DwConv: return "dwconv_kernel";
        case KernelType::AttentionTc: return "attention_tc_kernel";
        case KernelType::TransposeV: return "transpose_v_kernel";
        case KernelType::Stencil: return "miniweather_step_kernel";
        case KernelType::DenseRows: return "dense_rows_kernel";
        case KernelType::GraphWl: return "graphwl_kernel";
    }
    return "kernel";
}

static const char *dtype_name(int fmt) {
    return fmt == PF_BF16 ? "bfloat16" : fmt == PF_F16 ? "float16" : "float32";
}

// mod.json and host.json of an opened model.
static void render_graph(const gpx_model *m, Json *graph, Json *host) {
    Json nodes = Json::array(), arg_nodes = Json::array(), dltype = Json::array(), shapes = Json::array(),
         row_ptr = Json::array();
    std::unordered_map<int, int> storage_to_json;  // storage index -> json node id
    int jid = 0;
    auto shape_of = [&](const Storage &s) {
        Json sh = Json::array();
        if (s.token_major) {  // sequence activations are [N][S][C]
            sh.push(Json((long long)s.dims[0]));
            sh.push(Json((long long)s.dims[3]));
            sh.push(Json((long long)s.dims[1]));
            return sh;
        }
        for (int d = 0; d < s.rank; ++d) sh.push(Json((long long)s.dims[d]));
        return sh;
    };
    auto add_null = [&](int storage, const char *kind) {
        if (storage_to_json.count(storage)) return;
        const Storage &s = m->storages[storage];
        Json n = Json::object();
        n.set("op", "null");
        n.set("name", s.name);
        n.set("inputs", Json::array());
        Json a = Json::object();
        a.set("gpx_kind", kind);
        if (s.is_param) {
            a.set("init_mean", Json((double)s.init_mean));
            a.set("init_std", Json((double)s.init_std));
        }
        n.set("attrs", a);
        nodes.push(n);
        arg_nodes.push(Json(jid));
        dltype.push(Json(s.stype));
        shapes.push(shape_of(s));
        row_ptr.push(Json(jid));
        storage_to_json[storage] = jid++;
    };
    // temporaries of host.json: hidden storages (patch matrices, sub-sampled copies), 1-based
    std::unordered_map<int, int> temp_index;
    Json temp_args = Json::array();
    for (size_t i = 0; i < m->storages.size(); ++i)
        if (m->storages[i].hidden) {
            temp_index[(int)i] = (int)temp_args.size() + 1;
            temp_args.push(Json((long long)m->storages[i].bytes));
        }
    Json funcs = Json::array();
    int head_json = -1;
    for (size_t ni = 0; ni < m->nodes.size(); ++ni) {
        const Node &n = m->nodes[ni];
        const Storage &out = m->storages[n.storage];
        if (n.op == Op::Input) {
            add_null(n.storage, "input");
            continue;
        }
        if (n.op == Op::Buffer) {
            Json jn = Json::object();
            jn.set("op", "null");
            jn.set("name", n.name);
            jn.set("inputs", Json::array());
            Json a = Json::object();
            a.set("gpx_kind", "buffer");
            jn.set("attrs", a);
            nodes.push(jn);
            dltype.push(Json(out.stype));
            shapes.push(shape_of(out));
            row_ptr.push(Json(jid));
            storage_to_json[n.storage] = jid++;
            continue;
        }
        // parameters first, in the order the graph builder created them
        for (int t = 0; t < 3; ++t)
            if (n.tables[t] >= 0) add_null(n.tables[t], "table");
        if (n.weight >= 0) add_null(n.weight, "param");
        if (n.bias >= 0) add_null(n.bias, "param");
        if (n.scale >= 0) add_null(n.scale, "param");
        if (n.shift >= 0) add_null(n.shift, "param");
        Json jn = Json::object();
        jn.set("op", "tvm_op");
        jn.set("name", n.name);
        Json attrs = Json::object();
        attrs.set("func_name", func_name_of(n));
        attrs.set("flatten_data", "0");
        attrs.set("num_outputs", "1");
        attrs.set("kernel", Json(n.k));
        attrs.set("stride", Json(n.stride));
        attrs.set("padding", Json(n.pad));
        if (n.kw) attrs.set("kernel_w", Json(n.kw));
        if (n.pad_w >= 0) attrs.set("padding_w", Json(n.pad_w));
        if (n.count_pad) attrs.set("count_include_pad", Json(true));
        attrs.set("relu", Json(n.act == ACT_RELU));
        attrs.set("activation", Json(n.act));
        attrs.set("channels", Json(n.C));
        if (n.heads) attrs.set("heads", Json(n.heads));
        if (n.in_c) attrs.set("in_channels", Json(n.in_c));
        if (out.token_major) attrs.set("token_major", Json(true));
        if (out.parent >= 0) {
            attrs.set("slice_of", Json(storage_to_json[out.parent]));
            attrs.set("channel_offset", Json(out.ch_off));
        }
        Json inputs = Json::array();
        auto ref = [&](int storage) {
            Json r = Json::array();
            r.push(Json(storage_to_json[storage]));
            r.push(Json(0));
            r.push(Json(0));
            inputs.push(r);
        };
        if (n.op == Op::Attention) {
            for (int in : n.inputs) ref(m->nodes[in].storage);
        } else {
            ref(m->nodes[n.inputs[0]].storage);
            for (int t = 0; t < 3; ++t)
                if (n.tables[t] >= 0) ref(n.tables[t]);
            if (n.weight >= 0) ref(n.weight);
            if (n.bias >= 0) ref(n.bias);
            if (n.scale >= 0) ref(n.scale);
            if (n.shift >= 0) ref(n.shift);
            if (n.residual >= 0) {
                ref(m->nodes[n.residual].storage);
                attrs.set("residual", Json(true));
            }
        }
        attrs.set("num_inputs", std::to_string(inputs.size()));
        jn.set("attrs", attrs);
        jn.set("inputs", inputs);
        nodes.push(jn);
        dltype.push(Json(out.stype));
        shapes.push(shape_of(out));
        row_ptr.push(Json(jid));
        if ((int)ni == m->head_node) head_json = jid;
        storage_to_json[n.storage] = jid++;
        // host.json: this function's kernels (the entries of the kernel list that belong to the node)
        Json jf = Json::object();
        jf.set("name", func_name_of(n));
        Json kernels = Json::array();
        for (const Kernel &k : m->kernels) {
            if (k.node != (int)ni) continue;
            Json jk = Json::object();
            jk.set("name", std::string(kernel_type_name(k.type)) + ":" + k.name);
            Json lp = Json::array();
            lp.push(Json(k.grid));
            lp.push(Json(1));
            lp.push(Json(1));
            lp.push(Json(k.threads));
            lp.push(Json(1));
            lp.push(Json(1));
            jk.set("launch_params", lp);
            // arguments: the function's inputs and output by position; a kernel that reads or
            // writes a temporary names it by its negative 1-based index
            Json args = Json::array();
            for (size_t a = 0; a <= inputs.size(); ++a) args.push(Json((int)a));
            if (n.sub_storage >= 0 && temp_index.count(n.sub_storage) &&
                (k.type == KernelType::Im2col || k.type == KernelType::Cgemm || k.type == KernelType::Pool))
                args.push(Json(-temp_index[n.sub_storage]));
            jk.set("args", args);
            kernels.push(jk);
        }
        jf.set("kernels", kernels);
        funcs.push(jf);
    }
    row_ptr.push(Json(jid));
    Json root = Json::object();
    root.set("nodes", nodes);
    root.set("arg_nodes", arg_nodes);
    Json heads = Json::array(), h = Json::array();
    h.push(Json(head_json));
    h.push(Json(0));
    h.push(Json(0));
    heads.push(h);
    root.set("heads", heads);
    Json attrs = Json::object();
    Json dl = Json::array();
    dl.push("list_str");
    dl.push(dltype);
    attrs.set("dltype", dl);
    Json sh = Json::array();
    sh.push("list_shape");
    sh.push(shapes);
    attrs.set("shape", sh);
    root.set("attrs", attrs);
    root.set("node_row_ptr", row_ptr);
    Json meta = Json::object();
    meta.set("model", m->name);
    meta.set("batch", Json(m->batch));
    meta.set("dtype", dtype_name(m->fmt));
    meta.set("pad_channels", Json(m->pad_channels));
    root.set("gpx", meta);
    *graph = root;
    Json hroot = Json::object();
    hroot.set("temp_args", temp_args);
    hroot.set("funcs", funcs);
    *host = hroot;
}

static bool read_file(const std::string &path, std::string *out) {
    std::ifstream f(path, std::ios::binary);
    if (!f.is_open()) return false;
    std::stringstream ss;
    ss << f.rdbuf();
    *out = ss.str();
    return true;
}

bool model_dir_exists(const std::string &dir) {
    struct stat st;
    return ::stat((dir + "/mod.json").c_str(), &st) == 0;
}

// Rebuilds the graph of `dir`/mod.json in `m` (before finalize_model).
int build_graph_from_dir(gpx_model &m, const std::string &dir, const gpx_model_opts &opts) {
    std::string text, err;
    GPX_REQUIRE(read_file(dir + "/mod.json", &text), GPX_NOT_FOUND, "cannot open %s/mod.json", dir.c_str());
    Json root;
    GPX_REQUIRE(Json::parse(text, &root, &err), GPX_FAIL, "%s/mod.json is not valid JSON: %s", dir.c_str(), err.c_str());
    const Json &nodes = root["nodes"];
    const Json &shapes = root["attrs"]["shape"][(size_t)1];
    const Json &dltypes = root["attrs"]["dltype"][(size_t)1];
    GPX_REQUIRE(nodes.is_array() && nodes.size() > 0 && shapes.size() == nodes.size() && dltypes.size() == nodes.size(),
                GPX_FAIL, "%s/mod.json: nodes, attrs.shape and attrs.dltype do not agree", dir.c_str());
    const Json &meta = root["gpx"];
    GPX_REQUIRE(meta.is_object(), GPX_NOT_FOUND,
                "%s/mod.json has no \"gpx\" section: it was not written by gpx_model_export_dir (a TVM-generated graph "
                "keeps its operators in mod.cu, which this library does not load)", dir.c_str());
    m.pad_channels = meta["pad_channels"].as_bool(false);
    std::string dt = opts.dtype && opts.dtype[0] ? opts.dtype : meta["dtype"].as_string();
    m.fmt = PF_SPLIT;
    if (dt == "bfloat16" || dt == "bf16") m.fmt = PF_BF16;
    else if (dt == "float16" || dt == "fp16") m.fmt = PF_F16;
    else GPX_REQUIRE(dt.empty() || dt == "float32" || dt == "fp32", GPX_NOT_FOUND, "dtype '%s' is not available", dt.c_str());
    m.batch = (int)meta["batch"].as_int(1);
    GPX_REQUIRE(opts.batch <= 0 || opts.batch == m.batch, GPX_OUT_OF_RANGE,
                "%s was exported for batch %d, batch %d requested", dir.c_str(), m.batch, opts.batch);
    const long long head_id = root["heads"][(size_t)0][(size_t)0].as_int(-1);
    GPX_REQUIRE(head_id >= 0 && head_id < (long long)nodes.size(), GPX_FAIL, "%s/mod.json: bad heads entry", dir.c_str());

    GraphBuilder g(m);
    std::vector<int> node_of(nodes.size(), -1);     // json id -> graph node (activations)
    auto dim = [&](size_t i, int d) { return (int)shapes[i][d].as_int(1); };
    // Renames a storage the builder created to the name the file gives it.
    auto rename = [&](int storage, const std::string &name) {
        if (storage < 0 || m.storages[storage].name == name) return;
        m.storage_idx.erase(m.storages[storage].name);
        m.storages[storage].name = name;
        m.storage_idx[name] = storage;
    };
    auto apply_init = [&](int storage, const Json &jn) {
        if (storage < 0) return;
        const Json &a = jn["attrs"];
        if (a.has("init_std")) m.storages[storage].init_std = (float)a["init_std"].as_double();
        if (a.has("init_mean")) m.storages[storage].init_mean = (float)a["init_mean"].as_double();
    };
    for (size_t i = 0; i < nodes.size(); ++i) {
        const Json &jn = nodes[i];
        const std::string name = jn["name"].as_string();
        const Json &a = jn["attrs"];
        const Json &in = jn["inputs"];
        if (in.size() == 0) {
            const std::string kind = a["gpx_kind"].as_string();
            if (kind == "input") {
                if (dltypes[i].as_string() == "int64")
                    node_of[i] = g.input_ids(name, dim(i, 0), dim(i, 1));
                else
                    node_of[i] = g.input(name, dim(i, 0), dim(i, 1), dim(i, 2), dim(i, 3));
            } else if (kind == "buffer") {
                node_of[i] = g.buffer(name, dim(i, 0), dim(i, 1), dim(i, 2), dim(i, 3));
            } else {
                GPX_REQUIRE(kind == "param" || kind == "table", GPX_NOT_FOUND,
                            "%s/mod.json: node %zu (%s) has no gpx_kind attribute", dir.c_str(), i, name.c_str());
            }
            continue;  // parameters are created by the operator that owns them
        }
        const std::string fn = a["func_name"].as_string();
        GPX_REQUIRE(a.has("kernel") || fn == "gpx_attention" || fn == "gpx_layer_norm", GPX_NOT_FOUND,
                    "%s/mod.json: function %s of node %s carries no operator attributes", dir.c_str(), fn.c_str(), name.c_str());
        auto in_id = [&](size_t k) { return (size_t)in[k][(size_t)0].as_int(); };
        auto act_in = [&](size_t k) -> int { return k < in.size() && in_id(k) < node_of.size() ? node_of[in_id(k)] : -1; };
        auto in_name = [&](size_t k) { return nodes[in_id(k)]["name"].as_string(); };
        const int src = act_in(0);
        GPX_REQUIRE(src >= 0, GPX_FAIL, "%s/mod.json: node %s reads a tensor that is not defined before it", dir.c_str(), name.c_str());
        const int k = (int)a["kernel"].as_int(1), stride = (int)a["stride"].as_int(1), pad = (int)a["padding"].as_int(0);
        const int act = (int)a["activation"].as_int(0);
        const bool is_head = (long long)i == head_id;
        int id = -1;
        if (fn == "gpx_conv2d") {
            GPX_REQUIRE(in.size() >= 3, GPX_FAIL, "%s: convolution needs input, weight and bias", name.c_str());
            const bool tm = a["token_major"].as_bool(false);
            const int cout = tm ? dim(i, 2) : dim(i, 1);
            int res = a["residual"].as_bool(false) ? act_in(3) : -1;
            if (a.has("kernel_w") || a.has("padding_w")) {
                GPX_REQUIRE(res < 0 && !is_head, GPX_FAIL, "%s: a one-sided filter takes no residual and is no graph output", name.c_str());
                id = g.conv_rect(name, src, cout, k, (int)a["kernel_w"].as_int(k), stride, pad, (int)a["padding_w"].as_int(pad), false);
            } else {
                id = g.conv(name, src, cout, k, stride, pad, false, res, "", is_head);
            }
            m.nodes[id].act = act;
            if (tm) m.storages[m.nodes[id].storage].token_major = true;
        } else if (fn == "gpx_depthwise_conv2d") {
            id = g.dwconv(name, src, k, stride, pad, act);
        } else if (fn == "gpx_max_pool2d" || fn == "gpx_avg_pool2d") {
            std::string prefix;
            if (in.size() >= 3) {
                prefix = in_name(1);
                if (prefix.size() > 7 && prefix.compare(prefix.size() - 7, 7, ".weight") == 0) prefix.erase(prefix.size() - 7);
            }
            id = g.pool(name, src, fn == "gpx_max_pool2d" ? Op::MaxPool : Op::AvgPool, k, stride, pad, prefix);
            m.nodes[id].count_pad = a["count_include_pad"].as_bool(false);
        } else if (fn == "gpx_affine") {
            id = g.affine(name, src, (int)a["in_channels"].as_int(0), act);
        } else if (fn == "gpx_layer_norm") {
            const bool from_ids = m.storages[m.nodes[src].storage].kind == Storage::InputI64;
            const int C = dim(i, 2);
            int tables[3] = {-1, -1, -1};
            size_t p = 1;
            if (from_ids) {
                // inputs: ids, the embedding tables (word, position and, in BERT, token type), weight, bias
                GPX_REQUIRE(in.size() == 5 || in.size() == 6, GPX_FAIL, "%s: embedding layer norm needs two or three tables", name.c_str());
                const int ntab = (int)in.size() - 3;
                for (int t = 0; t < ntab; ++t, ++p) {
                    const size_t tid = in_id(p);
                    tables[t] = g.add_table(in_name(p), dim(tid, 0), dim(tid, 1), 0.02f);
                    apply_init(tables[t], nodes[tid]);
                }
            }
            std::string prefix = in_name(p);
            if (prefix.size() > 7 && prefix.compare(prefix.size() - 7, 7, ".weight") == 0) prefix.erase(prefix.size() - 7);
            id = g.layer_norm(name, src, C, prefix, from_ids ? tables : nullptr, is_head);
            rename(m.nodes[id].weight, in_name(p));
            rename(m.nodes[id].bias, in_name(p + 1));
            apply_init(m.nodes[id].weight, nodes[in_id(p)]);
            apply_init(m.nodes[id].bias, nodes[in_id(p + 1)]);
        } else if (fn == "gpx_attention") {
            GPX_REQUIRE(in.size() == 3 && act_in(1) >= 0 && act_in(2) >= 0, GPX_FAIL, "%s: attention needs q, k and v", name.c_str());
            id = g.attention(name, src, act_in(1), act_in(2), (int)a["heads"].as_int(1));
        } else {
            set_error("%s/mod.json: node %s uses function '%s', which this library does not provide", dir.c_str(),
                      name.c_str(), fn.c_str());
            return GPX_NOT_FOUND;
        }
        node_of[i] = id;
        Node &n = m.nodes[id];
        if (fn != "gpx_layer_norm") {
            // parameter names and initialisers as the file gives them (inputs after the activation)
            size_t p = 1;
            if (n.weight >= 0 && p < in.size()) {
                rename(n.weight, in_name(p));
                apply_init(n.weight, nodes[in_id(p)]);
                ++p;
            }
            if (n.bias >= 0 && p < in.size()) {
                rename(n.bias, in_name(p));
                apply_init(n.bias, nodes[in_id(p)]);
                ++p;
            }
            if (n.scale >= 0 && p < in.size()) {
                rename(n.scale, in_name(p));
                apply_init(n.scale, nodes[in_id(p)]);
                ++p;
            }
            if (n.shift >= 0 && p < in.size()) {
                rename(n.shift, in_name(p));
                apply_init(n.shift, nodes[in_id(p)]);
                ++p;
            }
        }
        if (a.has("slice_of")) {
            const size_t bid = (size_t)a["slice_of"].as_int();
            GPX_REQUIRE(bid < node_of.size() && node_of[bid] >= 0 && m.nodes[node_of[bid]].op == Op::Buffer, GPX_FAIL,
                        "%s: slice_of does not name a buffer node", name.c_str());
            g.place(id, node_of[bid], (int)a["channel_offset"].as_int(0));
        }
        if (is_head) m.head_node = id;
    }
    GPX_REQUIRE(m.head_node >= 0, GPX_FAIL, "%s/mod.json: heads does not name an operator node", dir.c_str());
    m.name = meta["model"].as_string();
    if (m.name.empty()) m.name = dir;
    return GPX_SUCC;
}

// After finalize_model: host.json must describe the functions of this graph, in order, as the
// reference checks ("Function name mismatch", src/model.cpp:200-214).
int check_host_json(const gpx_model &m, const std::string &dir) {
    std::string text, err;
    GPX_REQUIRE(read_file(dir + "/host.json", &text), GPX_NOT_FOUND, "cannot open %s/host.json", dir.c_str());
    Json host;
    GPX_REQUIRE(Json::parse(text, &host, &err), GPX_FAIL, "%s/host.json is not valid JSON: %s", dir.c_str(), err.c_str());
    const Json &funcs = host["funcs"];
    size_t fi = 0;
    for (size_t ni = 0; ni < m.nodes.size(); ++ni) {
        const Node &n = m.nodes[ni];
        if (n.op == Op::Input || n.op == Op::Buffer) continue;
        GPX_REQUIRE(fi < funcs.size(), GPX_FAIL, "%s/host.json lists %zu functions, the graph has more", dir.c_str(), funcs.size());
        const std::string want = func_name_of(n), got = funcs[fi]["name"].as_string();
        GPX_REQUIRE(want == got, GPX_FAIL, "Function name mismatch: %s vs %s (node %s)", got.c_str(), want.c_str(), n.name.c_str());
        size_t mine = 0;
        for (const Kernel &k : m.kernels) mine += k.node == (int)ni ? 1 : 0;
        // The kernel count of a function depends on the GPU (split K, column tiles): it is
        // informative in the file, only its presence is required.
        GPX_REQUIRE(funcs[fi]["kernels"].is_array() && (mine == 0 || funcs[fi]["kernels"].size() > 0), GPX_FAIL,
                    "%s/host.json: function %zu (%s) lists no kernels", dir.c_str(), fi, got.c_str());
        ++fi;
    }
    GPX_REQUIRE(fi == funcs.size(), GPX_FAIL, "%s/host.json lists %zu functions, the graph has %zu", dir.c_str(), funcs.size(), fi);
    return GPX_SUCC;
}

}  // namespace gpx

extern "C" {

int gpx_model_export_json(gpx_model *m, char *buf, size_t cap, size_t *needed) {
    GPX_REQUIRE(m, GPX_FAIL, "NULL model");
    GPX_REQUIRE(!m->sci, GPX_NOT_FOUND, "model '%s' has no graph to export", m->name.c_str());
    Json graph, host;
    render_graph(m, &graph, &host);
    std::string text = graph.dump(1);
    if (needed) *needed = text.size() + 1;
    if (!buf || cap < text.size() + 1) return buf ? GPX_OUT_OF_RANGE : GPX_SUCC;
    memcpy(buf, text.c_str(), text.size() + 1);
    return GPX_SUCC;
}

int gpx_model_export_dir(gpx_model *m, const char *dir) {
    GPX_REQUIRE(m && dir, GPX_FAIL, "NULL argument");
    GPX_REQUIRE(!m->sci, GPX_NOT_FOUND, "model '%s' has no graph to export", m->name.c_str());
    if (::mkdir(dir, 0777) != 0 && errno != EEXIST) {
        set_error("cannot create %s", dir);
        return GPX_FAIL;
    }
    Json graph, host;
    render_graph(m, &graph, &host);
    const std::string d(dir);
    {
        std::ofstream f(d + "/mod.json");
        GPX_REQUIRE(f.is_open(), GPX_FAIL, "cannot write %s/mod.json", dir);
        f << graph.dump(1);
    }
    {
        std::ofstream f(d + "/host.json");
        GPX_REQUIRE(f.is_open(), GPX_FAIL, "cannot write %s/host.json", dir);
        f << host.dump(1);
    }
    return gpx_model_save_params(m, (d + "/mod.params").c_str());
}

}  // extern "C"
