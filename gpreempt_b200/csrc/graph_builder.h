// Construction of a model graph node by node: storages for parameters and activations are
// created in call order, which also fixes the order the seeded initialiser visits them in.  Used
// by the built-in graphs (model.cu) and by the loader of graph files (artifacts.cu).
#pragma once

#include "model.h"

namespace gpx {

struct GraphBuilder {
    gpx_model &m;
    explicit GraphBuilder(gpx_model &model) : m(model) {}

    int add_act(const std::string &name, int N, int C, int H, int W, Storage::Kind kind) {
        Storage s;
        s.name = name;
        s.kind = kind;
        if (H == 1 && W == 1) {
            s.rank = 2;
            s.dims[0] = N;
            s.dims[1] = C;
        } else {
            s.rank = 4;
            s.dims[0] = N;
            s.dims[1] = C;
            s.dims[2] = H;
            s.dims[3] = W;
        }
        s.bytes = (size_t)N * C * H * W * sizeof(float);
        // Models with channel counts that are not multiples of 64 keep their activations padded
        // with zero channels, so every convolution still fits the tensor-core tile shapes.
        if (kind == Storage::ActSplit && m.pad_channels) s.cs = (C + 63) / 64 * 64;
        return m.add_storage(s);
    }

    // Depthwise k x k convolution + bias + activation (MobileNet's spatial filter).
    int dwconv(const std::string &name, int in, int k, int stride, int pad, int act) {
        const Node &src = m.nodes[in];
        Node n;
        n.name = name;
        n.op = Op::DwConv;
        n.inputs.push_back(in);
        n.k = k;
        n.stride = stride;
        n.pad = pad;
        n.act = act;
        n.N = src.N;
        n.C = src.C;
        n.H = (src.H + 2 * pad - k) / stride + 1;
        n.W = (src.W + 2 * pad - k) / stride + 1;
        Storage w;
        w.name = name + ".weight";
        w.kind = Storage::Weight;
        w.is_param = true;
        w.depthwise = true;
        w.rank = 4;
        w.dims[0] = src.C;
        w.dims[1] = 1;
        w.dims[2] = k;
        w.dims[3] = k;
        w.bytes = (size_t)src.C * k * k * sizeof(float);
        w.fan_in = k * k;
        n.weight = m.add_storage(w);
        n.bias = add_vec(name + ".bias", src.C, 0.f, 0.f);
        n.storage = add_act(name, n.N, n.C, n.H, n.W, Storage::ActSplit);
        m.nodes.push_back(n);
        return (int)m.nodes.size() - 1;
    }

    int input(const std::string &name, int N, int C, int H, int W) {
        Node n;
        n.name = name;
        n.op = Op::Input;
        n.N = N;
        n.H = H;
        n.W = W;
        n.C = C;
        n.storage = add_act(name, N, C, H, W, Storage::InputF32);
        m.nodes.push_back(n);
        return (int)m.nodes.size() - 1;
    }

    int conv(const std::string &name, int in, int cout, int k, int stride, int pad, bool relu,
             int residual = -1, const std::string &param_prefix = "", bool is_head = false) {
        const Node &src = m.nodes[in];
        Node n;
        n.name = name;
        n.op = Op::Conv;
        n.inputs.push_back(in);
        if (residual >= 0) n.inputs.push_back(residual);
        n.residual = residual;
        n.k = k;
        n.stride = stride;
        n.pad = pad;
        n.act = relu ? ACT_RELU : ACT_NONE;
        n.N = src.N;
        n.H = (src.H + 2 * pad - k) / stride + 1;
        n.W = (src.W + 2 * pad - k) / stride + 1;
        n.C = cout;
        const std::string pp = param_prefix.empty() ? name : param_prefix;
        Storage w;
        w.name = pp + ".weight";
        w.kind = Storage::Weight;
        w.is_param = true;
        w.rank = 4;
        w.dims[0] = cout;
        w.dims[1] = src.C;
        w.dims[2] = k;
        w.dims[3] = k;
        w.bytes = (size_t)cout * src.C * k * k * sizeof(float);
        w.fan_in = src.C * k * k;
        n.weight = m.add_storage(w);
        Storage b;
        b.name = pp + ".bias";
        b.kind = Storage::Vec;
        b.is_param = true;
        b.rank = 1;
        b.dims[0] = cout;
        b.bytes = (size_t)cout * sizeof(float);
        n.bias = m.add_storage(b);
        n.storage = add_act(name, n.N, n.C, n.H, n.W, is_head ? Storage::OutputF32 : Storage::ActSplit);
        m.nodes.push_back(n);
        return (int)m.nodes.size() - 1;
    }

    // Convolution with a kh x kw filter and separate vertical / horizontal padding (the factorised
    // 1x7 / 7x1 / 1x3 / 3x1 convolutions of Inception-v3), + bias + ReLU.
    int conv_rect(const std::string &name, int in, int cout, int kh, int kw, int stride, int ph, int pw,
                  bool relu) {
        int id = conv(name, in, cout, kh, stride, ph, relu);
        if (kh == kw && ph == pw) return id;
        Node &n = m.nodes[id];
        const Node &src = m.nodes[in];
        n.kw = kw;
        n.pad_w = pw;
        n.W = (src.W + 2 * pw - kw) / stride + 1;
        Storage &w = m.storages[n.weight];
        w.dims[3] = kw;
        w.bytes = (size_t)cout * src.C * kh * kw * sizeof(float);
        w.fan_in = src.C * kh * kw;
        Storage &out = m.storages[n.storage];
        out.dims[3] = n.W;
        out.bytes = (size_t)n.N * n.C * n.H * n.W * sizeof(float);
        return id;
    }

    // Fully connected layer over the flattened (C, H, W) input: a convolution whose filter
    // covers the whole feature map, so the canonical weight [out][C*H*W] is its OIHW filter.
    int dense(const std::string &name, int in, int cout, bool relu) {
        const Node &src = m.nodes[in];
        return conv(name, in, cout, src.H, 1, 0, relu);
    }

    // Token ids [N][S] (int64), the "data" input of sequence models.
    int input_ids(const std::string &name, int N, int S) {
        Node n;
        n.name = name;
        n.op = Op::Input;
        n.N = N;
        n.H = 1;
        n.W = S;
        n.C = 1;
        Storage s;
        s.name = name;
        s.kind = Storage::InputI64;
        s.stype = "int64";
        s.rank = 2;
        s.dims[0] = N;
        s.dims[1] = S;
        s.bytes = (size_t)N * S * sizeof(long long);
        n.storage = m.add_storage(s);
        m.nodes.push_back(n);
        return (int)m.nodes.size() - 1;
    }

    int add_vec(const std::string &name, int n, float mean, float std) {
        Storage s;
        s.name = name;
        s.kind = Storage::Vec;
        s.is_param = true;
        s.rank = 1;
        s.dims[0] = n;
        s.bytes = (size_t)n * sizeof(float);
        s.init_mean = mean;
        s.init_std = std;
        return m.add_storage(s);
    }

    int add_table(const std::string &name, int rows, int cols, float std) {
        Storage s;
        s.name = name;
        s.kind = Storage::Table;
        s.is_param = true;
        s.rank = 2;
        s.dims[0] = rows;
        s.dims[1] = cols;
        s.bytes = (size_t)rows * cols * sizeof(float);
        s.init_std = std;
        return m.add_storage(s);
    }

    // LayerNorm over channels.  `in` is an activation, or the token-id input when `tables` names
    // the word / position / token-type embedding tables (the sum is formed on the fly).
    int layer_norm(const std::string &name, int in, int C, const std::string &param_prefix,
                   const int *tables = nullptr, bool is_head = false) {
        const Node &src = m.nodes[in];
        Node n;
        n.name = name;
        n.op = Op::LayerNorm;
        n.inputs.push_back(in);
        n.N = src.N;
        n.H = src.H;
        n.W = src.W;
        n.C = C;
        n.weight = add_vec(param_prefix + ".weight", C, 1.0f, 0.02f);
        n.bias = add_vec(param_prefix + ".bias", C, 0.0f, 0.02f);
        if (tables)
            for (int i = 0; i < 3; ++i) n.tables[i] = tables[i];
        n.storage = add_act(name, n.N, n.C, n.H, n.W, is_head ? Storage::OutputF32 : Storage::ActSplit);
        m.storages[n.storage].token_major = true;
        m.nodes.push_back(n);
        return (int)m.nodes.size() - 1;
    }

    int attention(const std::string &name, int q, int k, int v, int heads) {
        const Node &src = m.nodes[q];
        Node n;
        n.name = name;
        n.op = Op::Attention;
        n.inputs = {q, k, v};
        n.N = src.N;
        n.H = src.H;
        n.W = src.W;
        n.C = src.C;
        n.heads = heads;
        n.storage = add_act(name, n.N, n.C, n.H, n.W, Storage::ActSplit);
        m.storages[n.storage].token_major = true;
        m.nodes.push_back(n);
        return (int)m.nodes.size() - 1;
    }

    // Dense layer of a sequence model: a 1x1 convolution over [N][1][S][C] with N(0, 0.02) weights.
    int linear(const std::string &name, int in, int cout, int act, int residual = -1) {
        int id = conv(name + ".out", in, cout, 1, 1, 0, false, residual, name);
        m.nodes[id].act = act;
        m.storages[m.nodes[id].storage].token_major = true;
        m.storages[m.nodes[id].weight].init_std = 0.02f;
        m.storages[m.nodes[id].bias].init_std = 0.02f;
        return id;
    }

    // Pooling; with `norm_prefix` the input first goes through a per-channel affine + ReLU (a
    // batch norm that sits between the producer and the pooling, as DenseNet's last one does).
    int pool(const std::string &name, int in, Op op, int k, int stride, int pad,
             const std::string &norm_prefix = "") {
        const Node &src = m.nodes[in];
        Node n;
        n.name = name;
        n.op = op;
        n.inputs.push_back(in);
        n.k = k;
        n.stride = stride;
        n.pad = pad;
        n.N = src.N;
        n.C = src.C;
        n.H = (src.H + 2 * pad - k) / stride + 1;
        n.W = (src.W + 2 * pad - k) / stride + 1;
        if (!norm_prefix.empty()) {
            n.scale = add_vec(norm_prefix + ".weight", src.C, 1.0f, 0.02f);
            n.shift = add_vec(norm_prefix + ".bias", src.C, 0.0f, 0.02f);
            n.act = ACT_RELU;
        }
        n.storage = add_act(name, n.N, n.C, n.H, n.W, Storage::ActSplit);
        m.nodes.push_back(n);
        return (int)m.nodes.size() - 1;
    }

    // A tensor that other nodes fill slice by slice: concatenation along channels by placement.
    int buffer(const std::string &name, int N, int C, int H, int W) {
        Node n;
        n.name = name;
        n.op = Op::Buffer;
        n.N = N;
        n.C = C;
        n.H = H;
        n.W = W;
        n.storage = add_act(name, N, C, H, W, Storage::ActSplit);
        m.nodes.push_back(n);
        return (int)m.nodes.size() - 1;
    }

    // Makes the output of node `id` the channels [off, off + C) of the buffer node `buf`.
    void place(int id, int buf, int off) {
        Storage &s = m.storages[m.nodes[id].storage];
        s.parent = m.nodes[buf].storage;
        s.ch_off = off;
        s.cs = 0;
    }

    // act(x * scale + shift) over the first `in_c` channels of `in` (a batch norm ahead of its
    // convolution, folded to an affine map), written as a tensor of its own.
    int affine(const std::string &name, int in, int in_c, int act) {
        const Node &src = m.nodes[in];
        Node n;
        n.name = name;
        n.op = Op::Affine;
        n.inputs.push_back(in);
        n.in_c = in_c;
        n.act = act;
        n.N = src.N;
        n.C = in_c;
        n.H = src.H;
        n.W = src.W;
        n.scale = add_vec(name + ".weight", in_c, 1.0f, 0.02f);
        n.shift = add_vec(name + ".bias", in_c, 0.0f, 0.02f);
        n.storage = add_act(name, n.N, n.C, n.H, n.W, Storage::ActSplit);
        m.nodes.push_back(n);
        return (int)m.nodes.size() - 1;
    }
};


}  // namespace gpx
