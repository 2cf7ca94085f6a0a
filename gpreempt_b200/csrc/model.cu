// Model runtime: built-in graphs, storages, parameter files, name-addressed tensor I/O and
// the kernel list.  Counterpart of src/model.cpp in the reference (Model::load_model :79-125,
// load_from_json :128-235, load_param :263-282, get/set :288-321, ModelParamParser :15-55).
#include "model.h"
#include "graph_builder.h"
#include "json.h"

#include <algorithm>
#include <cmath>
#include <memory>

using namespace gpx;

int gpx_model::add_storage(const Storage &s) {
    storage_idx[s.name] = storages.size();
    storages.push_back(s);
    return (int)storages.size() - 1;
}

int gpx_model::find(const std::string &n) const {
    auto it = storage_idx.find(n);
    return it == storage_idx.end() ? -1 : (int)it->second;
}

namespace gpx {

// ---- seeded synthetic data ------------------------------------------------------------------
// Counter-based generator: element i of stream t under seed s is a pure function of (s, t, i),
// so tensors can be produced in any order and on any number of threads.

static inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static inline uint64_t counter_bits(uint64_t seed, uint64_t stream, uint64_t i) {
    return mix64(mix64(seed * 0xD1342543DE82EF95ull + stream) ^ (i * 0x2545F4914F6CDD1Dull + 1));
}

void normal_fill(float *dst, size_t n, uint64_t seed, uint64_t stream, float mean, float std) {
    const double two_pi = 6.283185307179586476925286766559;
    for (size_t i = 0; i < n; ++i) {
        uint64_t h = counter_bits(seed, stream, i);
        double u1 = ((double)(uint32_t)(h >> 32) + 1.0) * (1.0 / 4294967296.0);  // (0, 1]
        double u2 = (double)(uint32_t)h * (1.0 / 4294967296.0);                  // [0, 1)
        double z = std::sqrt(-2.0 * std::log(u1)) * std::cos(two_pi * u2);
        dst[i] = (float)(mean + std * z);
    }
}

void uniform_fill(float *dst, size_t n, uint64_t seed, uint64_t stream, float lo, float hi) {
    for (size_t i = 0; i < n; ++i) {
        uint64_t h = counter_bits(seed, stream, i);
        double u = (double)(h >> 11) * (1.0 / 9007199254740992.0);  // [0, 1)
        dst[i] = (float)(lo + (hi - lo) * u);
    }
}

// ---- built-in graphs ------------------------------------------------------------------------

// ResNet v1.5 with bottleneck blocks (stride on the 3x3 convolution), batch norm folded into
// each convolution's bias.  layers = {3,4,6,3} gives ResNet-50, {3,8,36,3} ResNet-152.
static void build_resnet(gpx_model &m, int batch, const int layers[4]) {
    GraphBuilder g(m);
    int x = g.input("data", batch, 3, 224, 224);
    x = g.conv("conv1", x, 64, 7, 2, 3, true);
    x = g.pool("maxpool", x, Op::MaxPool, 3, 2, 1);
    int planes = 64;
    for (int l = 0; l < 4; ++l) {
        for (int b = 0; b < layers[l]; ++b) {
            std::string p = "layer" + std::to_string(l + 1) + "." + std::to_string(b);
            int stride = (b == 0 && l > 0) ? 2 : 1;
            int identity = x;
            if (b == 0) identity = g.conv(p + ".downsample", x, planes * 4, 1, stride, 0, false);
            int y = g.conv(p + ".conv1", x, planes, 1, 1, 0, true);
            y = g.conv(p + ".conv2", y, planes, 3, stride, 1, true);
            x = g.conv(p + ".conv3", y, planes * 4, 1, 1, 0, true, identity);
        }
        planes *= 2;
    }
    x = g.pool("avgpool", x, Op::AvgPool, 7, 1, 0);
    x = g.conv("heads", x, 1000, 1, 1, 0, false, -1, "fc", true);
    m.head_node = x;
}

// VGG configuration D/E: 3x3 convolutions + ReLU, 2x2 max pooling, three dense layers.
static void build_vgg(gpx_model &m, int batch, const int *cfg, int ncfg) {
    GraphBuilder g(m);
    int x = g.input("data", batch, 3, 224, 224);
    int ci = 0, pi = 0;
    for (int i = 0; i < ncfg; ++i) {
        if (cfg[i] == 0) {
            x = g.pool("pool" + std::to_string(pi++), x, Op::MaxPool, 2, 2, 0);
        } else {
            x = g.conv("features." + std::to_string(ci++), x, cfg[i], 3, 1, 1, true);
        }
    }
    x = g.dense("classifier.0", x, 4096, true);
    x = g.dense("classifier.3", x, 4096, true);
    x = g.conv("heads", x, 1000, 1, 1, 0, false, -1, "classifier.6", true);
    m.head_node = x;
}

// MobileNetV2 (Sandler et al. 2018, the torchvision layer schedule): 3x3 stride-2 stem, 17
// inverted-residual blocks (1x1 expand + ReLU6, 3x3 depthwise + ReLU6, 1x1 linear projection,
// identity shortcut when the shape is kept), 1x1 to 1280 channels, global average pool, dense.
// Batch norm is folded into each convolution's bias.
static void build_mobilenet_v2(gpx_model &m, int batch) {
    m.pad_channels = true;
    GraphBuilder g(m);
    int x = g.input("data", batch, 3, 224, 224);
    x = g.conv("features.0", x, 32, 3, 2, 1, false);
    m.nodes[x].act = ACT_RELU6;
    static const int cfg[7][4] = {{1, 16, 1, 1}, {6, 24, 2, 2}, {6, 32, 3, 2}, {6, 64, 4, 2},
                                  {6, 96, 3, 1}, {6, 160, 3, 2}, {6, 320, 1, 1}};
    int cin = 32, idx = 1;
    for (int s = 0; s < 7; ++s) {
        for (int r = 0; r < cfg[s][2]; ++r, ++idx) {
            const std::string p = "features." + std::to_string(idx);
            const int t = cfg[s][0], cout = cfg[s][1], stride = r == 0 ? cfg[s][3] : 1;
            int y = x;
            if (t != 1) {
                y = g.conv(p + ".expand", y, cin * t, 1, 1, 0, false);
                m.nodes[y].act = ACT_RELU6;
            }
            y = g.dwconv(p + ".dw", y, 3, stride, 1, ACT_RELU6);
            const bool shortcut = stride == 1 && cin == cout;
            x = g.conv(p + ".project", y, cout, 1, 1, 0, false, shortcut ? x : -1);
            cin = cout;
        }
    }
    x = g.conv("features.18", x, 1280, 1, 1, 0, false);
    m.nodes[x].act = ACT_RELU6;
    x = g.pool("avgpool", x, Op::AvgPool, 7, 1, 0);
    x = g.conv("heads", x, 1000, 1, 1, 0, false, -1, "classifier", true);
    m.head_node = x;
    // Without batch norm a He-normal draw drives the ReLU6 units into saturation through the
    // linear bottlenecks; N(0, 1/fan_in) keeps the seeded activations in the unclamped range.
    for (auto &s : m.storages)
        if (s.kind == Storage::Weight && s.fan_in > 0) s.init_std = sqrtf(1.0f / (float)s.fan_in);
}

// DenseNet (Huang et al. 2017, the torchvision layer schedule and parameter names): 7x7 stem,
// four dense blocks of {6, 12, 48, 32} layers for DenseNet-201 with growth 32, transitions that
// halve channels and resolution.  Every dense layer is norm-ReLU-1x1(128)-norm-ReLU-3x3(32); the
// first norm acts on the running concatenation and stays an affine node of its own, the second
// is folded into the 1x1 convolution's bias.  A block's concatenation is one buffer that the
// block's layers write 32-channel slices of.
static void build_densenet(gpx_model &m, int batch, const int *cfg, int growth, int init_features) {
    m.pad_channels = true;
    GraphBuilder g(m);
    int x = g.input("data", batch, 3, 224, 224);
    x = g.conv("features.conv0", x, init_features, 7, 2, 3, true);
    int C = init_features, H = 56;
    int buf = g.buffer("features.denseblock1", batch, C + growth * cfg[0], H, H);
    g.place(g.pool("features.pool0", x, Op::MaxPool, 3, 2, 1), buf, 0);
    for (int b = 0; b < 4; ++b) {
        for (int l = 0; l < cfg[b]; ++l) {
            const std::string p = "features.denseblock" + std::to_string(b + 1) + ".denselayer" + std::to_string(l + 1);
            const int cin = C + growth * l;
            int a = g.affine(p + ".norm1", buf, cin, ACT_RELU);
            int y = g.conv(p + ".conv1", a, 4 * growth, 1, 1, 0, true);
            int z = g.conv(p + ".conv2", y, growth, 3, 1, 1, false);
            g.place(z, buf, cin);
        }
        C += growth * cfg[b];
        if (b == 3) break;
        const std::string t = "features.transition" + std::to_string(b + 1);
        int a = g.affine(t + ".norm", buf, C, ACT_RELU);
        int y = g.conv(t + ".conv", a, C / 2, 1, 1, 0, false);
        C /= 2;
        H /= 2;
        buf = g.buffer("features.denseblock" + std::to_string(b + 2), batch, C + growth * cfg[b + 1], H, H);
        g.place(g.pool(t + ".pool", y, Op::AvgPool, 2, 2, 0), buf, 0);
    }
    x = g.pool("avgpool", buf, Op::AvgPool, H, 1, 0, "features.norm5");
    x = g.conv("heads", x, 1000, 1, 1, 0, false, -1, "classifier", true);
    m.head_node = x;
}

// BERT encoder (post-LayerNorm): embeddings + LayerNorm, then per layer Q/K/V projections,
// multi-head attention, output projection + residual + LayerNorm, GELU feed-forward + residual +
// LayerNorm.  "heads" is the last hidden state [N][S][hidden] in fp32.  Parameter names follow
// the Hugging Face BertModel state dict.
static void build_bert(gpx_model &m, int batch, int seq, int layers, int hidden, int heads, int ffn,
                       int vocab, int max_pos) {
    GraphBuilder g(m);
    int ids = g.input_ids("data", batch, seq);
    int tables[3];
    tables[0] = g.add_table("embeddings.word_embeddings.weight", vocab, hidden, 0.02f);
    tables[1] = g.add_table("embeddings.position_embeddings.weight", max_pos, hidden, 0.02f);
    tables[2] = g.add_table("embeddings.token_type_embeddings.weight", 2, hidden, 0.02f);
    int x = g.layer_norm("embeddings", ids, hidden, "embeddings.LayerNorm", tables);
    for (int l = 0; l < layers; ++l) {
        const std::string p = "encoder.layer." + std::to_string(l);
        int q = g.linear(p + ".attention.self.query", x, hidden, ACT_NONE);
        int k = g.linear(p + ".attention.self.key", x, hidden, ACT_NONE);
        int v = g.linear(p + ".attention.self.value", x, hidden, ACT_NONE);
        int ctx = g.attention(p + ".attention.context", q, k, v, heads);
        int a = g.linear(p + ".attention.output.dense", ctx, hidden, ACT_NONE, x);
        x = g.layer_norm(p + ".attention.output", a, hidden, p + ".attention.output.LayerNorm");
        int h = g.linear(p + ".intermediate.dense", x, ffn, ACT_GELU);
        int o = g.linear(p + ".output.dense", h, hidden, ACT_NONE, x);
        bool last = l == layers - 1;
        x = g.layer_norm(last ? "heads" : p + ".output", o, hidden, p + ".output.LayerNorm", nullptr, last);
    }
    m.head_node = x;
}

// Inception-v3 (Szegedy et al. 2016) in the torchvision layer schedule and parameter names: one
// of the models the reference compiles (scripts/compile/compile.py:27-36, 3x299x299 input; its
// relay.testing definition pools the last block's pooling branch with max where this one
// averages).  Every convolution carries its folded batch norm as a bias and a ReLU; a block's
// concatenation is one buffer its branches write channel slices of.  The 1x1 and padded 3x3
// convolutions run on the tensor cores, the one-sided (1x7, 7x1, 1x3, 3x1), 5x5 and unpadded
// stride-2 filters on the CUDA-core kernel.
static void build_inception_v3(gpx_model &m, int batch) {
    m.pad_channels = true;
    GraphBuilder g(m);
    auto cv = [&](const std::string &name, int in, int cout, int kh, int kw, int stride, int ph, int pw) {
        return g.conv_rect(name, in, cout, kh, kw, stride, ph, pw, true);
    };
    auto avg3 = [&](const std::string &name, int in) {
        int id = g.pool(name, in, Op::AvgPool, 3, 1, 1);
        m.nodes[id].count_pad = true;
        return id;
    };
    int x = g.input("data", batch, 3, 299, 299);
    x = cv("Conv2d_1a_3x3", x, 32, 3, 3, 2, 0, 0);
    x = cv("Conv2d_2a_3x3", x, 32, 3, 3, 1, 0, 0);
    x = cv("Conv2d_2b_3x3", x, 64, 3, 3, 1, 1, 1);
    x = g.pool("maxpool1", x, Op::MaxPool, 3, 2, 0);
    x = cv("Conv2d_3b_1x1", x, 80, 1, 1, 1, 0, 0);
    x = cv("Conv2d_4a_3x3", x, 192, 3, 3, 1, 0, 0);
    x = g.pool("maxpool2", x, Op::MaxPool, 3, 2, 0);
    int S = 35;
    const int pool_features[3] = {32, 64, 64};
    const char *a_names[3] = {"Mixed_5b", "Mixed_5c", "Mixed_5d"};
    for (int b = 0; b < 3; ++b) {
        const std::string p = a_names[b];
        int buf = g.buffer(p, batch, 64 + 64 + 96 + pool_features[b], S, S);
        g.place(cv(p + ".branch1x1", x, 64, 1, 1, 1, 0, 0), buf, 0);
        int t = cv(p + ".branch5x5_1", x, 48, 1, 1, 1, 0, 0);
        g.place(cv(p + ".branch5x5_2", t, 64, 5, 5, 1, 2, 2), buf, 64);
        t = cv(p + ".branch3x3dbl_1", x, 64, 1, 1, 1, 0, 0);
        t = cv(p + ".branch3x3dbl_2", t, 96, 3, 3, 1, 1, 1);
        g.place(cv(p + ".branch3x3dbl_3", t, 96, 3, 3, 1, 1, 1), buf, 128);
        g.place(cv(p + ".branch_pool", avg3(p + ".pool", x), pool_features[b], 1, 1, 1, 0, 0), buf, 224);
        x = buf;
    }
    {
        const std::string p = "Mixed_6a";
        S = 17;
        int buf = g.buffer(p, batch, 384 + 96 + 288, S, S);
        g.place(cv(p + ".branch3x3", x, 384, 3, 3, 2, 0, 0), buf, 0);
        int t = cv(p + ".branch3x3dbl_1", x, 64, 1, 1, 1, 0, 0);
        t = cv(p + ".branch3x3dbl_2", t, 96, 3, 3, 1, 1, 1);
        g.place(cv(p + ".branch3x3dbl_3", t, 96, 3, 3, 2, 0, 0), buf, 384);
        g.place(g.pool(p + ".pool", x, Op::MaxPool, 3, 2, 0), buf, 480);
        x = buf;
    }
    const int c7s[4] = {128, 160, 160, 192};
    const char *c_names[4] = {"Mixed_6b", "Mixed_6c", "Mixed_6d", "Mixed_6e"};
    for (int b = 0; b < 4; ++b) {
        const std::string p = c_names[b];
        const int c7 = c7s[b];
        int buf = g.buffer(p, batch, 768, S, S);
        g.place(cv(p + ".branch1x1", x, 192, 1, 1, 1, 0, 0), buf, 0);
        int t = cv(p + ".branch7x7_1", x, c7, 1, 1, 1, 0, 0);
        t = cv(p + ".branch7x7_2", t, c7, 1, 7, 1, 0, 3);
        g.place(cv(p + ".branch7x7_3", t, 192, 7, 1, 1, 3, 0), buf, 192);
        t = cv(p + ".branch7x7dbl_1", x, c7, 1, 1, 1, 0, 0);
        t = cv(p + ".branch7x7dbl_2", t, c7, 7, 1, 1, 3, 0);
        t = cv(p + ".branch7x7dbl_3", t, c7, 1, 7, 1, 0, 3);
        t = cv(p + ".branch7x7dbl_4", t, c7, 7, 1, 1, 3, 0);
        g.place(cv(p + ".branch7x7dbl_5", t, 192, 1, 7, 1, 0, 3), buf, 384);
        g.place(cv(p + ".branch_pool", avg3(p + ".pool", x), 192, 1, 1, 1, 0, 0), buf, 576);
        x = buf;
    }
    {
        const std::string p = "Mixed_7a";
        S = 8;
        int buf = g.buffer(p, batch, 320 + 192 + 768, S, S);
        int t = cv(p + ".branch3x3_1", x, 192, 1, 1, 1, 0, 0);
        g.place(cv(p + ".branch3x3_2", t, 320, 3, 3, 2, 0, 0), buf, 0);
        t = cv(p + ".branch7x7x3_1", x, 192, 1, 1, 1, 0, 0);
        t = cv(p + ".branch7x7x3_2", t, 192, 1, 7, 1, 0, 3);
        t = cv(p + ".branch7x7x3_3", t, 192, 7, 1, 1, 3, 0);
        g.place(cv(p + ".branch7x7x3_4", t, 192, 3, 3, 2, 0, 0), buf, 320);
        g.place(g.pool(p + ".pool", x, Op::MaxPool, 3, 2, 0), buf, 512);
        x = buf;
    }
    const char *e_names[2] = {"Mixed_7b", "Mixed_7c"};
    for (int b = 0; b < 2; ++b) {
        const std::string p = e_names[b];
        int buf = g.buffer(p, batch, 2048, S, S);
        g.place(cv(p + ".branch1x1", x, 320, 1, 1, 1, 0, 0), buf, 0);
        int t = cv(p + ".branch3x3_1", x, 384, 1, 1, 1, 0, 0);
        g.place(cv(p + ".branch3x3_2a", t, 384, 1, 3, 1, 0, 1), buf, 320);
        g.place(cv(p + ".branch3x3_2b", t, 384, 3, 1, 1, 1, 0), buf, 704);
        t = cv(p + ".branch3x3dbl_1", x, 448, 1, 1, 1, 0, 0);
        t = cv(p + ".branch3x3dbl_2", t, 384, 3, 3, 1, 1, 1);
        g.place(cv(p + ".branch3x3dbl_3a", t, 384, 1, 3, 1, 0, 1), buf, 1088);
        g.place(cv(p + ".branch3x3dbl_3b", t, 384, 3, 1, 1, 1, 0), buf, 1472);
        g.place(cv(p + ".branch_pool", avg3(p + ".pool", x), 192, 1, 1, 1, 0, 0), buf, 1856);
        x = buf;
    }
    x = g.pool("avgpool", x, Op::AvgPool, S, 1, 0);
    x = g.conv("heads", x, 1000, 1, 1, 0, false, -1, "fc", true);
    m.head_node = x;
}

// DistilBERT (Sanh et al. 2019; the Hugging Face DistilBertModel layout and parameter names): the
// BERT encoder without token-type embeddings, 6 layers for distilbert-base.  This is the sequence
// model the reference compiles (scripts/compile/compile-bert.py:33-52, traced on a 6-token input);
// "heads" is the last hidden state.
static void build_distilbert(gpx_model &m, int batch, int seq, int layers, int hidden, int heads, int ffn,
                             int vocab, int max_pos) {
    GraphBuilder g(m);
    int ids = g.input_ids("data", batch, seq);
    int tables[3];
    tables[0] = g.add_table("embeddings.word_embeddings.weight", vocab, hidden, 0.02f);
    tables[1] = g.add_table("embeddings.position_embeddings.weight", max_pos, hidden, 0.02f);
    tables[2] = -1;
    int x = g.layer_norm("embeddings", ids, hidden, "embeddings.LayerNorm", tables);
    for (int l = 0; l < layers; ++l) {
        const std::string p = "transformer.layer." + std::to_string(l);
        int q = g.linear(p + ".attention.q_lin", x, hidden, ACT_NONE);
        int k = g.linear(p + ".attention.k_lin", x, hidden, ACT_NONE);
        int v = g.linear(p + ".attention.v_lin", x, hidden, ACT_NONE);
        int ctx = g.attention(p + ".attention.context", q, k, v, heads);
        int a = g.linear(p + ".attention.out_lin", ctx, hidden, ACT_NONE, x);
        x = g.layer_norm(p + ".sa_output", a, hidden, p + ".sa_layer_norm");
        int h = g.linear(p + ".ffn.lin1", x, ffn, ACT_GELU);
        int o = g.linear(p + ".ffn.lin2", h, hidden, ACT_NONE, x);
        bool last = l == layers - 1;
        x = g.layer_norm(last ? "heads" : p + ".output", o, hidden, p + ".output_layer_norm", nullptr, last);
    }
    m.head_node = x;
}

int build_builtin_graph(gpx_model &m, const std::string &name, const gpx_model_opts &opts) {
    int batch = opts.batch > 0 ? opts.batch : 1;
    m.batch = batch;
    if (is_miniweather(name)) {
        // The scientific workload (Executor::init, src/executor.cpp:35-38): no graph, no parameters.
        m.name = name;
        return build_miniweather(m, name, opts);
    }
    if (is_graph_workload(name)) {
        // The graph-analytics workloads (Executor::init, src/executor.cpp:24-34).
        m.name = name;
        return build_graph_workload(m, name, opts);
    }
    // Storage and tensor-core operand format between layers; inputs, outputs, parameters and all
    // arithmetic outside the tensor-core products stay fp32.
    m.fmt = PF_SPLIT;
    if (opts.dtype && opts.dtype[0]) {
        const std::string dt = opts.dtype;
        if (dt == "float32" || dt == "fp32")
            m.fmt = PF_SPLIT;
        else if (dt == "bfloat16" || dt == "bf16")
            m.fmt = PF_BF16;
        else if (dt == "float16" || dt == "fp16")
            m.fmt = PF_F16;
        else {
            set_error("dtype '%s' is not available for model '%s' (float32, bfloat16, float16)", opts.dtype,
                      name.c_str());
            return GPX_NOT_FOUND;
        }
    }
    if (name == "resnet50") {
        const int l[4] = {3, 4, 6, 3};
        build_resnet(m, batch, l);
    } else if (name == "resnet152") {
        const int l[4] = {3, 8, 36, 3};
        build_resnet(m, batch, l);
    } else if (name == "resnet_tiny") {
        // Two-stage miniature with the same block structure, for fast tests.
        const int l[4] = {1, 1, 1, 1};
        build_resnet(m, batch, l);
    } else if (name == "vgg16") {
        const int cfg[] = {64, 64, 0, 128, 128, 0, 256, 256, 256, 0, 512, 512, 512, 0, 512, 512, 512, 0};
        build_vgg(m, batch, cfg, (int)(sizeof(cfg) / sizeof(int)));
    } else if (name == "vgg" || name == "vgg19") {
        const int cfg[] = {64, 64, 0, 128, 128, 0, 256, 256, 256, 256, 0, 512, 512, 512, 512, 0,
                           512, 512, 512, 512, 0};
        build_vgg(m, batch, cfg, (int)(sizeof(cfg) / sizeof(int)));
    } else if (name == "mobilenet_v2") {
        build_mobilenet_v2(m, batch);
    } else if (name == "inception_v3" || name == "inception") {
        build_inception_v3(m, batch);
    } else if (name == "densenet201" || name == "densenet") {
        const int cfg[4] = {6, 12, 48, 32};
        build_densenet(m, batch, cfg, 32, 64);
    } else if (name == "densenet_tiny") {
        // Same structure with a few layers per block (channel counts stay multiples of 32), for
        // fast tests.
        const int cfg[4] = {2, 2, 4, 2};
        build_densenet(m, batch, cfg, 32, 64);
    } else if (name == "distilbert" || name == "bert") {
        // "bert" is what the reference's task configs call its DistilBERT build (config/C.json); its
        // sequence length is the 6 tokens the model was traced on unless the client gives one.
        int seq = opts.seq_len > 0 ? opts.seq_len : 6;
        if (seq > 512 || (m.fmt != PF_SPLIT && seq % 8 != 0)) {
            set_error("distilbert: seq_len %d must be at most 512 (and a multiple of 8 in the 16-bit formats)", seq);
            return GPX_OUT_OF_RANGE;
        }
        build_distilbert(m, batch, seq, 6, 768, 12, 3072, 30522, 512);
    } else if (name == "distilbert_tiny") {
        int seq = opts.seq_len > 0 ? opts.seq_len : 6;
        build_distilbert(m, batch, seq, 2, 128, 2, 256, 1000, 512);
    } else if (name == "bert_base") {
        int seq = opts.seq_len > 0 ? opts.seq_len : 128;
        if (seq > 512 || seq % 8 != 0) {
            set_error("bert_base: seq_len %d must be a multiple of 8 and at most 512", seq);
            return GPX_OUT_OF_RANGE;
        }
        build_bert(m, batch, seq, 12, 768, 12, 3072, 30522, 512);
    } else if (name == "bert_tiny") {
        // Two-layer miniature with the same structure, for fast tests.
        int seq = opts.seq_len > 0 ? opts.seq_len : 64;
        build_bert(m, batch, seq, 2, 128, 2, 256, 1000, 512);
    } else {
        set_error("unknown model '%s'", name.c_str());
        return GPX_NOT_FOUND;
    }
    m.name = name;
    return GPX_SUCC;
}

// ---- storages and kernel list ---------------------------------------------------------------

static inline bf16_bits host_f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_bits)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (bf16_bits)(u >> 16);
}
static inline float host_bf16_to_f32(bf16_bits v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// One element into / out of host copies of the planes (`pe` = elements per plane; the second
// plane exists only in the two-plane format).
static inline void host_put(std::vector<bf16_bits> &pl, size_t pe, size_t off, float v, int fmt) {
    if (fmt == PF_F16) {
        __half h = __float2half_rn(v);
        memcpy(&pl[off], &h, 2);
        return;
    }
    bf16_bits hi = host_f32_to_bf16(v);
    pl[off] = hi;
    if (fmt == PF_SPLIT) pl[pe + off] = host_f32_to_bf16(v - host_bf16_to_f32(hi));
}
static inline float host_take(const std::vector<bf16_bits> &pl, size_t pe, size_t off, int fmt) {
    if (fmt == PF_F16) {
        __half h;
        memcpy(&h, &pl[off], 2);
        return __half2float(h);
    }
    float v = host_bf16_to_f32(pl[off]);
    if (fmt == PF_SPLIT) v += host_bf16_to_f32(pl[pe + off]);
    return v;
}
static inline size_t plane_count(int fmt) { return fmt == PF_SPLIT ? 2 : 1; }

// Shape test for the tensor-core convolution: 64-channel granularity on both sides and one of
// the four geometries it implements as row-shifted GEMMs.
// Channels as stored: the logical count, or its padding to 64 in models that pad.
static int stored_c(const gpx_model &m, const Node &n) {
    const Storage &s = m.storages[n.storage];
    return s.cs ? s.cs : n.C;
}

static bool full_map_dense(const Node &n, const Node &src) {
    return n.op == Op::Conv && n.k > 1 && n.k == src.H && n.k == src.W && n.pad == 0 && n.stride == 1;
}

static bool tensor_core_shape(const gpx_model &m, const Node &n, const Node &src) {
    if (n.op != Op::Conv) return false;
    if ((n.kw && n.kw != n.k) || (n.pad_w >= 0 && n.pad_w != n.pad)) return false;  // one-sided filters: CUDA cores
    // Input channels in whole 64-wide K blocks; output channels in 16-byte vectors (the epilogue
    // masks the last column tile).
    if (stored_c(m, src) % 64 != 0 || stored_c(m, n) % 8 != 0) return false;
    if (n.k == 1 && n.pad == 0 && n.stride == 1) return true;
    if (n.k == 1 && n.pad == 0 && n.stride == 2) return src.H % 2 == 0 && src.W % 2 == 0;
    if (n.k == 3 && n.pad == 1 && n.stride == 1) return true;
    if (n.k == 3 && n.pad == 1 && n.stride == 2) return src.H % 2 == 0 && src.W % 2 == 0;
    // A filter that covers the whole feature map (the first dense layer of VGG): with plain rows
    // the (h, w, c) values of one image are contiguous, so the layer is a GEMM over [N][H*W*C].
    if (full_map_dense(n, src)) return (long long)n.k * n.k * stored_c(m, src) % 64 == 0;
    return false;
}

static int wanted_order(const Node &n) {
    if (n.k == 3 && n.stride == 1) return ACT_PADDED;
    if (n.k == 3 && n.stride == 2) return ACT_PHASED;
    return ACT_PLAIN;
}

static ActView view_of(const gpx_model &m, const Node &node) {
    const Storage &s = m.storages[node.storage];
    ActView v{};
    if (s.kind == Storage::InputF32) {
        v.f32 = s.dptr;
        v.l = make_layout(node.N, node.H, node.W, node.C, ACT_PLAIN);
    } else {
        v.hi = s.hi;
        v.lo = s.lo;
        v.l = s.layout;
    }
    return v;
}

// Largest tile of the memory-bound kernels, in 8-channel vectors.  A claimed tile always completes
// (scripts/compile/convert_to_blp.py:39-70), so the tile bounds the drain after a preemption: 2048
// vectors of the stem's 3x3 max pooling took 86 us, 256 keep every such kernel under ~10 us.
constexpr long long kMaxTileVectors = 256;

int finalize_model(gpx_model &m) {
    const DeviceInfo &d = device_info();
    GPX_REQUIRE(d.device >= 0, GPX_FAIL, "gpx_init was not called");
    m.device = d.device;
    m.sm_count = d.sm_count;
    const char *force = getenv("GPX_CONV");
    const bool allow_tc = !(force && std::string(force) == "simt");

    // 1. which convolutions can run on the tensor cores, judged by shape alone
    for (auto &n : m.nodes) {
        if (n.op != Op::Conv) continue;
        const Node &src = m.nodes[n.inputs[0]];
        const Storage &out = m.storages[n.storage];
        const Storage &in = m.storages[src.storage];
        n.tensor_core = allow_tc && tensor_core_shape(m, n, src) && in.kind == Storage::ActSplit &&
                        out.kind == Storage::ActSplit;
        // The graph head: a dense layer with any number of outputs written as fp32.
        if (allow_tc && out.kind == Storage::OutputF32 && in.kind == Storage::ActSplit && n.k == 1 &&
            n.stride == 1 && n.pad == 0 && src.H == 1 && src.W == 1 && stored_c(m, src) % 64 == 0)
            n.tensor_core = true;
        // Few input channels (the stem): build the patch matrix, then a 1x1 tensor-core GEMM.
        if (allow_tc && !n.tensor_core && out.kind == Storage::ActSplit && stored_c(m, n) % 64 == 0 &&
            in.kind == Storage::InputF32 && n.k * n.k * src.C <= 1024 && (!n.kw || n.kw == n.k) &&
            (n.pad_w < 0 || n.pad_w == n.pad)) {
            n.tensor_core = true;
            n.via_im2col = true;
            // A 7x7 stride-2 stem on at most four channels: instead of a patch matrix (308 MB at
            // batch 32) the input is rearranged once into 2x2 blocks of 16 channels, and every
            // block position stores the four consecutive blocks wb .. wb+3 (64 channels, 108 MB).
            // An output pixel then reads four block rows, each one 64-channel row of that tensor:
            // a four-tap row-shifted GEMM (K = 256) like the 3x3 convolutions.
            const char *e = getenv("GPX_STEM_S2D");
            if (n.k == 7 && !n.kw && n.stride == 2 && n.pad == 3 && src.C * 4 <= 16 && !(e && e[0] == '0'))
                n.via_s2d = true;
        }
        // Shapes the row-shift scheme does not take (one-sided 1x7 / 7x1 / 1x3 / 3x1 filters, 5x5,
        // unpadded or stride-2 3x3 on a plain input: Inception-v3): a patch matrix copied from the
        // planes, 16 bytes per tap and eight channels, then a 1x1 tensor-core GEMM.
        const char *e_pm = getenv("GPX_PATCH_GEMM");
        if (allow_tc && !n.tensor_core && out.kind == Storage::ActSplit && in.kind == Storage::ActSplit &&
            stored_c(m, n) % 64 == 0 && stored_c(m, src) % 8 == 0 && n.residual < 0 && !(e_pm && e_pm[0] == '0')) {
            n.tensor_core = true;
            n.via_im2col = true;
        }
    }
    // 2. row order of every activation: what its 3x3 tensor-core consumers need, if they agree
    std::vector<int> order(m.storages.size(), ACT_PLAIN);
    std::vector<int> votes(m.storages.size(), -1);
    std::vector<bool> conflict(m.storages.size(), false);
    for (auto &n : m.nodes) {
        if (n.op != Op::Conv || !n.tensor_core || n.k != 3 || n.via_im2col) continue;
        if (full_map_dense(n, m.nodes[n.inputs[0]])) continue;
        int st = m.nodes[n.inputs[0]].storage;
        int want = wanted_order(n);
        if (votes[st] >= 0 && votes[st] != want) conflict[st] = true;
        votes[st] = want;
    }
    for (size_t i = 0; i < m.storages.size(); ++i)
        if (votes[i] >= 0 && !conflict[i]) order[i] = votes[i];
    // 3. final decision given the layouts
    for (auto &n : m.nodes) {
        if (n.op != Op::Conv || !n.tensor_core || n.via_im2col) continue;
        int st = m.nodes[n.inputs[0]].storage;
        if (n.k == 3 && !full_map_dense(n, m.nodes[n.inputs[0]]) && order[st] != wanted_order(n)) n.tensor_core = false;
        if (n.k == 1 && order[st] == ACT_PHASED) n.tensor_core = false;
        if (n.k == 1 && n.stride == 2 && order[st] != ACT_PLAIN) n.tensor_core = false;
        if (full_map_dense(n, m.nodes[n.inputs[0]]) && order[st] != ACT_PLAIN) n.tensor_core = false;
        if (n.residual >= 0 && m.storages[m.nodes[n.residual].storage].kind != Storage::ActSplit)
            n.tensor_core = false;
    }
    // 4. compact copies for stride-2 1x1 convolutions (hidden storages)
    for (size_t ni = 0; ni < m.nodes.size(); ++ni) {
        Node &n = m.nodes[ni];
        if (n.op != Op::Conv || !n.tensor_core) continue;
        const bool sub2 = n.k == 1 && n.stride == 2 && !n.via_im2col;
        if (!sub2 && !n.via_im2col) continue;
        const Node &src = m.nodes[n.inputs[0]];
        Storage s;
        s.name = n.name + (n.via_im2col ? ".patches" : ".subsampled");
        s.kind = Storage::ActSplit;
        s.hidden = true;
        s.rank = 4;
        s.dims[0] = n.N;
        // Patch-matrix rows are padded to whole 16-byte vectors only: TMA zero-fills the rest of
        // the last 64-column K block, and the matrix (written once, read once) stays 21 % smaller
        // than with rows padded to 64 columns (7x7x3 = 147 -> 152 instead of 192).
        s.dims[1] = n.via_im2col ? (n.k * n.k * src.C + 7) / 8 * 8 : src.C;
        if (n.via_im2col && m.storages[src.storage].kind == Storage::ActSplit)
            s.dims[1] = (int64_t)n.k * (n.kw ? n.kw : n.k) * stored_c(m, src);
        s.dims[2] = n.H;
        s.dims[3] = n.W;
        if (n.via_s2d) {
            s.name = n.name + ".s2d";
            s.dims[1] = 64;
            s.dims[2] = (src.H + 2 * n.pad + 1) / 2;
            s.dims[3] = (src.W + 2 * n.pad + 1) / 2;
        }
        s.bytes = (size_t)n.N * s.dims[1] * s.dims[2] * s.dims[3] * sizeof(float);
        if (!n.via_im2col && stored_c(m, src) != src.C) s.cs = stored_c(m, src);
        n.sub_storage = m.add_storage(s);
        order.push_back(ACT_PLAIN);
    }
    for (auto &n : m.nodes)
        if (n.op == Op::DwConv) m.storages[n.weight].cin_pad = stored_c(m, n);
    for (auto &n : m.nodes)
        if (n.op == Op::Conv && n.tensor_core) {
            const Node &src = m.nodes[n.inputs[0]];
            Storage &w = m.storages[n.weight];
            w.wants_split = true;
            // rows of the planes: [tap][stored input channel], zero where the channel is padding
            // patch columns are [tap][channel]: the logical channels of an fp32 input, the stored ones of planes
            w.cin_pad = (n.via_im2col && m.storages[src.storage].kind == Storage::InputF32) ? src.C : stored_c(m, src);
            w.cout_pad = m.storages[n.storage].kind == Storage::OutputF32 ? n.C : (stored_c(m, n) + 63) / 64 * 64;
            w.split_k = (int)((w.dims[2] * w.dims[3] * w.cin_pad + 63) / 64 * 64);
            if (n.via_s2d) {
                w.s2d = true;
                w.split_k = 256;  // four block rows x four blocks x 16 channels
            }
        }

    // 5. allocation: one buffer per storage, zero-filled, no sharing (src/model.cpp:101-113)
    for (size_t i = 0; i < m.storages.size(); ++i) {
        Storage &s = m.storages[i];
        if (s.kind == Storage::ActSplit && s.parent >= 0) continue;  // a slice: bound below
        if (s.kind == Storage::ActSplit) {
            int N = (int)s.dims[0], C = s.cs ? s.cs : (int)s.dims[1];
            int H = s.rank == 4 ? (int)s.dims[2] : 1, W = s.rank == 4 ? (int)s.dims[3] : 1;
            GPX_REQUIRE(C % 8 == 0, GPX_FAIL, "%s: %d channels, need a multiple of 8", s.name.c_str(), C);
            s.layout = make_layout(N, H, W, C, order[i]);
            s.layout.fmt = m.fmt;
            s.plane_elems = (size_t)s.layout.rows * C;
            GPX_REQUIRE(s.plane_elems < 0xffffffffull, GPX_OUT_OF_RANGE, "%s: %zu elements per plane, the kernels index with 32 bits",
                        s.name.c_str(), s.plane_elems);
            GPX_CUDA(cudaMalloc((void **)&s.hi, plane_count(m.fmt) * s.plane_elems * sizeof(bf16_bits)));
            GPX_CUDA(cudaMemset(s.hi, 0, plane_count(m.fmt) * s.plane_elems * sizeof(bf16_bits)));
            s.lo = m.fmt == PF_SPLIT ? s.hi + s.plane_elems : nullptr;
        } else {
            // Rounded up to 512 bytes so a kernel may read a bias in whole 128-channel tiles.
            size_t alloc = (s.bytes + 511) / 512 * 512;
            // A depthwise filter is stored [kh*kw][stored channels].
            if (s.kind == Storage::Weight && s.depthwise)
                alloc = (size_t)s.dims[2] * s.dims[3] * s.cin_pad * sizeof(float);
            GPX_CUDA(cudaMalloc((void **)&s.dptr, alloc));
            GPX_CUDA(cudaMemset(s.dptr, 0, alloc));
            if (s.kind == Storage::Weight && s.wants_split) {
                s.plane_elems = (size_t)s.cout_pad * s.split_k;
                GPX_CUDA(cudaMalloc((void **)&s.hi, plane_count(m.fmt) * s.plane_elems * sizeof(bf16_bits)));
                GPX_CUDA(cudaMemset(s.hi, 0, plane_count(m.fmt) * s.plane_elems * sizeof(bf16_bits)));
                s.lo = m.fmt == PF_SPLIT ? s.hi + s.plane_elems : nullptr;
            }
        }
    }
    for (auto &s : m.storages) {
        if (s.kind != Storage::ActSplit || s.parent < 0) continue;
        const Storage &par = m.storages[s.parent];
        GPX_REQUIRE(par.parent < 0 && par.layout.order == ACT_PLAIN && s.ch_off % 8 == 0 && s.dims[1] % 8 == 0 &&
                        s.ch_off + s.dims[1] <= par.layout.C,
                    GPX_FAIL, "%s: bad slice of %s", s.name.c_str(), par.name.c_str());
        s.layout = par.layout;
        s.plane_elems = par.plane_elems;
        s.hi = par.hi + s.ch_off;
        s.lo = par.lo ? par.lo + s.ch_off : nullptr;
    }
    {
        // 128 x 128 identity in the plane format: the W operand of residual K blocks.
        std::vector<bf16_bits> eye(128 * 128, 0);
        const bf16_bits one = m.fmt == PF_F16 ? 0x3C00 : 0x3F80;
        for (int i = 0; i < 128; ++i) eye[i * 128 + i] = one;
        GPX_CUDA(cudaMalloc((void **)&m.identity, eye.size() * sizeof(bf16_bits)));
        GPX_CUDA(cudaMemcpy(m.identity, eye.data(), eye.size() * sizeof(bf16_bits), cudaMemcpyHostToDevice));
    }
    GPX_CUDA(cgemm_prepare(d.device));

    // 6. kernel list
    for (size_t ni = 0; ni < m.nodes.size(); ++ni) {
        const Node &n = m.nodes[ni];
        if (n.op == Op::Input || n.op == Op::Buffer) continue;
        const Node &src = m.nodes[n.inputs[0]];
        const Storage &out = m.storages[n.storage];
        auto add_pool = [&](const std::string &name, const ActView &in, const Storage &dst, int k,
                            int stride, int pad, int mode, int in_valid = -1, int scale = -1,
                            int shift = -1, int act = 0) {
            Kernel kn;
            kn.name = name;
            kn.node = (int)ni;
            kn.type = KernelType::Pool;
            PoolParams &p = kn.pool;
            p.in = in;
            p.out_hi = dst.hi;
            p.out_lo = dst.lo;
            p.out = dst.layout;
            p.k = k;
            p.stride = stride;
            p.pad = pad;
            p.mode = mode;
            p.channels = dst.parent >= 0 ? (int)dst.dims[1] : dst.layout.C;
            p.in_valid = in_valid >= 0 ? in_valid : std::min(p.channels, in.l.C);
            if (scale >= 0) {
                p.scale = m.storages[scale].dptr;
                p.shift = m.storages[shift].dptr;
                p.act = act;
            }
            long long total = (long long)dst.layout.N * dst.layout.H * dst.layout.W * (p.channels / 8);
            // Enough tiles to fill the GPU even when the tensor is small (global average pool).
            long long want_tiles = 4LL * m.sm_count;
            // the cap is per unit of work: a copy or an affine map reads one tap per vector, a 3x3
            // pooling nine
            const int taps_per_vec = mode == 2 ? 1 : k * k;
            const long long tile_cap = std::min<long long>(2048, std::max<long long>(kMaxTileVectors, 9 * kMaxTileVectors / taps_per_vec));
            p.tile_elems = (int)std::max<long long>(mode == 1 && k * k >= 16 ? 8 : 64,
                                                    std::min<long long>(tile_cap, total / want_tiles / 8 * 8));
            p.total_tiles = (int)((total + p.tile_elems - 1) / p.tile_elems);
            kn.total_tiles = p.total_tiles;
            kn.grid = pool_grid(p, m.sm_count);
            int taps = mode == 2 ? 1 : k * k;
            kn.flops = (double)total * 8 * taps;
            kn.bytes = 4.0 * ((double)total * 8 * (mode == 2 ? 1 : stride * stride) + (double)total * 8);
            m.kernels.push_back(kn);
        };
        if (n.op == Op::LayerNorm) {
            Kernel kn;
            kn.name = n.name;
            kn.node = (int)ni;
            kn.type = KernelType::LayerNorm;
            LayerNormParams &q = kn.ln;
            const Storage &in = m.storages[src.storage];
            GPX_REQUIRE(n.C % 8 == 0 && n.C <= 1024, GPX_FAIL, "%s: LayerNorm width %d unsupported",
                        n.name.c_str(), n.C);
            if (in.kind == Storage::InputI64) {
                GPX_REQUIRE(n.tables[0] >= 0, GPX_FAIL, "%s: token input without embedding tables", n.name.c_str());
                q.ids = reinterpret_cast<const long long *>(in.dptr);
                q.word = m.storages[n.tables[0]].dptr;
                q.pos = m.storages[n.tables[1]].dptr;
                q.type = n.tables[2] >= 0 ? m.storages[n.tables[2]].dptr : nullptr;
            } else {
                GPX_REQUIRE(in.kind == Storage::ActSplit && in.layout.order == ACT_PLAIN, GPX_FAIL,
                            "%s: LayerNorm needs a plain activation", n.name.c_str());
                q.in_hi = in.hi;
                q.in_lo = in.lo;
            }
            q.fmt = m.fmt;
            q.gamma = m.storages[n.weight].dptr;
            q.beta = m.storages[n.bias].dptr;
            if (out.kind == Storage::OutputF32) {
                q.out_f32 = out.dptr;
            } else {
                q.out_hi = out.hi;
                q.out_lo = out.lo;
            }
            q.rows = n.N * n.H * n.W;
            q.H = n.C;
            q.S = n.W;
            q.eps = 1e-12f;
            q.total_tiles = (q.rows + 7) / 8;
            kn.total_tiles = q.total_tiles;
            kn.grid = (int)std::min<long long>((long long)m.sm_count * 8, q.total_tiles);
            kn.flops = 8.0 * q.rows * q.H;
            kn.bytes = 8.0 * q.rows * q.H;
            m.kernels.push_back(kn);
            continue;
        }
        if (n.op == Op::Attention) {
            Kernel kn;
            kn.name = n.name;
            kn.node = (int)ni;
            kn.type = KernelType::Attention;
            kn.threads = 128;
            AttnParams &q = kn.attn;
            const Storage &sq = m.storages[m.nodes[n.inputs[0]].storage];
            const Storage &sk = m.storages[m.nodes[n.inputs[1]].storage];
            const Storage &sv = m.storages[m.nodes[n.inputs[2]].storage];
            GPX_REQUIRE(n.heads > 0 && n.C == n.heads * 64, GPX_FAIL, "%s: head dimension must be 64", n.name.c_str());
            q.fmt = m.fmt;
            q.q_hi = sq.hi;
            q.q_lo = sq.lo;
            q.k_hi = sk.hi;
            q.k_lo = sk.lo;
            q.v_hi = sv.hi;
            q.v_lo = sv.lo;
            q.out_hi = out.hi;
            q.out_lo = out.lo;
            q.B = n.N;
            q.S = n.W;
            q.heads = n.heads;
            q.ld = n.C;
            q.scale = 0.125f;  // 1 / sqrt(64)
            kn.flops = 4.0 * n.N * n.heads * (double)n.W * n.W * 64;
            kn.bytes = 4.0 * 4 * (double)n.N * n.W * n.C;
            const char *force_simt = getenv("GPX_ATTN");
            if (m.fmt != PF_SPLIT && !(force_simt && std::string(force_simt) == "simt")) {
                // Single-plane models: both products on the tensor cores.  The values are first
                // written with keys contiguous (the B operand of the second product).
                const size_t vt_elems = (size_t)n.N * n.heads * 64 * n.W;
                GPX_CUDA(cudaMalloc((void **)&q.vt, vt_elems * sizeof(bf16_bits)));
                GPX_CUDA(cudaMemset(q.vt, 0, vt_elems * sizeof(bf16_bits)));
                m.scratch.push_back(q.vt);
                const uint64_t rows = (uint64_t)n.N * n.W;
                GPX_TRY(make_tmap_2d_bf16(&q.tq, sq.hi, rows, (uint64_t)n.C, 128, 64));
                GPX_TRY(make_tmap_2d_bf16(&q.tk, sk.hi, rows, (uint64_t)n.C, 128, 64));
                GPX_TRY(make_tmap_2d_bf16(&q.tvt, q.vt, (uint64_t)n.N * n.heads * 64, (uint64_t)n.W, 64, 64));
                GPX_CUDA(attention_tc_prepare());
                Kernel kt = kn;
                kt.name = n.name + ".vt";
                kt.type = KernelType::TransposeV;
                kt.threads = 256;
                kt.total_tiles = n.N * n.heads * ((n.W + 63) / 64);
                kt.grid = (int)std::min<long long>((long long)m.sm_count * 8, kt.total_tiles);
                kt.flops = 0;
                kt.bytes = 2.0 * 2 * (double)n.N * n.W * n.C;
                kt.attn.total_tiles = kt.total_tiles;
                m.kernels.push_back(kt);
                kn.type = KernelType::AttentionTc;
                q.total_tiles = n.N * n.heads * ((n.W + 127) / 128);
                kn.total_tiles = q.total_tiles;
                kn.grid = (int)std::min<long long>((long long)m.sm_count * 2, q.total_tiles);
                m.kernels.push_back(kn);
                continue;
            }
            q.total_tiles = n.N * n.heads * ((n.W + 31) / 32);
            kn.total_tiles = q.total_tiles;
            kn.grid = (int)std::min<long long>((long long)m.sm_count * 4, q.total_tiles);
            m.kernels.push_back(kn);
            continue;
        }
        if (n.op == Op::DwConv) {
            GPX_REQUIRE(m.storages[src.storage].kind == Storage::ActSplit && out.kind == Storage::ActSplit,
                        GPX_FAIL, "%s: depthwise convolution needs plane activations", n.name.c_str());
            Kernel kn;
            kn.name = n.name;
            kn.node = (int)ni;
            kn.type = KernelType::DwConv;
            DwConvParams &q = kn.dw;
            q.in = view_of(m, src);
            q.w = m.storages[n.weight].dptr;
            q.bias = m.storages[n.bias].dptr;
            q.out_hi = out.hi;
            q.out_lo = out.lo;
            q.out = out.layout;
            GPX_REQUIRE(q.in.l.C == q.out.C, GPX_FAIL, "%s: channel counts differ", n.name.c_str());
            q.k = n.k;
            q.stride = n.stride;
            q.pad = n.pad;
            q.act = n.act;
            long long total = (long long)n.N * n.H * n.W * (q.out.C / 8);
            q.tile_elems = (int)std::max<long long>(256, std::min<long long>(kMaxTileVectors, total / (8LL * m.sm_count) / 32 * 32));
            q.total_tiles = (int)((total + q.tile_elems - 1) / q.tile_elems);
            kn.total_tiles = q.total_tiles;
            kn.grid = (int)std::min<long long>((long long)m.sm_count * 8, q.total_tiles);
            kn.flops = 2.0 * n.N * n.H * n.W * (double)n.k * n.k * n.C;
            kn.bytes = 4.0 * ((double)src.N * src.H * src.W * src.C + (double)n.N * n.H * n.W * n.C);
            m.kernels.push_back(kn);
            continue;
        }
        if (n.op == Op::Affine) {
            GPX_REQUIRE(m.storages[src.storage].kind == Storage::ActSplit && n.in_c % 8 == 0, GPX_FAIL,
                        "%s: affine needs a plane activation and a channel count in eights", n.name.c_str());
            add_pool(n.name, view_of(m, src), out, 1, 1, 0, 2, n.in_c, n.scale, n.shift, n.act);
            continue;
        }
        if (n.op != Op::Conv) {
            GPX_REQUIRE(m.storages[src.storage].kind == Storage::ActSplit, GPX_FAIL,
                        "%s: pooling the graph input is not supported", n.name.c_str());
            add_pool(n.name, view_of(m, src), out, n.k, n.stride, n.pad,
                     n.op == Op::MaxPool ? 0 : (n.count_pad ? 3 : 1), -1, n.scale, n.shift, n.act);
            continue;
        }
        const Storage &w = m.storages[n.weight];
        const int n_kw = n.kw ? n.kw : n.k;
        const double flops = 2.0 * n.N * n.H * n.W * (double)n.k * n_kw * src.C * n.C;
        const double bytes = 4.0 * ((double)src.N * src.H * src.W * src.C + (double)n.k * n_kw * src.C * n.C +
                                    (double)n.N * n.H * n.W * n.C * (n.residual >= 0 ? 2 : 1));
        if (!n.tensor_core) {
            Kernel kn;
            kn.name = n.name;
            kn.node = (int)ni;
            kn.type = KernelType::ConvSimt;
            GPX_REQUIRE(n.C % 4 == 0, GPX_FAIL, "%s: Cout %d not a multiple of 4", n.name.c_str(), n.C);
            ConvParams &p = kn.conv;
            p.in = view_of(m, src);
            p.w = w.dptr;
            p.bias = m.storages[n.bias].dptr;
            if (n.residual >= 0) p.res = view_of(m, m.nodes[n.residual]);
            if (out.kind == Storage::OutputF32) {
                GPX_REQUIRE(n.H == 1 && n.W == 1, GPX_FAIL, "%s: fp32 outputs must be [N][C]", n.name.c_str());
                p.out_f32 = out.dptr;
                p.out = make_layout(n.N, 1, 1, n.C, ACT_PLAIN);
            } else {
                p.out_hi = out.hi;
                p.out_lo = out.lo;
                p.out = out.layout;
            }
            p.Cin = src.C;
            p.Ho = n.H;
            p.Wo = n.W;
            p.Cout = n.C;
            p.kh = n.k;
            p.kw = n_kw;
            p.stride = n.stride;
            p.pad = n.pad;
            p.pad_w = n.pad_w >= 0 ? n.pad_w : n.pad;
            p.M = n.N * n.H * n.W;
            p.K = n.k * n_kw * src.C;
            p.relu = n.act;
            kn.tile = conv_pick_tile(p, m.sm_count);
            conv_set_tiles(p, kn.tile);
            kn.total_tiles = p.tiles_m * p.tiles_n;
            kn.grid = conv_grid(p, kn.tile, m.sm_count);
            kn.flops = flops;
            kn.bytes = bytes;
            m.kernels.push_back(kn);
            continue;
        }
        // A dense layer on at most eight rows: matrix-vector products on the CUDA cores, bound by
        // reading the weights once (GPX_DENSE_ROWS=0 keeps the tensor-core tile).
        {
            const char *e_dr = getenv("GPX_DENSE_ROWS");
            const bool one_pixel = n.k == 1 && n.stride == 1 && n.pad == 0 && src.H == 1 && src.W == 1;
            const bool dense = one_pixel || full_map_dense(n, src);
            const Storage &in0 = m.storages[src.storage];
            const int k_len = (one_pixel ? 1 : n.k * n.k) * stored_c(m, src);
            if (dense && !n.via_im2col && n.N <= 8 && n.residual < 0 && in0.kind == Storage::ActSplit &&
                in0.layout.order == ACT_PLAIN && k_len % 8 == 0 && !(e_dr && e_dr[0] == '0')) {
                const Storage &w = m.storages[n.weight];
                const bool head = out.kind == Storage::OutputF32;
                Kernel kd;
                kd.name = n.name;
                kd.node = (int)ni;
                kd.type = KernelType::DenseRows;
                DenseRowsParams &q = kd.dense;
                q.a_hi = in0.hi;
                q.a_lo = in0.lo;
                q.a_ld = src.H * src.W * stored_c(m, src);
                q.w_hi = w.hi;
                q.w_lo = w.lo;
                q.w_ld = w.split_k;
                q.bias = m.storages[n.bias].dptr;
                q.M = n.N;
                q.K = k_len;
                q.cout = head ? n.C : stored_c(m, n);
                q.relu = n.act;
                q.fmt = m.fmt;
                if (head) {
                    q.out_f32 = out.dptr;
                } else {
                    q.out_hi = out.hi;
                    q.out_lo = out.lo;
                    q.out_ld = out.layout.C;
                }
                q.total_tiles = (q.cout + 7) / 8;
                kd.total_tiles = q.total_tiles;
                kd.grid = (int)std::min<long long>((long long)m.sm_count * 8, q.total_tiles);
                kd.flops = flops;
                kd.bytes = bytes;
                m.kernels.push_back(kd);
                continue;
            }
        }
        // tensor-core convolution
        const Storage *in = &m.storages[src.storage];
        int eff_k = n.k, eff_cin = stored_c(m, src);
        if (n.via_im2col) {
            const Storage &pm = m.storages[n.sub_storage];
            Kernel ki;
            ki.name = n.name + ".im2col";
            ki.node = (int)ni;
            ki.type = KernelType::Im2col;
            Im2colParams &q = ki.im2col;
            q.in = view_of(m, src);
            q.out_hi = pm.hi;
            q.out_lo = pm.lo;
            q.fmt = m.fmt;
            q.Cin = src.C;
            q.Ho = n.H;
            q.Wo = n.W;
            q.kh = q.kw = n.k;
            q.stride = n.stride;
            q.pad = n.pad;
            q.K = n.k * n.k * src.C;
            q.Kp = (int)pm.dims[1];
            q.M = n.N * n.H * n.W;
            if (m.storages[src.storage].kind == Storage::ActSplit) {
                ki.name = n.name + ".patches";
                q.planes_vec = 1;
                q.kh = n.k;
                q.kw = n.kw ? n.kw : n.k;
                q.pad_w = n.pad_w >= 0 ? n.pad_w : n.pad;
                q.K = q.Kp;
            }
            if (n.via_s2d) {
                ki.name = n.name + ".s2d";
                q.s2d = 1;
                q.Ho = (int)pm.dims[2];
                q.Wo = (int)pm.dims[3];
                q.M = n.N * q.Ho * q.Wo;
                q.Kp = 64;
            }
            long long total = (long long)q.M * (q.Kp / 8);
            if (n.via_s2d) total = (long long)n.N * q.Ho * (q.Wo + 3) * 2;  // half blocks, each stored up to four times
            // (twice the usual cap: a patch-matrix tile re-reads its lookup table, ~5 us per 256 vectors)
            q.tile_elems = (int)std::max<long long>(256, std::min<long long>(2 * kMaxTileVectors, total / (8LL * m.sm_count) / 32 * 32));
            q.total_tiles = (int)((total + q.tile_elems - 1) / q.tile_elems);
            {
                // fp32 NCHW input: tiles of up to 64 output pixels of one output row, staged window
                const char *off = getenv("GPX_IM2COL_WINDOW");
                const int chunks = (n.W + 63) / 64;
                const int win_w = (n.W + chunks - 1) / chunks;
                const long long window = (long long)src.C * n.k * ((win_w - 1) * n.stride + n.k);
                if (m.storages[src.storage].kind == Storage::InputF32 && window <= kIm2colWindowFloats &&
                    !(off && off[0] == '0') && !n.via_s2d) {
                    q.win_w = win_w;
                    q.win_chunks = chunks;
                    q.total_tiles = n.N * n.H * chunks;
                }
            }
            ki.total_tiles = q.total_tiles;
            ki.grid = (int)std::min<long long>((long long)m.sm_count * 8, q.total_tiles);
            ki.flops = 0;
            ki.bytes = 4.0 * (double)src.N * src.H * src.W * src.C + 4.0 * (double)q.M * q.Kp;
            m.kernels.push_back(ki);
            in = &pm;
            eff_k = 1;
            eff_cin = n.via_s2d ? 64 : q.Kp;
        } else if (n.k == 1 && n.stride == 2) {
            const Storage &sub = m.storages[n.sub_storage];
            add_pool(n.name + ".subsample", view_of(m, src), sub, 1, 2, 0, 2);
            in = &sub;
        }
        Kernel kn;
        kn.name = n.name;
        kn.node = (int)ni;
        kn.type = KernelType::Cgemm;
        kn.threads = cgemm_threads();
        CgemmParams &p = kn.cgemm;
        ActLayout il = in->layout;
        if (full_map_dense(n, src) && !n.via_im2col) {
            // one GEMM row per image, K = (h, w, c) in the stored order
            eff_cin = n.k * n.k * stored_c(m, src);
            eff_k = 1;
            il = make_layout(n.N, 1, 1, eff_cin, ACT_PLAIN);
        }
        const bool head = out.kind == Storage::OutputF32;
        const int cout_st = head ? n.C : stored_c(m, n);  // output channels as stored
        int bn = (cout_st % 128 == 0 || head) ? 128 : 64;
        {
            // Few output tiles (batch 1, late stages): narrower column tiles expose more CTAs.
            long long tiles128 = (long long)((il.plane + 127) / 128) * ((cout_st + 127) / 128);
            if (tiles128 * 2 <= m.sm_count) bn = 64;
            // Single-plane operands do one product per K step, so a 128x128 tile cannot be fed
            // fast enough (32 KB of TMA fill per 0.13 us of products): 256-column tiles halve the
            // activation bytes per product, as the stand-alone GEMM's 128x256 tiles do, wherever
            // they still fill the GPU and the K loop is long enough to outweigh the second
            // accumulator buffer they give up (ResNet-50's 1x1 convolutions with K <= 512 lose 6 %,
            // BERT's dense layers and VGG's 3x3 convolutions gain 17-19 %).
            const char *wide = getenv("GPX_CGEMM_BN256");
            const bool try_split = wide && wide[0] == 's';  // experiment: 256-column tiles for two-plane operands
            if ((m.fmt != PF_SPLIT || try_split) && !head && cout_st % 256 == 0 && tiles128 / 2 >= m.sm_count &&
                (long long)eff_k * eff_k * eff_cin >= 768 &&
                !(wide && wide[0] == '0'))
                bn = 256;
        }
        kn.tile = bn;
        p.taps = eff_k * eff_k;
        p.cin = eff_cin;
        p.cin_blocks = (eff_cin + 63) / 64;
        for (int t = 0; t < 9; ++t) p.tap_shift[t] = 0;
        if (n.via_s2d) {
            // four block rows; the four blocks of a row are the 64 channels of one stored pixel
            p.taps = 4;
            for (int t = 0; t < 4; ++t) p.tap_shift[t] = t * il.Ws;
        }
        if (eff_k == 3) {
            for (int fh = 0; fh < 3; ++fh)
                for (int fw = 0; fw < 3; ++fw) {
                    int t = fh * 3 + fw;
                    if (n.stride == 1)
                        p.tap_shift[t] = (fh - 1) * il.Ws + (fw - 1);
                    else
                        p.tap_shift[t] = (((fh & 1) << 1) | (fw & 1)) * il.plane + (fh >> 1) * il.Ws + (fw >> 1);
                }
        }
        p.m_rows = il.plane;
        p.in_hs = il.Hs;
        p.in_ws = il.Ws;
        p.in_off = il.order == ACT_PADDED ? 1 : 0;
        p.tiles_m = (p.m_rows + 127) / 128;
        p.tiles_n = (cout_st + bn - 1) / bn;
        p.cout_valid = cout_st;
        p.relu = n.act;
        p.bias = m.storages[n.bias].dptr;
        if (n.residual >= 0) {
            const Storage &r = m.storages[m.nodes[n.residual].storage];
            p.res_hi = r.hi;
            p.res_lo = r.lo;
            p.res = r.layout;
        }
        if (head) {
            p.out_f32 = out.dptr;
            p.out = make_layout(n.N, n.H, n.W, n.C, ACT_PLAIN);
        } else {
            p.out_hi = out.hi;
            p.out_lo = out.lo;
            p.out = out.layout;
        }
        // The epilogue moves 32 bytes per access: 16-channel granularity of rows and slices.
        GPX_REQUIRE(head || (out.layout.C % 16 == 0 && out.ch_off % 16 == 0), GPX_FAIL,
                    "%s: output channels %d (+%d) not in whole 16-channel groups", n.name.c_str(), out.layout.C, out.ch_off);
        GPX_TRY(make_tmap_2d_bf16(&p.a_hi, in->hi, (uint64_t)il.rows, (uint64_t)eff_cin, 128, 64));
        if (in->lo) GPX_TRY(make_tmap_2d_bf16(&p.a_lo, in->lo, (uint64_t)il.rows, (uint64_t)eff_cin, 128, 64));
        GPX_TRY(make_tmap_2d_bf16(&p.w_hi, w.hi, (uint64_t)w.cout_pad, (uint64_t)w.split_k, bn, 64));
        if (w.lo) GPX_TRY(make_tmap_2d_bf16(&p.w_lo, w.lo, (uint64_t)w.cout_pad, (uint64_t)w.split_k, bn, 64));
        p.fmt = m.fmt;
        // Split K when the output alone cannot fill the GPU: each split gets at least four K
        // blocks, the finishing kernel adds the splits in order.
        const int all_kb = p.taps * p.cin_blocks;
        const int out_tiles = p.tiles_m * p.tiles_n;
        p.k_splits = 1;
        p.kb_per_split = all_kb;
        // (GPX_SPLITK_MIN_KB: fewest K blocks per split, default 4; GPX_SPLITK_ALLKB: shortest K loop
        // that is split at all, default 8 - tuning knobs for the batch-1 latency.)
        const char *e_min = getenv("GPX_SPLITK_MIN_KB"), *e_all = getenv("GPX_SPLITK_ALLKB");
        const int min_kb = e_min ? std::max(1, atoi(e_min)) : 4;
        const int split_from = e_all ? atoi(e_all) : 8;
        if (out_tiles * 2 <= m.sm_count && all_kb >= split_from) {
            int s_want = std::min(all_kb / min_kb, m.sm_count / out_tiles);
            // Powers of two up to eight: the splits of an output block can then form a thread-block
            // cluster and reduce through distributed shared memory (non-preemptible launches).
            const char *e_cl = getenv("GPX_SPLITK_CLUSTER");
            if (!(e_cl && e_cl[0] == '0')) s_want = s_want >= 8 ? 8 : (s_want >= 4 ? 4 : (s_want >= 2 ? 2 : 1));
            if (s_want >= 2) {
                p.kb_per_split = (all_kb + s_want - 1) / s_want;
                p.k_splits = (all_kb + p.kb_per_split - 1) / p.kb_per_split;
            }
        }
        // Two accumulators per tile (hi*hi; both cross terms) in two TMEM buffers: the epilogue of one
        // tile overlaps the K loop of the next.  The single hi*hi chain costs at most 9e-6 of
        // truncation bias on the longest K range (4608) and keeps ResNet-50 b32 at 3.8e-5 of the
        // 1e-4 layer bound; GPX_CGEMM_DUAL=0 selects four accumulators in one buffer (even / odd
        // K steps, hi*lo, lo*hi), =1 uses that plan only for chains longer than 1024 products.
        p.dual = 1;
        if (const char *e = getenv("GPX_CGEMM_DUAL")) {
            if (atoi(e) == 0) p.dual = 0;
            if (atoi(e) == 1) p.dual = (m.fmt != PF_SPLIT || p.kb_per_split * 64 <= 1024) ? 1 : 0;
        }
        if (bn == 256) p.dual = 1;  // the only plan that fits 256-column tiles in tensor memory
        {
            const char *e = getenv("GPX_CGEMM_PACKED");
            p.packed = (bn <= 128 && !(e && e[0] == '0')) ? 1 : 0;
        }
        // The residual of a 1x1 stride-1 convolution on plain rows has the rows of the GEMM itself:
        // it is then added by the tensor core as identity K blocks instead of by the epilogue.
        p.res_kb = 0;
        if (n.residual >= 0 && p.k_splits == 1 && eff_k == 1 && !n.via_im2col && in == &m.storages[src.storage] &&
            il.order == ACT_PLAIN && !getenv("GPX_CGEMM_RES_EPILOGUE")) {
            const Storage &r = m.storages[m.nodes[n.residual].storage];
            if (r.layout.order == ACT_PLAIN && r.layout.rows == il.rows && r.parent < 0 && r.layout.C % 64 == 0) {
                GPX_TRY(make_tmap_2d_bf16(&p.r_hi, r.hi, (uint64_t)r.layout.rows, (uint64_t)r.layout.C, 128, 64));
                if (r.lo) GPX_TRY(make_tmap_2d_bf16(&p.r_lo, r.lo, (uint64_t)r.layout.rows, (uint64_t)r.layout.C, 128, 64));
                GPX_TRY(make_tmap_2d_bf16(&p.ident, m.identity, 128, 128, 64, 64));
                p.res_kb = bn / 64;
                p.res_hi = p.res_lo = nullptr;
            }
        }
        p.inv_k_splits = 1.0f / (float)p.k_splits;
        p.inv_tiles_n = 1.0f / (float)p.tiles_n;
        p.inv_img = 1.0f / (float)(p.in_hs * p.in_ws);
        p.inv_in_ws = 1.0f / (float)p.in_ws;
        // (the float quotient of fast_div is exact to within one below 2^24)
        GPX_REQUIRE((long long)p.tiles_m * 128 < (1 << 24) && (long long)out_tiles * p.k_splits < (1 << 24), GPX_OUT_OF_RANGE,
                    "%s: %d rows exceed what the tensor-core kernel indexes", n.name.c_str(), p.m_rows);
        {
            const Storage *res_st = n.residual >= 0 ? &m.storages[m.nodes[n.residual].storage] : nullptr;
            const bool res_plain = !res_st || (res_st->layout.order == ACT_PLAIN && res_st->layout.rows == il.rows);
            p.identity_rows = (!head && il.order == ACT_PLAIN && out.layout.order == ACT_PLAIN &&
                               out.layout.rows == il.rows && p.in_off == 0 && res_plain && !(full_map_dense(n, src) && !n.via_im2col))
                                  ? 1 : 0;
        }
        kn.total_tiles = out_tiles * p.k_splits;
        kn.grid = std::min(kn.total_tiles, m.sm_count);
        m.max_cgemm_grid = std::max(m.max_cgemm_grid, kn.grid);
        kn.flops = flops;
        kn.bytes = bytes;
        if (p.k_splits == 1) {
            m.kernels.push_back(kn);
            continue;
        }
        p.partial_rows = p.tiles_m * 128;
        p.partial_ld = p.tiles_n * bn;
        m.max_partial_floats = std::max(m.max_partial_floats,
                                        (size_t)p.k_splits * p.partial_rows * p.partial_ld);
        Kernel kf;
        kf.name = n.name + ".finish";
        kf.node = (int)ni;
        kf.type = KernelType::SplitK;
        SplitKParams &q = kf.splitk;
        q.k_splits = p.k_splits;
        q.partial_rows = p.partial_rows;
        q.partial_ld = p.partial_ld;
        q.m_rows = p.m_rows;
        q.in_hs = p.in_hs;
        q.in_ws = p.in_ws;
        q.in_off = p.in_off;
        q.relu = p.relu;
        q.bias = p.bias;
        q.res_hi = p.res_hi;
        q.res_lo = p.res_lo;
        q.res = p.res;
        q.out_hi = p.out_hi;
        q.out_lo = p.out_lo;
        q.out = p.out;
        q.out_f32 = p.out_f32;
        q.cout_valid = p.cout_valid;
        q.cout_padded = (p.cout_valid + 7) / 8 * 8;
        q.tile_elems = 256;
        long long total = (long long)q.m_rows * (q.cout_padded / 8);
        q.total_tiles = (int)((total + q.tile_elems - 1) / q.tile_elems);
        kf.total_tiles = q.total_tiles;
        kf.grid = (int)std::min<long long>((long long)m.sm_count * 8, q.total_tiles);
        kf.flops = 0;
        kf.bytes = 4.0 * p.k_splits * (double)q.m_rows * q.cout_padded;
        // In the GEMM kernel itself the epilogue only writes partial sums.
        p.bias = nullptr;
        p.res_hi = p.res_lo = nullptr;
        p.relu = 0;
        {
            // Eligible for the cluster reduction (which executors use it: executor.cu): a power-of-two
            // number of splits that divides the tile's rows, and every cluster resident at once.
            const char *e_cl = getenv("GPX_SPLITK_CLUSTER");
            const bool pow2 = p.k_splits == 2 || p.k_splits == 4 || p.k_splits == 8;
            if (pow2 && bn <= 128 && !(e_cl && e_cl[0] == '0') && cgemm_max_cluster(bn, p.k_splits) >= kn.total_tiles &&
                kn.grid == kn.total_tiles) {
                p.cluster_reduce = 1;
                p.fin = q;
                kf.fused_into_prev = true;
            }
        }
        m.kernels.push_back(kn);
        m.kernels.push_back(kf);
    }
    return GPX_SUCC;
}

// ---- conversions between canonical tensors (NCHW / OIHW fp32) and device layouts -------------

static void oihw_to_khwc_o(const float *src, float *dst, int O, int I, int KH, int KW) {
    for (int o = 0; o < O; ++o)
        for (int i = 0; i < I; ++i)
            for (int h = 0; h < KH; ++h)
                for (int w = 0; w < KW; ++w)
                    dst[(((size_t)h * KW + w) * I + i) * O + o] =
                        src[(((size_t)o * I + i) * KH + h) * KW + w];
}
static void khwc_o_to_oihw(const float *src, float *dst, int O, int I, int KH, int KW) {
    for (int o = 0; o < O; ++o)
        for (int i = 0; i < I; ++i)
            for (int h = 0; h < KH; ++h)
                for (int w = 0; w < KW; ++w)
                    dst[(((size_t)o * I + i) * KH + h) * KW + w] =
                        src[(((size_t)h * KW + w) * I + i) * O + o];
}

static int storage_set(gpx_model *m, Storage &s, const void *host, size_t len, cudaStream_t st) {
    // Model::set, src/model.cpp:313-321: `len < size` is rejected.
    GPX_REQUIRE(len >= s.bytes, GPX_OUT_OF_RANGE, "set %s: %zu bytes given, %zu needed",
                s.name.c_str(), len, s.bytes);
    const float *src = (const float *)host;
    if (s.kind == Storage::InputF32 || s.kind == Storage::OutputF32 || s.kind == Storage::Vec ||
        s.kind == Storage::InputI64 || s.kind == Storage::Table) {
        GPX_CUDA(cudaMemcpyAsync(s.dptr, host, s.bytes, cudaMemcpyHostToDevice, st));
        return GPX_SUCC;
    }
    if (s.kind == Storage::Weight) {
        const int O = (int)s.dims[0], I = (int)s.dims[1], KH = (int)s.dims[2], KW = (int)s.dims[3];
        if (s.depthwise) {
            // [C][1][kh][kw] -> [tap][stored channels], zero where the channel is padding
            std::vector<float> dw((size_t)KH * KW * s.cin_pad, 0.f);
            for (int c = 0; c < O; ++c)
                for (int t = 0; t < KH * KW; ++t) dw[(size_t)t * s.cin_pad + c] = src[(size_t)c * KH * KW + t];
            GPX_CUDA(cudaMemcpyAsync(s.dptr, dw.data(), dw.size() * sizeof(float), cudaMemcpyHostToDevice, st));
            GPX_CUDA(cudaStreamSynchronize(st));
            return GPX_SUCC;
        }
        std::vector<float> tmp(s.bytes / sizeof(float));
        oihw_to_khwc_o(src, tmp.data(), O, I, KH, KW);
        GPX_CUDA(cudaMemcpyAsync(s.dptr, tmp.data(), s.bytes, cudaMemcpyHostToDevice, st));
        GPX_CUDA(cudaStreamSynchronize(st));
        if (s.wants_split) {
            // [Cout][tap][Cin] hi/lo planes for the tensor-core kernel
            const int fmt = m->fmt;
            std::vector<bf16_bits> planes(plane_count(fmt) * s.plane_elems, 0);
            const size_t K = (size_t)s.split_k;  // rows are zero-padded to a multiple of 64
            for (int o = 0; o < O; ++o)
                for (int h = 0; h < KH; ++h)
                    for (int w = 0; w < KW; ++w)
                        for (int i = 0; i < I; ++i) {
                            float v = src[(((size_t)o * I + i) * KH + h) * KW + w];
                            size_t off = (size_t)o * K + ((size_t)h * KW + w) * s.cin_pad + i;
                            // space-to-depth order: block row h/2, block w/2, channel ((h&1)*2 + (w&1))*I + i
                            if (s.s2d) off = (size_t)o * K + (size_t)(h >> 1) * 64 + (size_t)(w >> 1) * 16 + (((h & 1) << 1) | (w & 1)) * I + i;
                            host_put(planes, s.plane_elems, off, v, fmt);
                        }
            GPX_CUDA(cudaMemcpyAsync(s.hi, planes.data(), planes.size() * sizeof(bf16_bits),
                                     cudaMemcpyHostToDevice, st));
            GPX_CUDA(cudaStreamSynchronize(st));
        }
        return GPX_SUCC;
    }
    // ActSplit: NCHW fp32 -> hi/lo planes in the storage's row order (borders stay zero)
    const ActLayout &l = s.layout;
    if (s.parent >= 0) {
        // A channel slice: patch the owning tensor's planes.
        Storage &par = m->storages[s.parent];
        std::vector<bf16_bits> pl(plane_count(l.fmt) * par.plane_elems);
        GPX_CUDA(cudaMemcpyAsync(pl.data(), par.hi, pl.size() * sizeof(bf16_bits), cudaMemcpyDeviceToHost, st));
        GPX_CUDA(cudaStreamSynchronize(st));
        const int C = (int)s.dims[1];
        for (int n = 0; n < l.N; ++n)
            for (int c = 0; c < C; ++c)
                for (int h = 0; h < l.H; ++h)
                    for (int w = 0; w < l.W; ++w) {
                        float v = src[(((size_t)n * C + c) * l.H + h) * l.W + w];
                        size_t off = (size_t)layout_row(l, n, h, w) * l.C + s.ch_off + c;
                        host_put(pl, par.plane_elems, off, v, l.fmt);
                    }
        GPX_CUDA(cudaMemcpyAsync(par.hi, pl.data(), pl.size() * sizeof(bf16_bits), cudaMemcpyHostToDevice, st));
        GPX_CUDA(cudaStreamSynchronize(st));
        return GPX_SUCC;
    }
    std::vector<bf16_bits> planes(plane_count(l.fmt) * s.plane_elems, 0);
    if (s.token_major) {
        const size_t total = (size_t)l.N * l.W * l.C;
        for (size_t i = 0; i < total; ++i) host_put(planes, s.plane_elems, i, src[i], l.fmt);
    } else
    for (int n = 0; n < l.N; ++n)
        for (int c = 0; c < (int)s.dims[1]; ++c)  // logical channels; stored padding stays zero
            for (int h = 0; h < l.H; ++h)
                for (int w = 0; w < l.W; ++w) {
                    float v = src[(((size_t)n * s.dims[1] + c) * l.H + h) * l.W + w];
                    size_t off = (size_t)layout_row(l, n, h, w) * l.C + c;
                    host_put(planes, s.plane_elems, off, v, l.fmt);
                }
    GPX_CUDA(cudaMemcpyAsync(s.hi, planes.data(), planes.size() * sizeof(bf16_bits),
                             cudaMemcpyHostToDevice, st));
    GPX_CUDA(cudaStreamSynchronize(st));
    return GPX_SUCC;
}

static int storage_get(gpx_model *m, Storage &s, void *host, size_t len, cudaStream_t st) {
    // Model::get, src/model.cpp:296-305.
    GPX_REQUIRE(len >= s.bytes, GPX_OUT_OF_RANGE, "get %s: %zu bytes given, %zu needed",
                s.name.c_str(), len, s.bytes);
    float *dst = (float *)host;
    if (s.kind == Storage::InputF32 || s.kind == Storage::OutputF32 || s.kind == Storage::Vec ||
        s.kind == Storage::InputI64 || s.kind == Storage::Table) {
        GPX_CUDA(cudaMemcpyAsync(host, s.dptr, s.bytes, cudaMemcpyDeviceToHost, st));
        return GPX_SUCC;
    }
    if (s.kind == Storage::Weight) {
        if (s.depthwise) {
            const int C = (int)s.dims[0], T = (int)(s.dims[2] * s.dims[3]);
            std::vector<float> dw((size_t)T * s.cin_pad);
            GPX_CUDA(cudaMemcpyAsync(dw.data(), s.dptr, dw.size() * sizeof(float), cudaMemcpyDeviceToHost, st));
            GPX_CUDA(cudaStreamSynchronize(st));
            for (int c = 0; c < C; ++c)
                for (int t = 0; t < T; ++t) dst[(size_t)c * T + t] = dw[(size_t)t * s.cin_pad + c];
            return GPX_SUCC;
        }
        std::vector<float> tmp(s.bytes / sizeof(float));
        GPX_CUDA(cudaMemcpyAsync(tmp.data(), s.dptr, s.bytes, cudaMemcpyDeviceToHost, st));
        GPX_CUDA(cudaStreamSynchronize(st));
        khwc_o_to_oihw(tmp.data(), dst, (int)s.dims[0], (int)s.dims[1], (int)s.dims[2], (int)s.dims[3]);
        return GPX_SUCC;
    }
    const ActLayout &l = s.layout;
    const Storage &own = s.parent >= 0 ? m->storages[s.parent] : s;  // who holds the planes
    const int coff = s.parent >= 0 ? s.ch_off : 0;
    std::vector<bf16_bits> planes(plane_count(l.fmt) * s.plane_elems);
    GPX_CUDA(cudaMemcpyAsync(planes.data(), own.hi, planes.size() * sizeof(bf16_bits),
                             cudaMemcpyDeviceToHost, st));
    GPX_CUDA(cudaStreamSynchronize(st));
    if (s.token_major) {
        // [N][S][C]: the stored rows in order
        const size_t total = (size_t)l.N * l.W * l.C;
        for (size_t i = 0; i < total; ++i)
            dst[i] = host_take(planes, s.plane_elems, i, l.fmt);
        return GPX_SUCC;
    }
    for (int n = 0; n < l.N; ++n)
        for (int h = 0; h < l.H; ++h)
            for (int w = 0; w < l.W; ++w) {
                size_t row = (size_t)layout_row(l, n, h, w) * l.C + coff;
                for (int c = 0; c < (int)s.dims[1]; ++c)
                    dst[(((size_t)n * s.dims[1] + c) * l.H + h) * l.W + w] =
                        host_take(planes, s.plane_elems, row + c, l.fmt);
            }
    return GPX_SUCC;
}

static const char kParamMagic[] = "TVM_MODEL_PARAMS";  // 17 bytes with the NUL, as the reference reads

}  // namespace gpx

extern "C" {

int gpx_synth_normal(float *host, size_t n, uint64_t seed, uint64_t stream, float mean,
                     float std) {
    GPX_REQUIRE(host || n == 0, GPX_FAIL, "host is NULL");
    normal_fill(host, n, seed, stream, mean, std);
    return GPX_SUCC;
}

int gpx_synth_uniform(float *host, size_t n, uint64_t seed, uint64_t stream, float lo, float hi) {
    GPX_REQUIRE(host || n == 0, GPX_FAIL, "host is NULL");
    uniform_fill(host, n, seed, stream, lo, hi);
    return GPX_SUCC;
}

int gpx_model_open(const char *name, const gpx_model_opts *opts, gpx_model **out) {
    GPX_REQUIRE(name && out, GPX_FAIL, "NULL argument");
    gpx_model_opts o{};
    if (opts) o = *opts;
    std::unique_ptr<gpx_model> m(new gpx_model());
    std::string nm(name);
    // A directory holding mod.json + host.json (+ mod.params), the layout the reference loads
    // (MODEL_PATH/<workload>/..., src/executor.cpp:110-117), or the name of a built-in graph.
    const bool from_dir = model_dir_exists(nm);
    if (from_dir) {
        GPX_TRY(build_graph_from_dir(*m, nm, o));
    } else {
        // Aliases for the model names the reference's task configs use (config/A.json, C.json).
        if (nm == "resnet") nm = "resnet152";
        GPX_TRY(build_builtin_graph(*m, nm, o));
    }
    int st = m->sci ? GPX_SUCC : finalize_model(*m);
    if (st == GPX_SUCC && from_dir) st = check_host_json(*m, nm);
    if (st == GPX_SUCC && from_dir) {
        // Parameters travel with the directory (Executor::load_param, src/executor.cpp:115-117).
        const std::string params = nm + "/mod.params";
        if (FILE *fp = fopen(params.c_str(), "rb")) {
            fclose(fp);
            st = gpx_model_load_params(m.get(), params.c_str());
        }
    }
    if (st != GPX_SUCC) {
        std::string saved = last_error();
        gpx_model_close(m.release());
        set_error("%s", saved.c_str());
        return st;
    }
    *out = m.release();
    return GPX_SUCC;
}

int gpx_model_close(gpx_model *m) {
    if (!m) return GPX_SUCC;
    for (auto &s : m->storages) {
        if (s.dptr) cudaFree(s.dptr);
        if (s.hi && s.parent < 0) cudaFree(s.hi);  // lo lives in the same allocation; slices own nothing
    }
    if (m->identity) cudaFree(m->identity);
    for (void *ptr : m->scratch) cudaFree(ptr);
    delete m;
    return GPX_SUCC;
}

int gpx_model_storage_num(gpx_model *m, size_t *n) {
    GPX_REQUIRE(m && n, GPX_FAIL, "NULL argument");
    *n = m->storages.size();
    return GPX_SUCC;
}

int gpx_model_storage_info(gpx_model *m, size_t idx, char *name, size_t name_cap, size_t *bytes,
                           char *stype, size_t stype_cap, int *is_param) {
    GPX_REQUIRE(m, GPX_FAIL, "NULL model");
    GPX_REQUIRE(idx < m->storages.size(), GPX_OUT_OF_RANGE, "storage index %zu out of range", idx);
    const Storage &s = m->storages[idx];
    if (name && name_cap) snprintf(name, name_cap, "%s", s.name.c_str());
    if (bytes) *bytes = s.bytes;
    if (stype && stype_cap) snprintf(stype, stype_cap, "%s", s.stype.c_str());
    if (is_param) *is_param = s.is_param ? 1 : 0;
    return GPX_SUCC;
}

int gpx_model_find(gpx_model *m, const char *name, size_t *idx) {
    GPX_REQUIRE(m && name && idx, GPX_FAIL, "NULL argument");
    int i = m->find(name);
    if (i < 0) {
        set_error("storage '%s' not found", name);
        return GPX_NOT_FOUND;
    }
    *idx = (size_t)i;
    return GPX_SUCC;
}

int gpx_model_set(gpx_model *m, const char *name, const void *host, size_t len, gpx_stream s) {
    GPX_REQUIRE(m && name && host, GPX_FAIL, "NULL argument");
    int i = m->find(name);
    if (i < 0) {
        set_error("storage '%s' not found", name);
        return GPX_NOT_FOUND;
    }
    return storage_set(m, m->storages[i], host, len, as_stream(s));
}

int gpx_model_get(gpx_model *m, const char *name, void *host, size_t len, gpx_stream s) {
    GPX_REQUIRE(m && name && host, GPX_FAIL, "NULL argument");
    int i = m->find(name);
    if (i < 0) {
        set_error("storage '%s' not found", name);
        return GPX_NOT_FOUND;
    }
    return storage_get(m, m->storages[i], host, len, as_stream(s));
}

int gpx_model_shape(gpx_model *m, const char *name, int64_t dims[4], int *rank) {
    GPX_REQUIRE(m && name && dims && rank, GPX_FAIL, "NULL argument");
    int i = m->find(name);
    if (i < 0) {
        set_error("storage '%s' not found", name);
        return GPX_NOT_FOUND;
    }
    const Storage &s = m->storages[i];
    if (s.token_major) {
        // sequence activations are reported as [N][S][C]
        *rank = 3;
        dims[0] = s.dims[0];
        dims[1] = s.dims[3];
        dims[2] = s.dims[1];
        dims[3] = 1;
        return GPX_SUCC;
    }
    *rank = s.rank;
    for (int d = 0; d < 4; ++d) dims[d] = d < s.rank ? s.dims[d] : 1;
    return GPX_SUCC;
}

int gpx_model_init_random(gpx_model *m, uint64_t seed) {
    GPX_REQUIRE(m, GPX_FAIL, "NULL model");
    if (m->graph_algo >= 0) return GPX_SUCC;  // nothing to initialise: every run starts from its own init kernel
    if (m->sci) {
        // No parameters: the call puts the simulation back to its initial state.
        for (const char *name : {"state", "state_tmp", "state_tmp2"})
            GPX_CUDA(cudaMemcpy(m->storages[m->find(name)].dptr, m->sci_initial.data(),
                                m->sci_initial.size() * sizeof(float), cudaMemcpyHostToDevice));
        return GPX_SUCC;
    }
    std::vector<float> tmp;
    uint64_t stream = 0;
    for (auto &s : m->storages) {
        if (!s.is_param) continue;
        size_t n = s.bytes / sizeof(float);
        tmp.resize(n);
        if (s.init_std > 0.f)
            normal_fill(tmp.data(), n, seed, stream, s.init_mean, s.init_std);
        else if (s.kind == Storage::Weight)
            normal_fill(tmp.data(), n, seed, stream, 0.f, std::sqrt(2.0f / (float)s.fan_in));
        else
            normal_fill(tmp.data(), n, seed, stream, 0.f, 0.01f);
        ++stream;
        GPX_TRY(storage_set(m, s, tmp.data(), s.bytes, nullptr));
    }
    GPX_CUDA(cudaStreamSynchronize(nullptr));
    return GPX_SUCC;
}

int gpx_model_load_params(gpx_model *m, const char *path) {
    GPX_REQUIRE(m && path, GPX_FAIL, "NULL argument");
    FILE *fp = fopen(path, "rb");
    GPX_REQUIRE(fp, GPX_NOT_FOUND, "cannot open %s", path);
    struct Closer {
        FILE *f;
        ~Closer() { fclose(f); }
    } closer{fp};
    char magic[sizeof(kParamMagic)];
    GPX_REQUIRE(fread(magic, 1, sizeof(magic), fp) == sizeof(magic) &&
                    memcmp(magic, kParamMagic, sizeof(magic)) == 0,
                GPX_FAIL, "%s: bad magic", path);
    uint64_t count = 0;
    GPX_REQUIRE(fread(&count, sizeof(count), 1, fp) == 1 && count != 0, GPX_FAIL,
                "%s: bad parameter count", path);
    std::vector<float> data;
    size_t loaded = 0;
    for (uint64_t i = 0; i < count; ++i) {
        std::string key;
        for (;;) {
            int c = fgetc(fp);
            GPX_REQUIRE(c != EOF && key.size() < 255, GPX_FAIL, "%s: truncated name", path);
            if (c == 0) break;
            key.push_back((char)c);
        }
        uint64_t n = 0;
        GPX_REQUIRE(fread(&n, sizeof(n), 1, fp) == 1 && n != 0, GPX_FAIL, "%s: bad size for %s",
                    path, key.c_str());
        GPX_REQUIRE(n <= (1ull << 34), GPX_FAIL, "%s: implausible size for %s", path, key.c_str());
        data.resize(n);
        GPX_REQUIRE(fread(data.data(), sizeof(float), n, fp) == n, GPX_FAIL,
                    "%s: truncated data for %s", path, key.c_str());
        int idx = m->find(key);
        // Names absent from the graph are skipped, as Model::load_param does
        // (src/model.cpp:270-276 looks names up and copies the ones it finds).
        if (idx < 0) continue;
        Storage &s = m->storages[idx];
        GPX_REQUIRE(n * sizeof(float) == s.bytes, GPX_OUT_OF_RANGE,
                    "%s: %s has %llu elements, model expects %zu", path, key.c_str(),
                    (unsigned long long)n, s.bytes / sizeof(float));
        GPX_TRY(storage_set(m, s, data.data(), s.bytes, nullptr));
        ++loaded;
    }
    GPX_CUDA(cudaStreamSynchronize(nullptr));
    GPX_REQUIRE(loaded > 0, GPX_NOT_FOUND, "%s: no parameter matched the model", path);
    return GPX_SUCC;
}

int gpx_model_save_params(gpx_model *m, const char *path) {
    GPX_REQUIRE(m && path, GPX_FAIL, "NULL argument");
    FILE *fp = fopen(path, "wb");
    GPX_REQUIRE(fp, GPX_FAIL, "cannot create %s", path);
    struct Closer {
        FILE *f;
        ~Closer() { fclose(f); }
    } closer{fp};
    uint64_t count = 0;
    for (auto &s : m->storages) count += s.is_param ? 1 : 0;
    fwrite(kParamMagic, 1, sizeof(kParamMagic), fp);
    fwrite(&count, sizeof(count), 1, fp);
    std::vector<float> data;
    for (auto &s : m->storages) {
        if (!s.is_param) continue;
        uint64_t n = s.bytes / sizeof(float);
        data.resize(n);
        GPX_TRY(storage_get(m, s, data.data(), s.bytes, nullptr));
        GPX_CUDA(cudaStreamSynchronize(nullptr));
        fwrite(s.name.c_str(), 1, s.name.size() + 1, fp);
        fwrite(&n, sizeof(n), 1, fp);
        GPX_REQUIRE(fwrite(data.data(), sizeof(float), n, fp) == n, GPX_FAIL, "short write to %s",
                    path);
    }
    return GPX_SUCC;
}

int gpx_model_kernel_num(gpx_model *m, size_t *n) {
    GPX_REQUIRE(m && n, GPX_FAIL, "NULL argument");
    *n = m->kernels.size();
    return GPX_SUCC;
}

int gpx_model_kernel_info(gpx_model *m, size_t idx, char *name, size_t name_cap,
                          uint32_t launch_params[6], int *total_tiles, double *flops,
                          double *bytes) {
    GPX_REQUIRE(m, GPX_FAIL, "NULL model");
    GPX_REQUIRE(idx < m->kernels.size(), GPX_OUT_OF_RANGE, "kernel index %zu out of range", idx);
    const Kernel &k = m->kernels[idx];
    if (name && name_cap) snprintf(name, name_cap, "%s", k.name.c_str());
    if (launch_params) {
        launch_params[0] = (uint32_t)k.grid;
        launch_params[1] = launch_params[2] = 1;
        launch_params[3] = (uint32_t)k.threads;
        launch_params[4] = launch_params[5] = 1;
    }
    if (total_tiles) *total_tiles = k.total_tiles;
    if (flops) *flops = k.flops;
    if (bytes) *bytes = k.bytes;
    return GPX_SUCC;
}

}  // extern "C"
