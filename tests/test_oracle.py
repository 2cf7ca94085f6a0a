"""Pins the CPU oracle (test infrastructure) against independent implementations.

The reference holds no golden vectors for this path (its DNN tests only print values), so the
oracle's layer functions are compared with PyTorch's CPU operators in float64, and its ResNet-50
restatement with torchvision's resnet50 topology (batch norm replaced by the folded bias).
"""
from fractions import Fraction

import numpy as np
import pytest
import torch
import torch.nn.functional as F


def _rel(a, b):
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))) /
                 max(float(np.max(np.abs(b))), 1e-30))


@pytest.mark.parametrize("cfg", [
    # n, cin, h, w, cout, k, stride, pad
    (1, 3, 23, 19, 8, 7, 2, 3),
    (2, 16, 14, 14, 32, 3, 1, 1),
    (2, 16, 15, 13, 32, 3, 2, 1),
    (3, 32, 9, 9, 24, 1, 1, 0),
    (1, 32, 9, 9, 24, 1, 2, 0),
    (2, 8, 7, 7, 12, 7, 1, 0),
])
def test_conv2d_matches_torch_float64(oracle, cfg):
    n, cin, h, w, cout, k, stride, pad = cfg
    rng = np.random.default_rng(hash(cfg) & 0xFFFF)
    x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = rng.standard_normal((cout, cin, k, k)).astype(np.float32)
    b = rng.standard_normal(cout).astype(np.float32)
    ref = F.conv2d(torch.from_numpy(x).double(), torch.from_numpy(wt).double(),
                   torch.from_numpy(b).double(), stride=stride, padding=pad)
    res = rng.standard_normal(tuple(ref.shape)).astype(np.float32)
    ref = torch.relu(ref + torch.from_numpy(res).double()).float().numpy()
    got = oracle.conv2d(x, wt, b, stride, pad, relu=True, residual=res)
    assert got.shape == ref.shape
    assert _rel(got, ref) < 2e-7
    fast = oracle.conv2d(x, wt, b, stride, pad, relu=True, residual=res, fast=True)
    assert _rel(fast, ref) < 1e-5


def test_pool2d_matches_torch(oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 8, 13, 11)).astype(np.float32)
    ref = F.max_pool2d(torch.from_numpy(x), 3, 2, 1).numpy()
    assert np.array_equal(oracle.pool2d(x, 3, 2, 1, "max"), ref)
    ref = F.max_pool2d(torch.from_numpy(x), 2, 2, 0).numpy()
    assert np.array_equal(oracle.pool2d(x, 2, 2, 0, "max"), ref)
    x7 = rng.standard_normal((2, 8, 7, 7)).astype(np.float32)
    ref = F.adaptive_avg_pool2d(torch.from_numpy(x7).double(), 1).float().numpy()
    assert _rel(oracle.pool2d(x7, 7, 1, 0, "avg"), ref) < 2e-7


def test_axpy_is_a_correctly_rounded_fma(oracle):
    rng = np.random.default_rng(7)
    x = rng.uniform(-1, 1, 257).astype(np.float32)
    y = rng.uniform(-1, 1, 257).astype(np.float32)
    a = np.float32(1.0009765625)
    got = oracle.axpy(a, x, y)
    for i in range(257):
        exact = Fraction(float(a)) * Fraction(float(x[i])) + Fraction(float(y[i]))
        want = np.float32(float(exact))  # float(Fraction) rounds once to double; check below
        # a*x+y needs at most 24+24+1 bits around y's exponent, so the double is exact or a
        # tie-free neighbour; confirm the float result is within half an ulp of the exact value.
        ulp = np.spacing(np.abs(got[i]))
        assert abs(Fraction(float(got[i])) - exact) <= Fraction(float(ulp)) / 2
        assert abs(float(want) - float(got[i])) <= float(ulp)


def test_bf16_conversion_and_gemm(oracle):
    rng = np.random.default_rng(11)
    f = rng.uniform(-1, 1, 4096).astype(np.float32)
    bits = oracle.f32_to_bf16(f)
    tb = torch.from_numpy(f).to(torch.bfloat16)
    assert np.array_equal(bits, tb.view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(oracle.bf16_to_f32(bits), tb.float().numpy())
    a = oracle.f32_to_bf16(rng.uniform(-1, 1, (48, 96)).astype(np.float32))
    b = oracle.f32_to_bf16(rng.uniform(-1, 1, (40, 96)).astype(np.float32))
    ref = (torch.from_numpy(oracle.bf16_to_f32(a)).double() @
           torch.from_numpy(oracle.bf16_to_f32(b)).double().T).numpy()
    got = oracle.gemm_bf16_nt(a, b)
    assert np.max(np.abs(got - ref)) < 1e-12
    rows = np.array([0, 5, 47], np.int32)
    cols = np.array([39, 0, 7], np.int32)
    assert np.allclose(oracle.gemm_bf16_nt_samples(a, b, rows, cols), ref[rows, cols], atol=1e-12)
    assert _rel(oracle.gemm_bf16_nt_fast(a, b), ref) < 1e-5


class _Bias(torch.nn.Module):
    """Stands where a batch norm sat: adds the folded per-channel bias."""

    def __init__(self, bias):
        super().__init__()
        self.bias = torch.nn.Parameter(bias)

    def forward(self, x):
        return x + self.bias.view(1, -1, 1, 1)


def test_resnet50_restatement_matches_torchvision_topology(oracle):
    import torchvision

    rng = np.random.default_rng(3)
    shapes = oracle.resnet_param_shapes()
    params = {}
    for name, shape in shapes.items():
        if name.endswith("weight"):
            fan_in = int(np.prod(shape[1:]))
            params[name] = (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
        else:
            params[name] = (rng.standard_normal(shape) * 0.01).astype(np.float32)
    net = torchvision.models.resnet50(weights=None).double().eval()

    def put(conv, bn_owner, bn_name, prefix):
        conv.weight.data = torch.from_numpy(params[prefix + ".weight"]).double()
        setattr(bn_owner, bn_name, _Bias(torch.from_numpy(params[prefix + ".bias"]).double()))

    put(net.conv1, net, "bn1", "conv1")
    for li in range(4):
        layer = getattr(net, f"layer{li + 1}")
        for bi, block in enumerate(layer):
            p = f"layer{li + 1}.{bi}"
            put(block.conv1, block, "bn1", p + ".conv1")
            put(block.conv2, block, "bn2", p + ".conv2")
            put(block.conv3, block, "bn3", p + ".conv3")
            if block.downsample is not None:
                block.downsample[0].weight.data = torch.from_numpy(
                    params[p + ".downsample.weight"]).double()
                block.downsample[1] = _Bias(torch.from_numpy(params[p + ".downsample.bias"]).double())
    net.fc.weight.data = torch.from_numpy(params["fc.weight"].reshape(1000, 2048)).double()
    net.fc.bias.data = torch.from_numpy(params["fc.bias"]).double()
    data = rng.standard_normal((1, 3, 224, 224)).astype(np.float32)
    with torch.no_grad():
        ref = net(torch.from_numpy(data).double()).numpy()
    got = oracle.forward("resnet50", params, data)
    assert got.shape == (1, 1000)
    assert _rel(got, ref) < 5e-6


def test_vgg16_restatement_matches_torchvision_topology(oracle):
    import torchvision

    rng = np.random.default_rng(4)
    net = torchvision.models.vgg16(weights=None).eval()
    params = {}
    ci = 0
    for m in net.features:
        if isinstance(m, torch.nn.Conv2d):
            params[f"features.{ci}.weight"] = m.weight.detach().numpy().copy()
            params[f"features.{ci}.bias"] = (rng.standard_normal(m.bias.shape) * 0.01).astype(np.float32)
            m.bias.data = torch.from_numpy(params[f"features.{ci}.bias"])
            ci += 1
    for idx, shape in ((0, (4096, 512, 7, 7)), (3, (4096, 4096, 1, 1)), (6, (1000, 4096, 1, 1))):
        lin = net.classifier[idx]
        params[f"classifier.{idx}.weight"] = lin.weight.detach().numpy().reshape(shape).copy()
        params[f"classifier.{idx}.bias"] = lin.bias.detach().numpy().copy()
    data = rng.standard_normal((1, 3, 224, 224)).astype(np.float32)
    with torch.no_grad():
        ref = net.double()(torch.from_numpy(data).double()).numpy()
    got = oracle.forward("vgg16", params, data)
    assert _rel(got, ref) < 5e-6


def test_mobilenet_v2_restatement_matches_torchvision_topology(oracle):
    import torchvision

    rng = np.random.default_rng(5)
    params = {}
    for name, shape in oracle.mobilenet_v2_param_shapes().items():
        if name.endswith("weight"):
            fan_in = int(np.prod(shape[1:]))
            params[name] = (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
        else:
            params[name] = (rng.standard_normal(shape) * 0.01).astype(np.float32)
    net = torchvision.models.mobilenet_v2(weights=None).double().eval()

    def put(seq, conv_idx, prefix):
        # seq[conv_idx] is the convolution, seq[conv_idx + 1] its batch norm
        seq[conv_idx].weight.data = torch.from_numpy(params[prefix + ".weight"]).double()
        seq[conv_idx + 1] = _Bias(torch.from_numpy(params[prefix + ".bias"]).double())

    put(net.features[0], 0, "features.0")
    for idx in range(1, 18):
        block = net.features[idx].conv
        p = f"features.{idx}"
        if len(block) == 4:
            put(block[0], 0, p + ".expand")
            put(block[1], 0, p + ".dw")
            put(block, 2, p + ".project")
        else:
            put(block[0], 0, p + ".dw")
            put(block, 1, p + ".project")
    put(net.features[18], 0, "features.18")
    net.classifier[1].weight.data = torch.from_numpy(params["classifier.weight"].reshape(1000, 1280)).double()
    net.classifier[1].bias.data = torch.from_numpy(params["classifier.bias"]).double()
    data = rng.standard_normal((1, 3, 224, 224)).astype(np.float32)
    with torch.no_grad():
        ref = net(torch.from_numpy(data).double()).numpy()
    got = oracle.forward("mobilenet_v2", params, data)
    assert got.shape == (1, 1000)
    assert _rel(got, ref) < 5e-6


class _Affine(torch.nn.Module):
    """Stand-in for an inference batch norm: per-channel scale and shift."""

    def __init__(self, scale, shift):
        super().__init__()
        self.scale, self.shift = scale, shift

    def forward(self, x):
        return x * self.scale.view(1, -1, 1, 1) + self.shift.view(1, -1, 1, 1)


def test_densenet201_restatement_matches_torchvision_topology(oracle):
    import torchvision

    rng = np.random.default_rng(6)
    params = {}
    for name, shape in oracle.densenet_param_shapes("densenet201").items():
        if len(shape) == 4:
            fan_in = int(np.prod(shape[1:]))
            params[name] = (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
        elif ".norm" in name and name.endswith("weight"):
            params[name] = (1.0 + rng.standard_normal(shape) * 0.02).astype(np.float32)
        else:
            params[name] = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    net = torchvision.models.densenet201(weights=None).double().eval()
    t = lambda k: torch.from_numpy(params[k]).double()

    def conv(mod, prefix, own_bias):
        mod.weight.data = t(prefix + ".weight")
        if own_bias:
            mod.bias = torch.nn.Parameter(t(prefix + ".bias"))

    f = net.features
    conv(f.conv0, "features.conv0", False)
    f.norm0 = _Bias(t("features.conv0.bias"))
    for b, nl in enumerate((6, 12, 48, 32)):
        block = getattr(f, f"denseblock{b + 1}")
        for l in range(nl):
            p = f"features.denseblock{b + 1}.denselayer{l + 1}"
            layer = getattr(block, f"denselayer{l + 1}")
            layer.norm1 = _Affine(t(p + ".norm1.weight"), t(p + ".norm1.bias"))
            conv(layer.conv1, p + ".conv1", False)
            layer.norm2 = _Bias(t(p + ".conv1.bias"))
            conv(layer.conv2, p + ".conv2", True)
        if b < 3:
            p = f"features.transition{b + 1}"
            tr = getattr(f, f"transition{b + 1}")
            tr.norm = _Affine(t(p + ".norm.weight"), t(p + ".norm.bias"))
            conv(tr.conv, p + ".conv", True)
    f.norm5 = _Affine(t("features.norm5.weight"), t("features.norm5.bias"))
    net.classifier.weight.data = t("classifier.weight").reshape(1000, 1920)
    net.classifier.bias.data = t("classifier.bias")
    data = rng.standard_normal((1, 3, 224, 224)).astype(np.float32)
    with torch.no_grad():
        ref = net(torch.from_numpy(data).double()).numpy()
    got = oracle.forward("densenet201", params, data)
    assert got.shape == (1, 1000)
    assert _rel(got, ref) < 5e-6


def test_blp_protocol_runs_every_tile_exactly_once_across_resumes(oracle):
    rng = np.random.default_rng(9)
    for trial in range(50):
        total = int(rng.integers(1, 400))
        ctas = int(rng.integers(1, 64))
        cost = lambda i: 1.0 + (i % 7) * 0.25
        done, cursor, stop = [], 0, -1
        for attempt in range(100):
            raise_at = float(rng.uniform(0, 10)) if attempt < 99 else None
            d, cursor, stop, _ = oracle.blp_simulate(total, ctas, cost, raise_at, cursor, -1, 5)
            done += d
            if stop == -1:
                break
            assert stop == 5
        assert sorted(done) == list(range(total))
        # a claimed tile always completes, so the drain never exceeds the longest tile
        d, c2, s2, t_exit = oracle.blp_simulate(total, ctas, cost, 3.0)
        assert t_exit <= 3.0 + 2.5 + 1e-9 or s2 == -1


def test_bert_restatement_matches_huggingface_bert(oracle):
    """The oracle's BERT encoder against transformers.BertModel (random weights, float64)."""
    transformers = pytest.importorskip("transformers")
    cfg = transformers.BertConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                                  intermediate_size=256, vocab_size=1000, max_position_embeddings=64,
                                  hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    net = transformers.BertModel(cfg, add_pooling_layer=False).double().eval()
    params = {k: v.detach().numpy() for k, v in net.state_dict().items() if "position_ids" not in k}
    ids = np.random.default_rng(6).integers(0, 1000, (2, 16))
    with torch.no_grad():
        ref = net(input_ids=torch.from_numpy(ids)).last_hidden_state.numpy()
    got = oracle.bert_forward(params, ids, layers=2, heads=4)
    assert got.shape == ref.shape
    assert _rel(got, ref) < 2e-6


def test_distilbert_restatement_matches_huggingface_distilbert(oracle):
    """The oracle's DistilBERT encoder (the sequence model the reference compiles,
    scripts/compile/compile-bert.py:33-52) against transformers.DistilBertModel on a 6-token input."""
    transformers = pytest.importorskip("transformers")
    cfg = transformers.DistilBertConfig(dim=128, n_layers=2, n_heads=4, hidden_dim=256, vocab_size=1000,
                                        max_position_embeddings=64, dropout=0.0, attention_dropout=0.0)
    torch.manual_seed(0)
    net = transformers.DistilBertModel(cfg).double().eval()
    params = {k: v.detach().numpy() for k, v in net.state_dict().items() if "position_ids" not in k}
    assert set(params) == set(oracle.distilbert_param_shapes(layers=2, hidden=128, heads=4, ffn=256, vocab=1000, max_pos=64))
    ids = np.random.default_rng(6).integers(0, 1000, (2, 6))
    with torch.no_grad():
        ref = net(input_ids=torch.from_numpy(ids)).last_hidden_state.numpy()
    got = oracle.distilbert_forward(params, ids, layers=2, heads=4)
    assert got.shape == ref.shape
    assert _rel(got, ref) < 2e-6


def test_inception_v3_restatement_matches_torchvision_topology(oracle):
    """The oracle's Inception-v3 (one-sided 1x7 / 7x1 / 1x3 / 3x1 kernels, unpadded stride-2
    convolutions, average pooling that counts the padding, four- and six-way concatenations)
    against torchvision.models.inception_v3 with every batch norm replaced by the folded bias."""
    import torchvision

    rng = np.random.default_rng(8)
    params = {}
    for name, shape in oracle.inception_v3_param_shapes().items():
        if name.endswith("weight"):
            fan_in = int(np.prod(shape[1:]))
            params[name] = (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
        else:
            params[name] = (rng.standard_normal(shape) * 0.01).astype(np.float32)
    net = torchvision.models.inception_v3(weights=None, aux_logits=False, transform_input=False,
                                          init_weights=False).double().eval()
    seen = 0
    for name, _, cout, _, _, _ in oracle.INCEPTION_CONVS:
        block = net.get_submodule(name)          # a BasicConv2d: conv + bn (+ relu in forward)
        assert tuple(block.conv.weight.shape) == params[name + ".weight"].shape, name
        block.conv.weight.data = torch.from_numpy(params[name + ".weight"]).double()
        block.bn = _Bias(torch.from_numpy(params[name + ".bias"]).double())
        seen += 1
    assert seen == sum(1 for m in net.modules() if isinstance(m, torch.nn.Conv2d))
    net.fc.weight.data = torch.from_numpy(params["fc.weight"].reshape(1000, 2048)).double()
    net.fc.bias.data = torch.from_numpy(params["fc.bias"]).double()
    data = rng.standard_normal((1, 3, 299, 299)).astype(np.float32)
    with torch.no_grad():
        ref = net(torch.from_numpy(data).double()).numpy()
    taps = {}
    got = oracle.forward("inception_v3", params, data, taps=taps)
    assert got.shape == (1, 1000)
    assert taps["Mixed_5d"].shape == (1, 288, 35, 35) and taps["Mixed_6e"].shape == (1, 768, 17, 17)
    assert taps["Mixed_7c"].shape == (1, 2048, 8, 8)
    assert _rel(got, ref) < 5e-6
