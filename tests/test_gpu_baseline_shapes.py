"""Parity at the shapes the benchmark configurations run, not at miniature ones.

Every configuration's model is executed at its own batch size, storage format and sequence length
(ResNet-50 b32 float32, VGG-16 b16 float16, DenseNet-201 b64 bfloat16, BERT-base s512 b32
bfloat16, and the batch-1 latency-critical shapes) and compared with the float64-accumulating CPU
oracle.  Inference is independent per batch item, so the oracle runs three items of the batch
(first, middle, last) one at a time and the matching slices of the GPU tensors are compared:
max|gpu - oracle| / max|oracle| <= 1e-4 for float32 models, <= 2e-2 for the 16-bit formats.
Mirrors src/tests/test-dnn.cpp:13-41 of the reference (forward, then look at the output), asserted.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL_FP32 = 1e-4
RTOL_16BIT = 2e-2


def _rel(a, b):
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))) /
                 max(float(np.max(np.abs(b))), 1e-30))


def _images(gpx, batch, seed=0):
    return gpx.synth_normal(batch * 3 * 224 * 224, seed, 0).reshape(batch, 3, 224, 224)


def _items(batch):
    return sorted({0, batch // 2, batch - 1})


def _kernel_names(ex):
    return [ex.model.get_kernel_info(i)["name"] for i in range(ex.get_kernel_num())]


def test_c1_resnet50_b32_float32(gpx, oracle):
    """The best-effort tenant of the contention benchmark: 128-column tiles, two accumulator
    buffers, no split K (unlike the batch-1 and batch-2 cases of the other parity tests)."""
    batch = 32
    ex = gpx.BaseExecutor()
    ex.init("resnet50", batch=batch, seed=1)
    names = _kernel_names(ex)
    assert not any(n.endswith(".finish") for n in names if n.startswith(("layer1", "layer2", "layer3"))), \
        "batch 32 is expected to run stages 1-3 without split K"
    data = _images(gpx, batch)
    ex.set_input("data", data)
    ex.execute()
    assert ex.error() == (0, 0)
    heads = ex.get_output("heads")
    assert heads.shape == (batch, 1000)
    params = ex.model.params()
    tap_names = ["conv1", "maxpool", "layer1.0.conv3", "layer2.0.conv2", "layer2.0.downsample",
                 "layer3.1.conv2", "layer3.5.conv3", "layer4.0.conv2", "layer4.2.conv3", "avgpool"]
    got = {n: ex.model.get(n) for n in tap_names}
    for i in _items(batch):
        taps = {}
        want = oracle.forward("resnet50", params, data[i:i + 1], taps=taps)
        for n in tap_names:
            ref = taps[n]
            g = got[n][i:i + 1].reshape(ref.shape)
            assert _rel(g, ref) <= RTOL_FP32, f"item {i} node {n}: {_rel(g, ref):.2e}"
        assert _rel(heads[i:i + 1], want) <= RTOL_FP32, f"item {i} heads"
    ex.clear()


def test_c0_resnet50_b1_float32_graph_replay(gpx, oracle):
    """The latency-critical request as the scheduler runs it: batch 1, replayed from a captured
    CUDA graph on a high-priority stream."""
    ex = gpx.BaseExecutor()
    ex.init("resnet50", batch=1, seed=1)
    s = gpx.Stream(0)
    ex.capture_graph(s)
    data = _images(gpx, 1, seed=11)
    ex.set_input("data", data)
    ex.execute(s)
    s.sync()
    assert ex.error() == (0, 0)
    want = oracle.forward("resnet50", ex.model.params(), data)
    assert _rel(ex.get_output("heads"), want) <= RTOL_FP32
    ex.clear()
    s.destroy()


def test_c3_vgg16_b16_float16(gpx, oracle):
    batch = 16
    ex = gpx.BaseExecutor()
    ex.init("vgg16", batch=batch, seed=7, dtype="float16")
    data = _images(gpx, batch, seed=8)
    ex.set_input("data", data)
    ex.execute()
    assert ex.error() == (0, 0)
    heads = ex.get_output("heads")
    params = ex.model.params()
    for i in _items(batch):
        want = oracle.forward("vgg16", params, data[i:i + 1])
        assert _rel(heads[i:i + 1], want) <= RTOL_16BIT, f"item {i}: {_rel(heads[i:i + 1], want):.2e}"
    ex.clear()


def test_c4_densenet201_b64_bfloat16(gpx, oracle):
    batch = 64
    ex = gpx.BaseExecutor()
    ex.init("densenet201", batch=batch, seed=1, dtype="bfloat16")
    data = _images(gpx, batch)
    ex.set_input("data", data)
    ex.execute()
    assert ex.error() == (0, 0)
    heads = ex.get_output("heads")
    params = ex.model.params()
    for i in _items(batch):
        want = oracle.forward("densenet201", params, data[i:i + 1])
        assert _rel(heads[i:i + 1], want) <= RTOL_16BIT, f"item {i}: {_rel(heads[i:i + 1], want):.2e}"
    ex.clear()


def test_c4_bert_base_s512_b32_bfloat16(gpx, oracle):
    batch, seq = 32, 512
    ex = gpx.BaseExecutor()
    ex.init("bert_base", batch=batch, seed=7, seq_len=seq, dtype="bfloat16")
    assert any(n.endswith(".vt") for n in _kernel_names(ex)), "tensor-core attention not selected"
    ids = np.random.default_rng(6).integers(0, 30522, (batch, seq)).astype(np.int64)
    ex.set_input("data", ids)
    ex.execute()
    assert ex.error() == (0, 0)
    heads = ex.get_output("heads")
    assert heads.shape == (batch, seq, 768)
    ctx = ex.model.get("encoder.layer.0.attention.context").reshape(batch, seq, 768)
    params = {k: v.reshape(v.shape[0], -1) if v.ndim == 4 else v for k, v in ex.model.params().items()}
    for i in (0, batch - 1):
        taps = {}
        want = oracle.bert_forward(params, ids[i:i + 1], layers=12, heads=12, taps=taps)
        ref_ctx = taps["encoder.layer.0.attention.context"].reshape(1, seq, 768)
        assert _rel(ctx[i:i + 1], ref_ctx) <= RTOL_16BIT, f"item {i} attention context"
        assert _rel(heads[i:i + 1], want.reshape(1, seq, 768)) <= RTOL_16BIT, f"item {i} heads"
    ex.clear()


@pytest.mark.parametrize("model,dtype", [("resnet50", "bfloat16"), ("mobilenet_v2", "bfloat16")])
def test_c4_latency_critical_b1_bfloat16(gpx, oracle, model, dtype):
    ex = gpx.BaseExecutor()
    ex.init(model, batch=1, seed=1, dtype=dtype)
    data = _images(gpx, 1, seed=12)
    ex.set_input("data", data)
    ex.execute()
    assert ex.error() == (0, 0)
    want = oracle.forward(model, ex.model.params(), data)
    assert _rel(ex.get_output("heads"), want) <= RTOL_16BIT
    ex.clear()


def test_c3_bert_base_s128_b1_float16(gpx, oracle):
    ex = gpx.BaseExecutor()
    ex.init("bert_base", batch=1, seed=7, seq_len=128, dtype="float16")
    ids = np.random.default_rng(6).integers(0, 30522, (1, 128)).astype(np.int64)
    ex.set_input("data", ids)
    ex.execute()
    assert ex.error() == (0, 0)
    params = {k: v.reshape(v.shape[0], -1) if v.ndim == 4 else v for k, v in ex.model.params().items()}
    want = oracle.bert_forward(params, ids, layers=12, heads=12)
    assert _rel(ex.get_output("heads"), want.reshape(1, 128, 768)) <= RTOL_16BIT
    ex.clear()
