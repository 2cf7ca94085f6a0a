"""Model-level parity (GPU forward vs the CPU oracle) and preempt/resume bit-exactness."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL_FP32 = 1e-4  # max|gpu - oracle| / max|oracle|, the fp32 tolerance of the parity contract


def _rel(a, b):
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))) /
                 max(float(np.max(np.abs(b))), 1e-30))


def _data(gpx, batch, seed=0):
    return gpx.synth_normal(batch * 3 * 224 * 224, seed, 0).reshape(batch, 3, 224, 224)


@pytest.mark.parametrize("model,batch", [("resnet_tiny", 1), ("resnet_tiny", 3), ("resnet50", 1),
                                         ("resnet50", 2), ("mobilenet_v2", 1), ("mobilenet_v2", 3),
                                         ("densenet_tiny", 1), ("densenet_tiny", 3), ("densenet201", 1)])
def test_forward_matches_oracle_layer_by_layer(gpx, oracle, model, batch):
    ex = gpx.BaseExecutor()
    ex.init(model, batch=batch, seed=1)
    data = _data(gpx, batch)
    ex.set_input("data", data)
    ex.execute()
    heads = ex.get_output("heads")
    params = ex.model.params()
    taps = {}
    want = oracle.forward(model, params, data, taps=taps)
    assert heads.shape == want.shape == (batch, 1000)
    for name, ref in taps.items():
        got = ex.model.get(name).reshape(ref.shape)
        assert _rel(got, ref) <= RTOL_FP32, f"{model} b{batch} node {name}"
    assert _rel(heads, want) <= RTOL_FP32
    ex.clear()


def test_all_ten_input_fixture(gpx, oracle):
    """The reference's DNN smoke input: every element 10.0 (src/tests/test-dnn.cpp:25-29)."""
    ex = gpx.BaseExecutor()
    ex.init("resnet_tiny", batch=1, seed=5)
    data = np.full((1, 3, 224, 224), 10.0, np.float32)
    ex.set_input("data", data)
    ex.execute()
    got = ex.get_output("heads")
    want = oracle.forward("resnet_tiny", ex.model.params(), data)
    assert _rel(got, want) <= RTOL_FP32
    ex.clear()


def test_vgg16_matches_oracle(gpx, oracle):
    ex = gpx.BaseExecutor()
    ex.init("vgg16", batch=1, seed=7)
    data = _data(gpx, 1, seed=8)
    ex.set_input("data", data)
    ex.execute()
    got = ex.get_output("heads")
    want = oracle.forward("vgg16", ex.model.params(), data)
    assert _rel(got, want) <= RTOL_FP32
    ex.clear()


def test_set_get_size_checks_and_names(gpx):
    from gpreempt_b200 import binding as B

    ex = gpx.BaseExecutor()
    ex.init("resnet_tiny", batch=1, seed=1)
    assert ex.get_data_size("data") == 3 * 224 * 224 * 4
    assert ex.get_data_size("heads") == 4000
    with pytest.raises(gpx.GpxError) as e:
        ex.set_input("data", np.zeros(10, np.float32))
    assert e.value.status == B.OUT_OF_RANGE  # `len < size` is rejected, src/model.cpp:317
    with pytest.raises(gpx.GpxError) as e:
        ex.model.find_storage_idx("no_such_tensor")
    assert e.value.status == B.NOT_FOUND
    with pytest.raises(gpx.GpxError) as e:
        ex.launch_kernel(10_000)
    assert e.value.status == B.OUT_OF_RANGE
    w = ex.model.get("conv1.weight")
    assert w.shape == (64, 3, 7, 7)
    ex.model.set("conv1.weight", w * 2)
    assert np.array_equal(ex.model.get("conv1.weight"), w * 2)
    ex.clear()


def test_params_file_round_trip(gpx, tmp_path):
    """mod.params format of ModelParamParser::parse_from_file (src/model.cpp:15-55)."""
    a = gpx.Model("resnet_tiny")
    a.init_random(3)
    path = str(tmp_path / "mod.params")
    a.save_param(path)
    raw = open(path, "rb").read()
    assert raw[:17] == b"TVM_MODEL_PARAMS\x00"
    count = int(np.frombuffer(raw[17:25], np.uint64)[0])
    pa = a.params()
    assert count == len(pa)
    b = gpx.Model("resnet_tiny")
    b.load_param(path)
    pb = b.params()
    for k in pa:
        assert np.array_equal(pa[k], pb[k]), k
    a.clear(), b.clear()


def test_graph_capture_matches_eager(gpx):
    ex = gpx.BaseExecutor()
    ex.init("resnet_tiny", batch=2, seed=1)
    data = _data(gpx, 2)
    ex.set_input("data", data)
    ex.execute()
    eager = ex.get_output("heads")
    s = gpx.Stream(0)
    ex.capture_graph(s)
    ex.set_input("data", data * 0.5)
    ex.execute(s)
    s.sync()
    ex.set_input("data", data)
    ex.execute(s)
    s.sync()
    assert np.array_equal(ex.get_output("heads"), eager)
    ex.clear()
    s.destroy()


def _all_activations(ex):
    out = {}
    for i in range(ex.model.get_storage_num()):
        info = ex.model.get_storage_info(i)
        if not info["is_param"] and info["name"] != "data":
            out[info["name"]] = ex.model.get(info["name"])
    return out


@pytest.mark.parametrize("model,batch,transport", [("resnet_tiny", 8, 0), ("resnet50", 8, 0),
                                                   ("resnet50", 8, 1), ("mobilenet_v2", 8, 0),
                                                   ("densenet_tiny", 8, 0)])
def test_model_preempt_resume_bit_identical(gpx, model, batch, transport):
    """Asserted form of src/tests/test-dnn-blp.cpp:36-43: execute, raise the word, drain, clear,
    resume; every activation equals the uninterrupted run bit for bit."""
    base = gpx.BaseExecutor()
    base.init(model, batch=batch, seed=1)
    data = _data(gpx, batch)
    base.set_input("data", data)
    base.execute()
    want = _all_activations(base)
    params = base.model.params()

    word = gpx.PreemptWord(transport)
    ex = gpx.BLPExecutor()
    ex.init(model, batch=batch)
    for k, v in params.items():
        ex.model.set(k, v)
    ex.set_word(word)
    ex.enable_trace(True)
    s = gpx.Stream(1)
    ex.set_input("data", data)

    # uninterrupted BLP run == static-schedule run
    ex.execute(s)
    assert ex.getStopPoint(s) == -1
    got = _all_activations(ex)
    for k in want:
        assert np.array_equal(got[k], want[k]), f"uninterrupted {k}"
    nk = ex.get_kernel_num()
    tiles = np.array([ex.model.get_kernel_info(i)["total_tiles"] for i in range(nk)])
    trace = ex.read_trace()
    assert np.array_equal(trace[:, 3].astype(np.int64), tiles)
    # kernels of one stream run in order: start times are non-decreasing
    assert np.all(np.diff(trace[:, 0].astype(np.int64)) >= 0)

    # time one uninterrupted run to place the triggers
    t0 = time.perf_counter()
    ex.execute(s)
    s.sync()
    run_us = (time.perf_counter() - t0) * 1e6

    rng = np.random.default_rng(17)
    stops_seen = 0
    for trial in range(10):
        ex.set_input("data", data * 0.0)
        ex.execute(s)
        s.sync()  # scrub every activation so stale results cannot pass
        ex.set_input("data", data)
        word.clear()
        time.sleep(0.001)
        ex.execute(s)
        rounds = 0
        while True:
            if rounds < 4:
                delay = float(rng.uniform(0, run_us / 2))
                t0 = time.perf_counter()
                while (time.perf_counter() - t0) * 1e6 < delay:
                    pass
                word.raise_()
            s.sync()           # BE drained
            word.clear()       # only now may later kernels run again
            time.sleep(0.0005)
            stop = ex.resume(s)
            rounds += 1
            if stop == -1:
                break
            stops_seen += 1
            assert 0 <= stop < nk
            assert rounds < 60
        s.sync()
        got = _all_activations(ex)
        for k in want:
            assert np.array_equal(got[k], want[k]), f"trial {trial}: {k} differs after resume"
        cursors = ex.read_cursors()
        assert np.all(cursors >= tiles), "a kernel finished with unclaimed tiles"
    assert stops_seen > 0, "no run was ever preempted"
    base.clear(), ex.clear(), word.destroy(), s.destroy()


def test_execute_with_word_raised_runs_nothing_then_resumes(gpx):
    """The reference's manual test raises the flag right after execute
    (src/tests/test-dnn-blp.cpp:36-43); kernels that start with the word raised retire with zero
    work and the stop point is the first of them."""
    base = gpx.BaseExecutor()
    base.init("resnet_tiny", batch=2, seed=2)
    data = _data(gpx, 2)
    base.set_input("data", data)
    base.execute()
    want = base.get_output("heads")
    word = gpx.PreemptWord(0)
    ex = gpx.BLPExecutor()
    ex.init("resnet_tiny", batch=2)
    for k, v in base.model.params().items():
        ex.model.set(k, v)
    ex.set_word(word)
    ex.set_input("data", data)
    s = gpx.Stream(1)
    word.raise_()
    ex.execute(s)
    assert ex.getStopPoint(s) == 0
    assert np.all(ex.read_cursors() == 0)
    word.clear()
    # getStopPoint re-armed the index; a plain relaunch from 0 is what resume would do
    for i in range(ex.get_kernel_num()):
        ex.launch_kernel(i, s)
    assert ex.getStopPoint(s) == -1
    assert np.array_equal(ex.get_output("heads"), want)
    base.clear(), ex.clear(), word.destroy(), s.destroy()


def test_export_json_has_the_tvm_graph_skeleton(gpx):
    import json

    m = gpx.Model("resnet_tiny")
    g = json.loads(m.export_json())
    assert set(["nodes", "arg_nodes", "heads", "attrs", "node_row_ptr"]) <= set(g)
    names = [n["name"] for n in g["nodes"]]
    assert names[0] == "data" and "heads" in names
    assert g["nodes"][g["heads"][0][0]]["name"] == "heads"
    assert g["attrs"]["dltype"][0] == "list_str" and len(g["attrs"]["dltype"][1]) == len(names)
    assert g["attrs"]["shape"][1][0] == [1, 3, 224, 224]
    m.clear()


def test_cuda_core_convolution_path_matches_oracle(gpx, oracle, monkeypatch):
    """GPX_CONV=simt keeps every convolution on the FFMA kernel (same split-plane storage); it
    must meet the same bound, which also pins the tensor-core path against a second GPU path."""
    monkeypatch.setenv("GPX_CONV", "simt")
    ex = gpx.BaseExecutor()
    ex.init("resnet_tiny", batch=2, seed=1)
    monkeypatch.delenv("GPX_CONV")
    threads = {ex.model.get_kernel_info(i)["launch_params"][3] for i in range(ex.get_kernel_num())}
    assert threads == {256}, "a tensor-core kernel was selected despite GPX_CONV=simt"
    data = _data(gpx, 2)
    ex.set_input("data", data)
    ex.execute()
    simt = ex.get_output("heads")
    want = oracle.forward("resnet_tiny", ex.model.params(), data)
    assert _rel(simt, want) <= RTOL_FP32
    tc = gpx.BaseExecutor()
    tc.init("resnet_tiny", batch=2, seed=1)
    assert max(tc.model.get_kernel_info(i)["launch_params"][3] for i in range(tc.get_kernel_num())) > 256
    tc.set_input("data", data)
    tc.execute()
    assert tc.error() == (0, 0)
    assert _rel(tc.get_output("heads"), simt) <= RTOL_FP32
    ex.clear(), tc.clear()


def test_batch_one_uses_split_k_and_matches_oracle(gpx, oracle):
    """Batch 1 (the latency-critical shape) cuts K over several CTAs; partial sums are added in
    split order by the finishing kernel."""
    ex = gpx.BaseExecutor()
    ex.init("resnet50", batch=1, seed=3)
    names = [ex.model.get_kernel_info(i)["name"] for i in range(ex.get_kernel_num())]
    assert any(n.endswith(".finish") for n in names)
    data = _data(gpx, 1, seed=9)
    ex.set_input("data", data)
    ex.execute()
    a = ex.get_output("heads")
    ex.execute()
    assert np.array_equal(a, ex.get_output("heads")), "split-K result changed between runs"
    assert _rel(a, oracle.forward("resnet50", ex.model.params(), data)) <= RTOL_FP32
    ex.clear()


def _ids(batch, seq, vocab, seed=6):
    return np.random.default_rng(seed).integers(0, vocab, (batch, seq)).astype(np.int64)


@pytest.mark.parametrize("model,batch,seq,layers,heads,vocab", [("bert_tiny", 2, 64, 2, 2, 1000),
                                                                ("bert_tiny", 1, 40, 2, 2, 1000),
                                                                ("bert_base", 1, 128, 12, 12, 30522)])
def test_bert_matches_oracle(gpx, oracle, model, batch, seq, layers, heads, vocab):
    """Token ids U[0, vocab), weights N(0, 0.02): last hidden state against the float64 oracle,
    layer by layer, with the fp32 bound."""
    ex = gpx.BaseExecutor()
    ex.init(model, batch=batch, seed=7, seq_len=seq)
    ids = _ids(batch, seq, vocab)
    ex.set_input("data", ids)
    ex.execute()
    assert ex.error() == (0, 0)
    heads_out = ex.get_output("heads")
    assert heads_out.shape == (batch, seq, ex.model.shape("heads")[2])
    params = {k: v.reshape(v.shape[0], -1) if v.ndim == 4 else v for k, v in ex.model.params().items()}
    taps = {}
    want = oracle.bert_forward(params, ids, layers=layers, heads=heads, taps=taps)
    for name, ref in taps.items():
        if name == "heads":
            continue
        got = ex.model.get(name).reshape(ref.shape)
        assert _rel(got, ref) <= RTOL_FP32, f"{model} node {name}"
    assert _rel(heads_out, want) <= RTOL_FP32
    ex.clear()


@pytest.mark.parametrize("dtype,seq", [("float32", 128), ("float16", 128), ("bfloat16", 512)])
def test_bert_preempt_resume_bit_identical(gpx, dtype, seq):
    """(At 512 tokens a tensor-core attention tile spans four key blocks and is given up at a
    key-block boundary when the word goes up, then recomputed by the relaunched CTA.)"""
    base = gpx.BaseExecutor()
    base.init("bert_tiny", batch=8, seed=7, seq_len=seq, dtype=dtype)
    ids = _ids(8, seq, 1000)
    base.set_input("data", ids)
    base.execute()
    want = base.get_output("heads")
    word = gpx.PreemptWord(1)
    ex = gpx.BLPExecutor()
    ex.init("bert_tiny", batch=8, seq_len=seq, dtype=dtype)
    for k, v in base.model.params().items():
        ex.model.set(k, v)
    ex.set_word(word)
    ex.set_input("data", ids)
    s = gpx.Stream(1)
    ex.execute(s)
    assert ex.getStopPoint(s) == -1
    assert np.array_equal(ex.get_output("heads"), want)
    t0 = time.perf_counter()
    ex.execute(s)
    s.sync()
    run_us = (time.perf_counter() - t0) * 1e6
    rng = np.random.default_rng(3)
    stops = 0
    for trial in range(12 if seq == 512 else 8):
        word.clear()
        time.sleep(0.001)
        ex.execute(s)
        rounds = 0
        while True:
            if rounds < 3:
                delay = float(rng.uniform(0, run_us / 2))
                t0 = time.perf_counter()
                while (time.perf_counter() - t0) * 1e6 < delay:
                    pass
                word.raise_()
            s.sync()
            word.clear()
            time.sleep(0.0005)
            stop = ex.resume(s)
            rounds += 1
            if stop == -1:
                break
            stops += 1
            assert rounds < 60
        s.sync()
        assert np.array_equal(ex.get_output("heads"), want), f"trial {trial}"
    assert stops > 0
    base.clear(), ex.clear(), word.destroy(), s.destroy()


RTOL_16BIT = 2e-2  # the bf16 / fp16 tolerance of the parity contract


@pytest.mark.parametrize("model,batch,dtype", [("resnet_tiny", 2, "bfloat16"), ("resnet_tiny", 2, "float16"),
                                               ("resnet50", 1, "bfloat16"), ("resnet50", 2, "float16"),
                                               ("vgg16", 1, "float16"), ("mobilenet_v2", 1, "bfloat16"),
                                               ("densenet_tiny", 2, "bfloat16"), ("densenet201", 1, "float16")])
def test_reduced_precision_forward_matches_fp32_oracle(gpx, oracle, model, batch, dtype):
    """One 16-bit plane between layers, one tensor-core product per K step, fp32 accumulation:
    `heads` against the float64-accumulating oracle on the same seeded weights and input."""
    ex = gpx.BaseExecutor()
    ex.init(model, batch=batch, seed=1, dtype=dtype)
    data = _data(gpx, batch)
    ex.set_input("data", data)
    ex.execute()
    assert ex.error() == (0, 0)
    got = ex.get_output("heads")
    ex.execute()
    assert np.array_equal(got, ex.get_output("heads"))
    want = oracle.forward(model, ex.model.params(), data)
    assert _rel(got, want) <= RTOL_16BIT, f"{model} {dtype}"
    ex.clear()


@pytest.mark.parametrize("model,batch,seq,layers,heads,vocab,dtype", [
    ("bert_base", 1, 128, 12, 12, 30522, "bfloat16"), ("bert_base", 1, 128, 12, 12, 30522, "float16"),
    ("bert_tiny", 2, 40, 2, 2, 1000, "float16"), ("bert_tiny", 3, 200, 2, 2, 1000, "bfloat16"),
    ("bert_base", 2, 512, 12, 12, 30522, "float16")])
def test_reduced_precision_bert_matches_oracle(gpx, oracle, model, batch, seq, layers, heads, vocab, dtype):
    """Single-plane BERT: dense layers and both attention products on the tensor cores (sequence
    lengths that are and are not multiples of the 128-key block), against the float64 oracle; the
    attention context is also checked on its own."""
    ex = gpx.BaseExecutor()
    ex.init(model, batch=batch, seed=7, seq_len=seq, dtype=dtype)
    names = [ex.model.get_kernel_info(i)["name"] for i in range(ex.get_kernel_num())]
    assert any(n.endswith(".vt") for n in names), "tensor-core attention not selected"
    ids = _ids(batch, seq, vocab)
    ex.set_input("data", ids)
    ex.execute()
    assert ex.error() == (0, 0)
    got = ex.get_output("heads")
    ex.execute()
    assert np.array_equal(got, ex.get_output("heads"))
    params = {k: v.reshape(v.shape[0], -1) if v.ndim == 4 else v for k, v in ex.model.params().items()}
    taps = {}
    want = oracle.bert_forward(params, ids, layers=layers, heads=heads, taps=taps)
    ctx = ex.model.get("encoder.layer.0.attention.context").reshape(taps["encoder.layer.0.attention.context"].shape)
    assert _rel(ctx, taps["encoder.layer.0.attention.context"]) <= RTOL_16BIT
    assert _rel(got, want) <= RTOL_16BIT
    ex.clear()


@pytest.mark.parametrize("dtype,drop", [("float16", False), ("float32", True), ("float16", True)])
def test_reduced_precision_preempt_resume_bit_identical(gpx, dtype, drop):
    """Preempt and resume in the single-plane format, and with the restart policy that drops the
    tile in flight (REEF's reset-and-restart at tile granularity) instead of saving it."""
    base = gpx.BaseExecutor()
    base.init("resnet50", batch=8, seed=1, dtype=dtype)
    data = _data(gpx, 8)
    base.set_input("data", data)
    base.execute()
    want = _all_activations(base)
    word = gpx.PreemptWord(1)
    ex = gpx.BLPExecutor()
    ex.init("resnet50", batch=8, dtype=dtype)
    ex.set_restart_policy(drop)
    for k, v in base.model.params().items():
        ex.model.set(k, v)
    ex.set_word(word)
    ex.set_input("data", data)
    s = gpx.Stream(1)
    t0 = time.perf_counter()
    ex.execute(s)
    s.sync()
    run_us = (time.perf_counter() - t0) * 1e6
    rng = np.random.default_rng(4)
    stops = 0
    for trial in range(8):
        ex.set_input("data", data * 0.0)
        ex.execute(s)
        s.sync()
        ex.set_input("data", data)
        word.clear()
        time.sleep(0.001)
        ex.execute(s)
        rounds = 0
        while True:
            if rounds < 4:
                delay = float(rng.uniform(0, run_us / 2))
                t0 = time.perf_counter()
                while (time.perf_counter() - t0) * 1e6 < delay:
                    pass
                word.raise_()
            s.sync()
            word.clear()
            time.sleep(0.0005)
            stop = ex.resume(s)
            rounds += 1
            if stop == -1:
                break
            stops += 1
            assert rounds < 60
        s.sync()
        got = _all_activations(ex)
        for k in want:
            assert np.array_equal(got[k], want[k]), f"trial {trial}: {k} differs after resume"
    assert stops > 0
    assert ex.error() == (0, 0)
    ex.clear()
    base.clear()
    s.destroy()


def test_wide_tile_layers_preempt_resume_bit_identical(gpx):
    """VGG-16 at batch 8 in fp16 runs its 256- and 512-channel convolutions on 128x256 tiles
    (one accumulator buffer); preempting and resuming them leaves every checked tensor bit-identical."""
    base = gpx.BaseExecutor()
    base.init("vgg16", batch=8, seed=2, dtype="float16")
    data = _data(gpx, 8, seed=3)
    base.set_input("data", data)
    base.execute()
    names = ["features.5", "features.9", "features.12", "heads"]
    want = {n: base.model.get(n) for n in names}
    word = gpx.PreemptWord(1)
    ex = gpx.BLPExecutor()
    ex.init("vgg16", batch=8, dtype="float16")
    for k, v in base.model.params().items():
        ex.model.set(k, v)
    ex.set_word(word)
    ex.set_input("data", data)
    s = gpx.Stream(1)
    t0 = time.perf_counter()
    ex.execute(s)
    s.sync()
    run_us = (time.perf_counter() - t0) * 1e6
    rng = np.random.default_rng(5)
    stops = 0
    for trial in range(6):
        word.clear()
        time.sleep(0.001)
        ex.execute(s)
        rounds = 0
        while True:
            if rounds < 5:
                delay = float(rng.uniform(0, run_us / 3))
                t0 = time.perf_counter()
                while (time.perf_counter() - t0) * 1e6 < delay:
                    pass
                word.raise_()
            s.sync()
            word.clear()
            time.sleep(0.0005)
            stop = ex.resume(s)
            rounds += 1
            if stop == -1:
                break
            stops += 1
            assert rounds < 80
        s.sync()
        for n in names:
            assert np.array_equal(ex.model.get(n), want[n]), f"trial {trial}: {n} differs after resume"
    assert stops > 0
    assert ex.error() == (0, 0)
    ex.clear()
    base.clear()
    s.destroy()


def test_schedule_order_from_device_timestamps(gpx):
    """Raise the word in the middle of a best-effort forward and read the per-kernel %globaltimer
    trace: kernels before the stop point ran all their tiles in stream order; the stopped kernel
    saw the word after the host wrote it and left within the drain bound; no kernel behind it did
    any tile; after the resume every kernel has run exactly its tiles."""
    ex = gpx.BLPExecutor()
    ex.init("resnet50", batch=16, seed=1)
    word = gpx.PreemptWord(1)
    ex.set_word(word)
    ex.enable_trace(True)
    ex.set_input("data", _data(gpx, 16))
    s = gpx.Stream(1)
    nk = ex.get_kernel_num()
    tiles = np.array([ex.model.get_kernel_info(i)["total_tiles"] for i in range(nk)], np.int64)
    t0 = time.perf_counter()
    ex.execute(s)
    s.sync()
    run_us = (time.perf_counter() - t0) * 1e6
    NONE = np.uint64(0xFFFFFFFFFFFFFFFF)
    checked = 0
    for trial, frac in enumerate((0.2, 0.35, 0.5, 0.65, 0.8)):
        word.clear()
        time.sleep(0.001)
        off, unc = gpx.clock_offset_ns()  # host clock minus device clock, and its uncertainty
        ex.execute(s)
        t0 = time.perf_counter()
        while (time.perf_counter() - t0) * 1e6 < run_us * frac:
            pass
        t_raise_dev = gpx.host_now_ns() - off
        word.raise_()
        s.sync()
        tr = ex.read_trace()
        begin, end, seen, done = tr[:, 0], tr[:, 1], tr[:, 2], tr[:, 3].astype(np.int64)
        unfinished = np.nonzero(done < tiles)[0]
        if unfinished.size == 0:
            continue  # the forward had already finished
        stop = int(unfinished[0])
        assert np.array_equal(done[:stop], tiles[:stop]), "a kernel before the stop point is incomplete"
        assert np.all(np.diff(begin[: stop + 1].astype(np.int64)) >= 0), "kernels started out of stream order"
        assert done[stop] < tiles[stop], "the stop point is a kernel that finished"
        assert seen[stop] != NONE
        slack = unc + 20_000  # clock correlation plus the raise call itself
        assert int(seen[stop]) + slack >= t_raise_dev, "the kernel saw the word before it was written"
        assert int(end[stop]) - int(seen[stop]) < 100_000, "drain of the stopped kernel above 100 us"
        assert np.all(done[stop + 1:] == 0), "a kernel behind the stop point ran a tile"
        later = begin[stop + 1:]
        started = later[later != NONE].astype(np.int64)
        assert np.all(started + slack >= t_raise_dev), "a kernel behind the stop point started before the raise"
        word.clear()
        time.sleep(0.0005)
        assert ex.resume(s) == stop, "the recorded stop point is not the first unfinished kernel"
        s.sync()
        assert ex.resume(s) == -1
        assert np.all(ex.read_cursors() >= tiles)
        checked += 1
    assert checked >= 3
    assert ex.error() == (0, 0)
    ex.clear(), word.destroy(), s.destroy()


@pytest.mark.parametrize("model,batch,seq,layers,heads,vocab", [("distilbert_tiny", 2, 6, 2, 2, 1000),
                                                                ("distilbert", 1, 6, 6, 12, 30522),
                                                                ("bert", 2, 40, 6, 12, 30522)])
def test_distilbert_matches_oracle(gpx, oracle, model, batch, seq, layers, heads, vocab):
    """The reference's sequence model (DistilBERT, 6 layers, traced on a 6-token input:
    scripts/compile/compile-bert.py:33-52; "bert" is its name in the task configs): last hidden
    state against the float64 oracle with the fp32 bound, including the reference test's own
    token ids (src/tests/test-dnn.cpp:21-23)."""
    ex = gpx.BaseExecutor()
    ex.init(model, batch=batch, seed=7, seq_len=seq)
    if batch == 1 and seq == 6:
        ids = np.array([[101, 7592, 1010, 2088, 999, 102]], np.int64)
    else:
        ids = _ids(batch, seq, vocab)
    ex.set_input("data", ids)
    ex.execute()
    assert ex.error() == (0, 0)
    got = ex.get_output("heads")
    assert got.shape == (batch, seq, ex.model.shape("heads")[2])
    params = {k: v.reshape(v.shape[0], -1) if v.ndim == 4 else v for k, v in ex.model.params().items()}
    assert "embeddings.token_type_embeddings.weight" not in params
    taps = {}
    want = oracle.distilbert_forward(params, ids, layers=layers, heads=heads, taps=taps)
    for name, ref in taps.items():
        if name == "heads":
            continue
        assert _rel(ex.model.get(name).reshape(ref.shape), ref) <= RTOL_FP32, f"{model} node {name}"
    assert _rel(got, want) <= RTOL_FP32
    ex.clear()


@pytest.mark.parametrize("batch", [1, 2])
def test_inception_v3_matches_oracle_layer_by_layer(gpx, oracle, batch):
    """Inception-v3 on 3x299x299 inputs (scripts/compile/compile.py:27-36): one-sided and unpadded
    filters on the CUDA-core kernel, 1x1 and padded 3x3 filters on the tensor cores, concatenation
    by placement, padding-counting average pools; every convolution, pool and concatenation against
    the float64 oracle with the fp32 bound."""
    ex = gpx.BaseExecutor()
    ex.init("inception_v3", batch=batch, seed=1)
    threads = {ex.model.get_kernel_info(i)["launch_params"][3] for i in range(ex.get_kernel_num())}
    assert max(threads) > 256, "no tensor-core kernel was selected"
    data = gpx.synth_normal(batch * 3 * 299 * 299, 0, 0).reshape(batch, 3, 299, 299)
    ex.set_input("data", data)
    ex.execute()
    assert ex.error() == (0, 0)
    heads = ex.get_output("heads")
    taps = {}
    want = oracle.forward("inception_v3", ex.model.params(), data, taps=taps)
    assert heads.shape == want.shape == (batch, 1000)
    for name, ref in taps.items():
        got = ex.model.get(name).reshape(ref.shape)
        assert _rel(got, ref) <= RTOL_FP32, f"inception_v3 b{batch} node {name}: {_rel(got, ref):.2e}"
    assert _rel(heads, want) <= RTOL_FP32
    ex.clear()


def test_inception_v3_bfloat16_and_preempt_resume(gpx, oracle):
    base = gpx.BaseExecutor()
    base.init("inception", batch=4, seed=1, dtype="bfloat16")   # the name the reference's configs use
    data = gpx.synth_normal(4 * 3 * 299 * 299, 0, 0).reshape(4, 3, 299, 299)
    base.set_input("data", data)
    base.execute()
    want = base.get_output("heads")
    ref = oracle.forward("inception_v3", base.model.params(), data[:1])
    assert _rel(want[:1], ref) <= RTOL_16BIT
    word = gpx.PreemptWord(1)
    ex = gpx.BLPExecutor()
    ex.init("inception_v3", batch=4, dtype="bfloat16")
    for k, v in base.model.params().items():
        ex.model.set(k, v)
    ex.set_word(word)
    ex.set_input("data", data)
    s = gpx.Stream(1)
    t0 = time.perf_counter()
    ex.execute(s)
    s.sync()
    run_us = (time.perf_counter() - t0) * 1e6
    rng = np.random.default_rng(8)
    stops = 0
    for trial in range(5):
        word.clear()
        time.sleep(0.001)
        ex.execute(s)
        rounds = 0
        while True:
            if rounds < 4:
                delay = float(rng.uniform(0, run_us / 2))
                t0 = time.perf_counter()
                while (time.perf_counter() - t0) * 1e6 < delay:
                    pass
                word.raise_()
            s.sync()
            word.clear()
            time.sleep(0.0005)
            stop = ex.resume(s)
            rounds += 1
            if stop == -1:
                break
            stops += 1
            assert rounds < 60
        s.sync()
        assert np.array_equal(ex.get_output("heads"), want), f"trial {trial}"
    assert stops > 0
    base.clear(), ex.clear(), word.destroy(), s.destroy()


@pytest.mark.parametrize("name,model", [("vgg", "vgg19"), ("resnet152", "resnet152")])
def test_reference_config_models_at_batch_one_match_oracle(gpx, oracle, name, model):
    """The two models of the reference's config/A.json under the names that file uses (`vgg`,
    `resnet152`), batch 1 fp32 as the reference compiles them (scripts/compile/compile.py:27-31):
    logits against the CPU forward of the same graph."""
    ex = gpx.BaseExecutor()
    ex.init(name, batch=1, seed=3)
    data = _data(gpx, 1, seed=4)
    ex.set_input("data", data)
    ex.execute()
    got = ex.get_output("heads")
    want = oracle.forward(model, ex.model.params(), data, fast=True)
    assert got.shape == want.shape == (1, 1000)
    assert _rel(got, want) <= RTOL_FP32
    ex.clear()
