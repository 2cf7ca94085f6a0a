"""Model directories in the reference's formats (mod.json + host.json + mod.params,
src/model.cpp:15-55,128-235): a model exported with gpx_model_export_dir and opened again from the
directory has the same storages, the same kernel list and produces the same output bit for bit."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _input(gpx, model, batch, seq):
    if model.startswith("bert"):
        return np.random.default_rng(6).integers(0, 1000, (batch, seq)).astype(np.int64)
    return gpx.synth_normal(batch * 3 * 224 * 224, 0, 0).reshape(batch, 3, 224, 224)


@pytest.mark.parametrize("model,batch,dtype,seq", [("resnet_tiny", 2, "float32", 0), ("resnet50", 1, "float32", 0),
                                                   ("mobilenet_v2", 1, "bfloat16", 0), ("densenet_tiny", 2, "float32", 0),
                                                   ("bert_tiny", 2, "float16", 64), ("vgg16", 1, "float16", 0)])
def test_exported_directory_loads_back_bit_identical(gpx, tmp_path, model, batch, dtype, seq):
    a = gpx.BaseExecutor()
    a.init(model, batch=batch, seed=3, dtype=dtype, seq_len=seq)
    d = str(tmp_path / model)
    a.model.export_dir(d)
    assert sorted(os.listdir(d)) == ["host.json", "mod.json", "mod.params"]
    graph = json.load(open(os.path.join(d, "mod.json")))
    host = json.load(open(os.path.join(d, "host.json")))
    # the skeleton Model::load_from_json walks
    assert graph["nodes"][graph["heads"][0][0]]["name"] == "heads"
    assert len(graph["attrs"]["dltype"][1]) == len(graph["attrs"]["shape"][1]) == len(graph["nodes"])
    funcs = [n["attrs"]["func_name"] for n in graph["nodes"] if n["inputs"]]
    assert [f["name"] for f in host["funcs"]] == funcs
    for f in host["funcs"]:
        for k in f["kernels"]:
            assert len(k["launch_params"]) == 6 and all(isinstance(i, int) for i in k["args"])
    assert all(isinstance(t, int) and t > 0 for t in host["temp_args"])

    b = gpx.BaseExecutor()
    b.dtype = dtype
    b.model = gpx.Model(d)           # the directory form of Model::load_model; parameters come with it
    from gpreempt_b200 import binding as B
    import ctypes
    B.check(B.load().gpx_exec_create(b.model.handle, B.EXEC_BASE, ctypes.byref(b.handle)))
    assert b.get_kernel_num() == a.get_kernel_num()
    for i in range(a.get_kernel_num()):
        ka, kb = a.model.get_kernel_info(i), b.model.get_kernel_info(i)
        assert ka["name"] == kb["name"] and ka["launch_params"] == kb["launch_params"] and ka["total_tiles"] == kb["total_tiles"]
    pa, pb = a.model.params(), b.model.params()
    assert list(pa) == list(pb)
    for k in pa:
        assert np.array_equal(pa[k], pb[k]), k
    x = _input(gpx, model, batch, seq)
    for ex in (a, b):
        ex.set_input("data", x)
        ex.execute()
        assert ex.error() == (0, 0)
    assert np.array_equal(a.get_output("heads"), b.get_output("heads"))
    # and the seeded initialiser visits the parameters of a loaded graph in the same order
    a.model.init_random(11)
    b.model.init_random(11)
    pa, pb = a.model.params(), b.model.params()
    for k in pa:
        assert np.array_equal(pa[k], pb[k]), k
    a.clear(), b.clear()


def test_directory_errors_are_reported_not_fatal(gpx, tmp_path):
    from gpreempt_b200 import binding as B

    a = gpx.Model("resnet_tiny")
    d = str(tmp_path / "m")
    a.export_dir(d)
    a.clear()
    # a graph without this library's operator attributes (what a TVM-written mod.json looks like)
    g = json.load(open(os.path.join(d, "mod.json")))
    del g["gpx"]
    d2 = str(tmp_path / "tvm_like")
    os.makedirs(d2)
    json.dump(g, open(os.path.join(d2, "mod.json"), "w"))
    with pytest.raises(gpx.GpxError) as e:
        gpx.Model(d2)
    assert e.value.status == B.NOT_FOUND and "mod.cu" in str(e.value)
    # host.json naming another function: the reference's "Function name mismatch"
    h = json.load(open(os.path.join(d, "host.json")))
    h["funcs"][0]["name"] = "tvmgen_default_fused_nn_conv2d"
    json.dump(h, open(os.path.join(d, "host.json"), "w"))
    with pytest.raises(gpx.GpxError) as e:
        gpx.Model(d)
    assert e.value.status == B.FAIL and "Function name mismatch" in str(e.value)
    # a batch the directory was not exported for
    with pytest.raises(gpx.GpxError) as e:
        gpx.Model(d, batch=4)
    assert e.value.status == B.OUT_OF_RANGE
