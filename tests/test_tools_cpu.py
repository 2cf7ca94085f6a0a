"""The command-line tools of the package (model_bench, hint_sweep, contention, microbench): their
argument formats and the configurations they generate, checked without a GPU."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_model_bench_spec_format():
    from gpreempt_b200 import model_bench as mb

    assert mb.parse_specs("resnet50:32:float32") == [("resnet50", 32, "float32", 0)]
    assert mb.parse_specs("bert_base:1:float16:128, vgg16:16:float16") == [
        ("bert_base", 1, "float16", 128), ("vgg16", 16, "float16", 0)]
    for bad in ("resnet50", "resnet50:32", "resnet50:32:int8", "a:1:float32:8:9"):
        with pytest.raises(ValueError):
            mb.parse_specs(bad)
    # the default list is the set of models and shapes the contention configurations use
    specs = {(m, b, d) for m, b, d, _ in mb.DEFAULT}
    assert ("resnet50", 32, "float32") in specs and ("densenet201", 64, "bfloat16") in specs
    assert ("bert_base", 32, "bfloat16") in specs and ("vgg16", 16, "float16") in specs


def test_hint_sweep_generates_the_reference_schema():
    from gpreempt_b200 import hint_sweep as hs

    cfg = hs.config(0, 4.0, 100.0, 300, True, 100, 32)
    assert cfg["hint_lead_us"] == 100 and cfg["preempt_hint"] is True
    ids = [t["id"] for t in cfg["tasks"]]
    assert ids == ["resnet50_rt", "resnet50_be"]
    for t in cfg["tasks"]:   # keys FooClient reads (src/cuda-clients/gpreemptclient.cpp:119-130)
        assert {"name", "model_name", "priority", "preprocess_time", "use_cuda_graph"} <= set(t["client"])
        assert t["load"]["type"] in ("poisson", "continuous")
    assert cfg["tasks"][0]["client"]["preprocess_time"] == 300
    json.dumps(cfg)


def test_shipped_configurations_follow_the_reference_schema():
    cfg_dir = os.path.join(ROOT, "config")
    names = sorted(f for f in os.listdir(cfg_dir) if f.endswith(".json"))
    assert {"C0_resnet50_solo.json", "C1_resnet50_contention.json", "C3_bert_vs_vgg16.json",
            "C4_mix_vs_densenet_bert.json"} <= set(names)
    for n in names:
        cfg = json.load(open(os.path.join(cfg_dir, n)))
        assert cfg["time"] > 0 and cfg["tasks"], n
        for t in cfg["tasks"]:
            assert {"id", "load", "client"} <= set(t), n
            assert t["load"]["type"] in ("continuous", "periodic", "poisson", "trace", "burst", "dependent"), n
            assert {"name", "model_name", "priority"} <= set(t["client"]), n
            assert t["client"]["priority"] in (0, 1), n


def test_bench_workload_config_is_the_baseline_configuration():
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    cfg = bench.workload_config(0, 100, 10, True)
    hp, be = cfg["tasks"]
    assert hp["client"]["model_name"] == be["client"]["model_name"] == "resnet50"
    assert hp["client"]["batch_size"] == 1 and be["client"]["batch_size"] == 32
    assert hp["load"] == {"type": "poisson", "priority": 0, "frequency": 100.0}
    assert be["load"]["max_requests"] == 100 and cfg["end_when"] == "resnet50_be"
    assert bench.BATCHES_PER_STEP * bench.BE_BATCH == 1600
    assert bench.LATENCY_RUN_S == 10.0 and bench.MICROBENCH_TRIGGERS == 1000
    assert bench.MICROBENCH_AXPY_ELEMS * 4 == 4 << 30   # 4 GiB per vector
    # sum-of-layers roofline: a layer is bound by whichever of its two times is longer
    assert abs(bench.model_roofline_ms([(2e12, 1e9), (1e9, 6.5e9)], 1000.0, 6500.0) - (2.0 + 1.0)) < 1e-9


def test_reference_workloads_tool_arguments_and_task_lists():
    from gpreempt_b200 import reference_workloads as rw

    assert set(rw.WORKLOADS) == {"A", "B", "C", "D", "E", "Y", "Z"}
    for name, tasks in rw.WORKLOADS.items():
        n_lc = 5 if name in "DE" else 1
        assert all(t["client"]["priority"] == 0 and t["id"].endswith("_rt") for t in tasks[:n_lc])
        assert all(t["client"]["priority"] == 1 for t in tasks[n_lc:])
        kind = "poisson" if name == "E" else "periodic"
        assert all(t["load"]["type"] == kind and t["client"]["batch_size"] == 1 for t in tasks)
    assert [t["load"]["frequency"] for t in rw.WORKLOADS["D"]] == [20] * 5 + [100] * 5
    assert [t["client"]["model_name"] for t in rw.WORKLOADS["Z"][1:]] == ["bfs", "sssp", "pagerank", "cc"]
    assert all("graph_path" in t["client"] and not t["client"]["use_cuda_graph"] for t in rw.WORKLOADS["Z"][1:])
    assert [t["load"]["frequency"] for t in rw.WORKLOADS["B"]] == [220, 220]
    assert len(rw.WORKLOADS["C"]) == 6
    assert rw.WORKLOADS["Y"][1]["client"]["model_name"] == "miniweather"
    res = subprocess.run([sys.executable, "-m", "gpreempt_b200.reference_workloads", "--only", "Q"],
                         capture_output=True, text=True, cwd=ROOT)
    assert res.returncode != 0 and "unknown workload" in res.stderr
