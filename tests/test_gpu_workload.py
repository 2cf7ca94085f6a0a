"""The workload driver end to end: every client policy on a small two-tenant config."""
import json

import pytest

pytestmark = pytest.mark.gpu


def _config(seconds=1.0, be_requests=None, hp_rate=200.0, resident=False):
    be_load = {"type": "continuous", "priority": 1}
    cfg = {
        "time": seconds, "seed": 5, "warmup": 3, "standalone": 5, "resident_inputs": resident,
        "tasks": [
            {"id": "tiny_rt", "load": {"type": "poisson", "priority": 0, "frequency": hp_rate},
             "client": {"name": "tiny_rt", "model_name": "resnet_tiny", "priority": 0,
                        "batch_size": 1, "use_cuda_graph": True, "preprocess_time": 50}},
            {"id": "tiny_be", "load": be_load,
             "client": {"name": "tiny_be", "model_name": "resnet_tiny", "priority": 1,
                        "batch_size": 16, "use_cuda_graph": True, "preprocess_time": 0}},
        ],
    }
    if be_requests is not None:
        be_load["max_requests"] = be_requests
        cfg["end_when"] = "tiny_be"
        cfg["time"] = 60.0
    return cfg


REPORT_KEYS = ["avgThroughput(req/s)", "standAloneTotalLatency(us)", "avgPrepareInputLatency(us)",
               "avgPreprocessLatency(us)", "avgCopyInputLatency(us)", "avgInferLatency(us)",
               "avgCopyOutputLatency(us)", "avgPostprocessLatency(us)", "avgTotalLatency(us)",
               "avgTotalLatencyIncrease(us)"]  # third_party/disb/src/analyzer.cpp:154-168


@pytest.mark.parametrize("client", ["gpreemptclient", "gpreemptclient_wo", "blpclient",
                                    "baseclient", "seqclient", "reefclient"])
def test_policy_runs_and_reports(gpx, client):
    rep = json.loads(gpx.run_workload(client, json.dumps(_config())))
    tasks = {t["id"]: t for t in rep["tasks"]}
    assert set(tasks) == {"tiny_rt", "tiny_be"}
    for t in tasks.values():
        for k in REPORT_KEYS:
            assert k in t, k
        assert t["requests"] > 0
        assert t["totalLatency(us)"]["p99"] >= t["totalLatency(us)"]["p50"] > 0
    # Poisson at 200 req/s for 1 s: late arrivals are dropped, never duplicated
    assert 100 <= tasks["tiny_rt"]["requests"] <= 300
    assert tasks["tiny_rt"]["avgPreprocessLatency(us)"] >= 50
    g = rep["gpus"][0]
    assert rep["drop_tile_in_flight"] is (client == "reefclient")
    if client in ("gpreemptclient", "gpreemptclient_wo", "blpclient", "reefclient"):
        assert g["wordRaises"] > 0
        assert g["beResumes"] >= 0
    else:
        assert g["wordRaises"] == 0


def test_rtonly_filters_best_effort_tasks(gpx):
    rep = json.loads(gpx.run_workload("rtonlyclient", json.dumps(_config(0.5))))
    assert [t["id"] for t in rep["tasks"]] == ["tiny_rt"]


def test_step_bounded_run_executes_exactly_k_best_effort_requests(gpx):
    rep = json.loads(gpx.run_workload("gpreemptclient", json.dumps(_config(be_requests=40, resident=True))))
    tasks = {t["id"]: t for t in rep["tasks"]}
    assert tasks["tiny_be"]["requests"] == 40
    assert tasks["tiny_be"]["deviceSpan(ms)"] > 0
    assert rep["resident_inputs"] is True


def test_unknown_client_and_bad_config(gpx):
    from gpreempt_b200 import binding as B

    with pytest.raises(gpx.GpxError) as e:
        gpx.run_workload("nosuchclient", json.dumps(_config()))
    assert e.value.status == B.NOT_FOUND
    with pytest.raises(gpx.GpxError) as e:
        gpx.run_workload("baseclient", "{not json")
    assert e.value.status == B.FAIL
    with pytest.raises(gpx.GpxError):
        gpx.run_workload("baseclient", json.dumps({"time": 1, "tasks": []}))


@pytest.mark.parametrize("name", ["C1_resnet50_contention", "C3_bert_vs_vgg16", "C4_mix_vs_densenet_bert"])
def test_shipped_contention_configs_run(gpx, name):
    """The contention configurations shipped under config/ (models, batches, dtypes and loads of
    the baseline's configs 1, 3 and 4) run under the GP policy: every tenant serves requests, the
    best-effort tenants are preempted and resumed, latency-critical tail stays finite."""
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "config", name + ".json")
    cfg = json.load(open(path))
    cfg["time"] = 2.0
    cfg["warmup"] = 2
    cfg["standalone"] = 3
    rep = json.loads(gpx.run_workload("gpreemptclient", json.dumps(cfg)))
    tasks = {t["id"]: t for t in rep["tasks"]}
    assert set(tasks) == {t["id"] for t in cfg["tasks"]}
    for t in tasks.values():
        assert t["requests"] > 0, t["id"]
        assert t["totalLatency(us)"]["p99"] > 0
    g = rep["gpus"][0]
    assert g["wordRaises"] > 0
    assert g["beResumes"] > 0


def test_input_double_buffering_keeps_results_and_counts(gpx):
    """`prefetch_inputs`: the best-effort tenant stages its next input while a request runs; the
    run serves the same number of step-bounded requests and reports the shorter copy phase."""
    base = _config(be_requests=30)
    rep0 = json.loads(gpx.run_workload("gpreemptclient", json.dumps(base)))
    cfg = _config(be_requests=30)
    cfg["prefetch_inputs"] = True
    rep1 = json.loads(gpx.run_workload("gpreemptclient", json.dumps(cfg)))
    assert rep1["prefetch_inputs"] is True and rep0["prefetch_inputs"] is False
    t0 = {t["id"]: t for t in rep0["tasks"]}
    t1 = {t["id"]: t for t in rep1["tasks"]}
    assert t1["tiny_be"]["requests"] == t0["tiny_be"]["requests"] == 30
    assert t1["tiny_be"]["avgCopyInputLatency(us)"] < t0["tiny_be"]["avgCopyInputLatency(us)"]
    assert t1["tiny_rt"]["requests"] > 0
