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


def _task(tid, model, priority, load, batch=1, preprocess=0, graph=True):
    return {"id": tid, "load": load,
            "client": {"name": tid, "model_name": model, "priority": priority, "batch_size": batch,
                       "use_cuda_graph": graph, "preprocess_time": preprocess}}


def test_trace_load_follows_its_arrival_list_and_drops_late_arrivals(gpx):
    """Trace load (third_party/disb/src/load.cpp:258-297): arrivals at the listed millisecond
    offsets; one whose successor has already arrived is given up."""
    trace = [0, 20, 40, 40.01, 40.02, 80, 120]   # three arrivals within 20 us: two of them cannot be served
    cfg = {"time": 0.4, "seed": 1, "warmup": 2, "standalone": 2,
           "tasks": [_task("tiny_rt", "resnet_tiny", 0, {"type": "trace", "priority": 0, "trace": trace})]}
    rep = json.loads(gpx.run_workload("baseclient", json.dumps(cfg)))
    t = rep["tasks"][0]
    assert t["requests"] + t["droppedArrivals"] == len(trace)
    assert t["droppedArrivals"] >= 1
    assert 4 <= t["requests"] <= 6
    assert t["firstLaunchOffset(us)"] < 5000


def test_periodic_load_counts_dropped_arrivals_when_it_cannot_keep_up(gpx):
    """Periodic load (load.cpp:143-177): at 200 Hz every arrival is served; at a rate far above what
    the model sustains, late arrivals are dropped and served + dropped covers the whole period."""
    ok = {"time": 0.5, "seed": 1, "warmup": 2, "standalone": 2,
          "tasks": [_task("tiny_rt", "resnet_tiny", 0, {"type": "periodic", "priority": 0, "frequency": 200})]}
    rep = json.loads(gpx.run_workload("baseclient", json.dumps(ok)))
    t = rep["tasks"][0]
    assert 95 <= t["requests"] <= 101 and t["droppedArrivals"] <= 2
    fast = {"time": 0.5, "seed": 1, "warmup": 2, "standalone": 2,
            "tasks": [_task("r50_rt", "resnet50", 0, {"type": "periodic", "priority": 0, "frequency": 20000})]}
    rep = json.loads(gpx.run_workload("baseclient", json.dumps(fast)))
    t = rep["tasks"][0]
    assert t["droppedArrivals"] > t["requests"] > 50
    assert 0.9 * 10000 <= t["requests"] + t["droppedArrivals"] <= 10100


def test_load_coordinator_staggers_equal_frequency_periodic_loads(gpx):
    """builtinLoadCoordinator (load.cpp:47-69): periodic loads whose load priority is 0 and whose
    frequencies are equal start one stand-alone latency after one another."""
    cfg = {"time": 0.5, "seed": 1, "warmup": 2, "standalone": 3,
           "tasks": [_task("a_rt", "resnet_tiny", 0, {"type": "periodic", "priority": 0, "frequency": 100}, preprocess=100),
                     _task("b_rt", "resnet_tiny", 0, {"type": "periodic", "priority": 0, "frequency": 100}, preprocess=100),
                     _task("c_rt", "resnet_tiny", 0, {"type": "periodic", "priority": 0, "frequency": 50}),
                     _task("d_be", "resnet_tiny", 1, {"type": "periodic", "priority": 1, "frequency": 100})]}
    rep = json.loads(gpx.run_workload("baseclient", json.dumps(cfg)))
    t = {x["id"]: x for x in rep["tasks"]}
    assert t["a_rt"]["launchDelay(us)"] == 0
    assert abs(t["b_rt"]["launchDelay(us)"] - t["a_rt"]["standAloneTotalLatency(us)"]) <= 2
    assert t["b_rt"]["launchDelay(us)"] >= 100
    assert t["c_rt"]["launchDelay(us)"] == 0      # another frequency
    assert t["d_be"]["launchDelay(us)"] == 0      # load priority 1 is not coordinated
    assert t["b_rt"]["firstLaunchOffset(us)"] >= t["b_rt"]["launchDelay(us)"]


def test_dependent_load_runs_after_its_predecessors(gpx):
    """DependentLoad (load.cpp:299-361): a request is launched once each task in prev_task_ids
    has delivered the result with the same serial number."""
    cfg = {"time": 0.5, "seed": 1, "warmup": 2, "standalone": 2,
           "tasks": [_task("det_rt", "resnet_tiny", 0, {"type": "periodic", "priority": 0, "frequency": 100}),
                     _task("aux_rt", "resnet_tiny", 0, {"type": "periodic", "priority": 0, "frequency": 50}),
                     _task("post_rt", "resnet_tiny", 0, {"type": "dependent", "prev_task_ids": ["det_rt", "aux_rt"]})]}
    rep = json.loads(gpx.run_workload("baseclient", json.dumps(cfg)))
    t = {x["id"]: x for x in rep["tasks"]}
    assert 0 < t["post_rt"]["requests"] <= min(t["det_rt"]["requests"], t["aux_rt"]["requests"])
    assert t["post_rt"]["requests"] >= t["aux_rt"]["requests"] - 2
    bad = dict(cfg, tasks=[_task("post_rt", "resnet_tiny", 0, {"type": "dependent", "prev_task_ids": ["nobody"]})])
    from gpreempt_b200 import binding as B
    with pytest.raises(gpx.GpxError) as e:
        gpx.run_workload("baseclient", json.dumps(bad))
    assert e.value.status == B.NOT_FOUND


def test_hint_lead_time_lowers_latency_critical_inference_latency(gpx):
    """Hint-based pre-preemption (src/cuda-clients/gpreemptclient.cpp:21,203-219): with 300 us of
    host preprocessing, raising the word 100 us before the phase ends lets the best-effort kernels
    drain before the request is submitted, so its inference phase is shorter than without hints."""
    def run(client, lead):
        cfg = {"time": 2.0, "seed": 3, "warmup": 3, "standalone": 3, "hint_lead_us": lead,
               "tasks": [_task("r50_rt", "resnet50", 0, {"type": "poisson", "priority": 0, "frequency": 150}, preprocess=300),
                         _task("r50_be", "resnet50", 1, {"type": "continuous", "priority": 1}, batch=32)]}
        rep = json.loads(gpx.run_workload(client, json.dumps(cfg)))
        assert rep["hint_lead_us"] == lead
        t = {x["id"]: x for x in rep["tasks"]}
        assert t["r50_be"]["requests"] > 0
        return t["r50_rt"]["inferLatency(us)"]["p50"], rep["gpus"][0]

    without, g0 = run("gpreemptclient_wo", 0)
    with_lead, g1 = run("gpreemptclient", 100)
    assert g0["wordRaises"] > 0 and g1["wordRaises"] > 0
    assert with_lead < without, (with_lead, without)


def test_be_window_outside_its_range_is_rejected(gpx):
    from gpreempt_b200 import binding as B

    cfg = _config(0.2)
    cfg["be_window"] = 3
    with pytest.raises(gpx.GpxError) as e:
        gpx.run_workload("gpreemptclient", json.dumps(cfg))
    assert e.value.status == B.OUT_OF_RANGE
    cfg["be_window"] = 64
    with pytest.raises(gpx.GpxError):
        gpx.run_workload("gpreemptclient", json.dumps(cfg))
    cfg["be_window"] = 8
    rep = json.loads(gpx.run_workload("gpreemptclient", json.dumps(cfg)))
    assert rep["be_window"] == 8


def test_schedule_order_across_tenants_from_device_timestamps(gpx):
    """Schedule order under the dispatcher, from the device-side %globaltimer trace of every
    executor (latency-critical ones included) put on the host timeline:
      * a latency-critical request's first CTA starts after the word was raised for it;
      * a best-effort launch that was stopped saw the word after it was raised, and no kernel
        behind its stop point ran a tile;
      * a best-effort launch (first or resumed) starts no CTA before the word was cleared;
      * every best-effort request ran each tile of each kernel exactly once over its launches."""
    cfg = {"time": 2.0, "seed": 9, "warmup": 3, "standalone": 3, "schedule_log": True,
           "tasks": [_task("r50_rt", "resnet50", 0, {"type": "poisson", "priority": 0, "frequency": 200}),
                     _task("tiny_rt", "resnet_tiny", 0, {"type": "poisson", "priority": 0, "frequency": 100}),
                     _task("r50_be", "resnet50", 1, {"type": "continuous", "priority": 1}, batch=16, graph=False),
                     _task("mnet_be", "mobilenet_v2", 1, {"type": "continuous", "priority": 1}, batch=8, graph=False)]}
    rep = json.loads(gpx.run_workload("gpreemptclient", json.dumps(cfg)))
    lg = rep["gpus"][0]["scheduleLog"]
    ev = lg["events"]
    o0, o1 = lg["offset_before_rel_ns"], lg["offset_after_rel_ns"]
    t0, t1 = lg["offset_before_at_rel_ns"], lg["offset_after_at_rel_ns"]
    slack = lg["uncertainty_ns"] + 30_000  # clock correlation, its drift between measurements, call overheads

    def to_host(dev_rel, near_host_rel):
        frac = min(max((near_host_rel - t0) / max(t1 - t0, 1), 0.0), 1.0)
        return dev_rel + o0 + (o1 - o0) * frac

    last_raise = last_clear = None
    raised = False
    be_start = {}
    hp_checked = stops = be_done = be_starts_checked = 0
    for e in ev:
        kind, client = e[0], e[1]
        if kind == 0:
            last_raise, raised = e[2], True
        elif kind == 1:
            last_clear, raised = e[2], False
        elif kind == 2:
            first, last, submit, launch = e[2], e[3], e[4], e[5]
            assert last_raise is not None and last_raise <= launch + 1000, "launched before the word was raised"
            assert to_host(first, launch) + slack >= last_raise, "a latency-critical CTA started before the raise"
            assert last >= first
            hp_checked += 1
        elif kind == 3:
            assert not raised, "a best-effort launch was issued while the word was up"
            be_start[client] = (e[2], last_clear)
        elif kind in (4, 5):
            started_at, cleared_at = be_start[client]
            if e[2] >= 0 and cleared_at is not None:
                assert to_host(e[2], started_at) + slack >= cleared_at, "a best-effort CTA started before the clear"
                be_starts_checked += 1
            if kind == 4:
                stop_kernel, seen, behind = e[3], e[4], e[5]
                assert behind == 0, "a kernel behind the stop point ran a tile"
                if seen >= 0:
                    assert to_host(seen, started_at) + slack >= last_raise, "the stopped kernel saw the word before the raise"
                stops += 1
            else:
                assert e[3] == 0, "a best-effort request did not run every tile exactly once"
                be_done += 1
    assert hp_checked > 100 and stops > 20 and be_done > 20 and be_starts_checked > 20


def test_reference_model_names_and_client_keys_run_unchanged(gpx):
    """A task list written the way the reference's own configurations are (config/A.json,
    config/C.json: model names vgg / resnet152 / densenet / inception / bert, batch 1, the
    tfs_grpc_addr / triton_grpc_addr keys no client reads, periodic loads that carry their own
    priority key): every task is served under the GP policy."""
    def client(name, model, prio):
        return {"name": name, "model_name": model, "priority": prio, "batch_size": 1,
                "tfs_grpc_addr": "localhost:8500", "triton_grpc_addr": "localhost:8001",
                "use_cuda_graph": True, "preprocess_time": 200}

    tasks = []
    for model in ("vgg", "resnet152", "densenet", "inception", "bert"):
        tasks.append({"id": model + "_rt", "load": {"type": "periodic", "priority": 0, "frequency": 20},
                      "client": client(model + "_rt", model, 0)})
    tasks.append({"id": "resnet152_be", "load": {"type": "periodic", "priority": 0, "frequency": 100},
                  "client": client("resnet152_be", "resnet152", 1)})
    cfg = {"time": 1.5, "warmup": 2, "standalone": 2, "tasks": tasks}
    rep = json.loads(gpx.run_workload("gpreemptclient", json.dumps(cfg)))
    t = {x["id"]: x for x in rep["tasks"]}
    assert set(t) == {x["id"] for x in tasks}
    for x in t.values():
        assert x["requests"] > 0 and x["avgPreprocessLatency(us)"] >= 200, x["id"]
    # equal-frequency periodic latency-critical loads are staggered (builtinLoadCoordinator)
    delays = sorted(t[m + "_rt"]["launchDelay(us)"] for m in ("vgg", "resnet152", "densenet", "inception", "bert"))
    assert delays[0] == 0 and delays[1] > 0
