"""The graph-analytics best-effort workloads (bfs, sssp, cc, pagerank) on the GPU: parity with the
CPU oracle and with the reference's own kernels, preempt/resume, and a tenant in the shape of the
reference's config/Z.json."""
import json
import os
import time

import numpy as np
import pytest

from gpreempt_b200 import graph_files

pytestmark = pytest.mark.gpu

ALGOS = ("bfs", "sssp", "cc", "pagerank")
RESULT = {"bfs": "label", "sssp": "cost", "cc": "comp", "pagerank": "value"}
# PageRank is float arithmetic with a threshold: a vertex whose residual is within rounding of the
# tolerance (0.001) may be pushed in one evaluation and held back in another, which moves its value
# by at most that residual; everything else differs by summation order only.
PAGERANK_ATOL = 1.1e-3
PAGERANK_MEAN_ATOL = 1e-5


def _oracle():
    from oracle import graphs

    graphs.build()
    return graphs


@pytest.fixture(scope="module")
def graphs_on_disk(tmp_path_factory):
    """Three graphs: small with four components, medium, and one of the size of the reference's
    dataset (crankseg_1: 52 804 vertices, ~10.6 M edges)."""
    root = tmp_path_factory.mktemp("graphs")
    out = {}
    for name, (v, deg, band, seed, comps) in {"small": (1500, 30, 100, 5, 4), "medium": (20000, 64, 400, 2, 1),
                                              "crank": (52804, 201, 1500, 1, 1)}.items():
        prefix = str(root / name / (name + ".bel"))
        graph_files.write_synthetic(prefix, v, deg, band, seed, comps)
        out[name] = prefix
    return out


def _expected(prefix):
    g = _oracle()
    offsets, neighbours, weights = graph_files.read_bel(prefix)
    return {"bfs": g.bfs(offsets, neighbours)[0], "sssp": g.sssp(offsets, neighbours, weights)[0],
            "cc": g.cc(offsets, neighbours)[0], "pagerank": g.pagerank(offsets, neighbours)[0]}


def _check(algo, got, want, what):
    if algo == "pagerank":
        err = np.abs(got.astype(np.float64) - want.astype(np.float64))
        assert err.max() <= PAGERANK_ATOL and err.mean() <= PAGERANK_MEAN_ATOL, \
            f"{what}: pagerank differs by max {err.max():.3e}, mean {err.mean():.3e}"
    else:
        assert np.array_equal(got.astype(np.uint64), want.astype(np.uint64)), \
            f"{what}: {algo} differs at {np.flatnonzero(got.astype(np.uint64) != want.astype(np.uint64))[:5]}"


@pytest.mark.parametrize("which", ["small", "medium", "crank"])
def test_results_match_oracle(gpx, graphs_on_disk, which):
    prefix = graphs_on_disk[which]
    want = _expected(prefix)
    for algo in ALGOS:
        ex = gpx.BaseExecutor()
        ex.set_graph_path(prefix)
        ex.init(algo)
        info = ex.model.graph_info()
        assert info["vertices"] == len(want["bfs"]) and info["edges"] > 0
        for run in range(2):  # every run starts from its own initial state
            ex.execute()
            got = ex.model.get(RESULT[algo])
            _check(algo, got, want[algo], f"{which} run {run}")
            info = ex.model.graph_info()
            assert info["converged"]
            # the list was sized by a run of the same, race-free iterations: two spare at the end
            assert info["live_iterations"] == info["listed_iterations"] - 2 or \
                (algo == "pagerank" and info["listed_iterations"] == 100)
        if algo == "bfs":
            assert info["live_iterations"] == int(want["bfs"][want["bfs"] != 0xFFFFFFFF].max()) + 1
        ex.clear()


def test_matches_the_reference_kernels(gpx, graphs_on_disk):
    """GraphComputeRaw::{BFS,SSSP,CC,PageRank}::compute of the reference, compiled unmodified, on the
    same files: labels, distances and components are identical, ranks agree within the tolerance."""
    g = _oracle()
    if not g.reference_available():
        pytest.skip("oracle/_ref/libgraphcompute_ref.so was not built (needs the reference checkout)")
    for which in ("small", "crank"):
        prefix = graphs_on_disk[which]
        for algo in ALGOS:
            ref = g.Reference(algo, prefix)
            ref.compute(1)
            want = ref.result()
            ref_ms = ref.compute(5) / 5
            ref.close()
            ex = gpx.BaseExecutor()
            ex.set_graph_path(prefix)
            ex.init(algo)
            ex.execute()
            got = ex.model.get(RESULT[algo])
            _check(algo, got, want, f"{which} vs reference")
            s = gpx.Stream(0)
            ex.capture_graph(s)
            ex.execute(s)
            s.sync()
            t0 = time.perf_counter()
            for _ in range(5):
                ex.execute(s)
            s.sync()
            ms = (time.perf_counter() - t0) * 1e3 / 5
            print(f"{which} {algo}: reference {ref_ms:.3f} ms per run, this library {ms:.3f} ms "
                  f"({ex.model.graph_info()['live_iterations']} iterations)")
            _check(algo, ex.model.get(RESULT[algo]), want, f"{which} graph launch vs reference")
            ex.clear(), s.destroy()


def test_preempt_resume_bit_identical(gpx, graphs_on_disk):
    """execute, raise the word mid-run, drain, clear, resume until done (the loop of
    GraphComputeBlp::*::compute, src/workloads/graphcompute.tr.cu:160-178, driven from outside): the
    results equal the uninterrupted run bit for bit - PageRank too, its sums have a fixed order."""
    prefix = graphs_on_disk["crank"]
    for algo in ALGOS:
        base = gpx.BaseExecutor()
        base.set_graph_path(prefix)
        base.init(algo)
        base.execute()
        want = base.model.get(RESULT[algo])
        base.clear()

        word = gpx.PreemptWord(0)
        ex = gpx.BLPExecutor()
        ex.set_graph_path(prefix)
        ex.init(algo)
        ex.set_word(word)
        ex.enable_trace(True)
        s = gpx.Stream(1)
        nk = ex.get_kernel_num()
        tiles = np.array([ex.model.get_kernel_info(i)["total_tiles"] for i in range(nk)])
        t0 = time.perf_counter()
        ex.execute(s)
        s.sync()
        run_us = (time.perf_counter() - t0) * 1e6
        assert np.array_equal(ex.read_trace()[:, 3].astype(np.int64), tiles), algo
        assert np.array_equal(ex.model.get(RESULT[algo]), want), algo
        rng = np.random.default_rng(7)
        stops_seen = 0
        for trial in range(6):
            word.clear()
            time.sleep(0.001)
            ex.execute(s)
            rounds = 0
            while True:
                if rounds < 6:
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
                stops_seen += 1
                assert 0 <= stop < nk and rounds < 100
            s.sync()
            assert np.all(ex.read_cursors() >= tiles)
            assert np.array_equal(ex.model.get(RESULT[algo]), want), f"{algo} trial {trial}"
            assert ex.model.graph_info()["converged"]
        assert stops_seen > 0, f"{algo}: no run was ever preempted"
        # the same from a captured CUDA graph (a best-effort client with use_cuda_graph): the first
        # launch is one graph launch, what a preemption leaves over is relaunched kernel by kernel
        ex.capture_graph(s)
        for trial in range(3):
            word.clear()
            time.sleep(0.001)
            ex.execute(s)
            delay = float(rng.uniform(0, run_us / 2))
            t0 = time.perf_counter()
            while (time.perf_counter() - t0) * 1e6 < delay:
                pass
            word.raise_()
            s.sync()
            word.clear()
            time.sleep(0.0005)
            rounds = 0
            while ex.resume(s) != -1:
                rounds += 1
                assert rounds < 100
            s.sync()
            assert np.array_equal(ex.model.get(RESULT[algo]), want), f"{algo} graph launch, trial {trial}"
        ex.clear(), word.destroy(), s.destroy()


def test_names_paths_and_errors(gpx, graphs_on_disk, tmp_path, monkeypatch):
    prefix = graphs_on_disk["small"]
    m = gpx.Model("bfs:" + prefix)  # the name form behind set_graph_path
    assert m.graph_info()["vertices"] == 1500
    assert m.get_storage_info(m.find_storage_idx("label"))["stype"] == "uint32"
    with pytest.raises(gpx.GpxError):
        m.find_storage_idx("data")
    with pytest.raises(gpx.GpxError):
        m.export_json()
    with pytest.raises(gpx.GpxError):
        m.reductions()
    m.clear()
    # a relative path is looked up under GPX_GRAPH_BASE_PATH (GRAPH_BASE_PATH of the reference)
    monkeypatch.setenv("GPX_GRAPH_BASE_PATH", os.path.dirname(os.path.dirname(prefix)))
    m = gpx.Model("cc:small/small.bel")
    assert m.graph_info()["vertices"] == 1500
    m.clear()
    monkeypatch.delenv("GPX_GRAPH_BASE_PATH")
    for bad in ("bfs", "bfs:" + str(tmp_path / "nothing.bel")):
        with pytest.raises(gpx.GpxError):
            gpx.Model(bad)
    with pytest.raises(gpx.GpxError):
        gpx.Model("resnet_tiny").graph_info()
    # a file shorter than its header says
    offsets, neighbours, _ = graph_files.read_bel(prefix)
    cut = str(tmp_path / "cut.bel")
    graph_files.write_bel(cut, offsets, neighbours)
    with open(cut + ".dst", "r+b") as f:
        f.truncate(16 + 8 * (len(neighbours) // 2))
    with pytest.raises(gpx.GpxError):
        gpx.Model("cc:" + cut)
    with pytest.raises(gpx.GpxError):  # sssp needs the weights file
        gpx.Model("sssp:" + cut)


def test_isolated_vertices_and_tiny_graphs(gpx, tmp_path):
    """Vertices without edges, unreachable vertices, a graph of one vertex and one without any edge."""
    g = _oracle()
    cases = {
        # 0-1-2 chain, 3 isolated, 4-5 pair
        "six": (np.array([0, 1, 3, 4, 4, 5, 6], np.uint64), np.array([1, 0, 2, 1, 5, 4], np.uint64),
                np.array([7, 7, 2, 2, 1, 1], np.uint32)),
        "one": (np.array([0, 0], np.uint64), np.array([], np.uint64), np.array([], np.uint32)),
        "no_edges": (np.zeros(41, np.uint64), np.array([], np.uint64), np.array([], np.uint32)),
    }
    # a path of 2 500 vertices: as many search levels as vertices, i.e. a kernel list of thousands
    n = 2500
    deg = np.full(n, 2, np.int64)
    deg[[0, -1]] = 1
    path_off = np.concatenate([[0], np.cumsum(deg)]).astype(np.uint64)
    path_nb = np.empty(int(path_off[-1]), np.uint64)
    for v in range(n):
        path_nb[int(path_off[v]):int(path_off[v + 1])] = [u for u in (v - 1, v + 1) if 0 <= u < n]
    cases["path"] = (path_off, path_nb, (np.arange(len(path_nb)) % 5 + 1).astype(np.uint32))
    for name, (offsets, neighbours, weights) in cases.items():
        prefix = str(tmp_path / name / (name + ".bel"))
        graph_files.write_bel(prefix, offsets, neighbours, weights)
        want = {"bfs": g.bfs(offsets, neighbours)[0], "sssp": g.sssp(offsets, neighbours, weights)[0],
                "cc": g.cc(offsets, neighbours)[0]}
        for algo in ("bfs", "sssp", "cc"):
            ex = gpx.BaseExecutor()
            ex.set_graph_path(prefix)
            ex.init(algo)
            ex.execute()
            _check(algo, ex.model.get(RESULT[algo]), want[algo], name)
            assert ex.model.graph_info()["converged"]
            if name == "path" and algo == "bfs":
                assert ex.model.graph_info()["live_iterations"] == n and ex.get_kernel_num() == n + 3
            ex.clear()
        # pagerank: a vertex nobody points at keeps 1 - alpha (its own delta, infinite without
        # out-edges as in the reference, is never read)
        ex = gpx.BaseExecutor()
        ex.set_graph_path(prefix)
        ex.init("pagerank")
        ex.execute()
        rank = ex.model.get("value")
        assert np.all(np.isfinite(rank))
        if name in ("one", "no_edges"):
            assert np.allclose(rank, 1 - g.ALPHA)
        else:
            _check("pagerank", rank, g.pagerank(offsets, neighbours)[0], name)
        ex.clear()


def test_best_effort_tenants_under_a_latency_critical_model(gpx, graphs_on_disk, monkeypatch):
    """config/Z_graph_analytics.json, the shape of the reference's config/Z.json: the four graph
    workloads as periodic best-effort tenants (client key graph_path, relative to the dataset
    directory) under a latency-critical DNN."""
    prefix = graphs_on_disk["crank"]  # <root>/crank/crank.bel, as the shipped configuration names it
    monkeypatch.setenv("GPX_GRAPH_BASE_PATH", os.path.dirname(os.path.dirname(prefix)))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "config", "Z_graph_analytics.json")) as f:
        cfg = json.load(f)
    tasks = cfg["tasks"]
    assert [t["client"]["model_name"] for t in tasks] == ["vgg", "bfs", "sssp", "pagerank", "cc"]
    tasks[0]["client"]["graph_path"] = prefix  # ignored by a model that is not a graph workload
    cfg.update({"time": 1.5, "seed": 3, "warmup": 2, "standalone": 2})
    rep = json.loads(gpx.run_workload("gpreemptclient", json.dumps(cfg)))
    by_id = {t["id"]: t for t in rep["tasks"]}
    assert 130 <= by_id["vgg_rt"]["requests"] <= 151
    for algo in ALGOS:
        assert by_id[algo + "_be"]["requests"] > 30, algo
        assert by_id[algo + "_be"]["in_bytes"] == 0
    assert rep["gpus"][0]["wordRaises"] > 0
    # closed-loop tenants keep the GPU busy, so latency-critical requests do interrupt them
    for t in tasks[1:]:
        t["load"] = {"type": "continuous"}
    cfg["schedule_log"] = True
    rep = json.loads(gpx.run_workload("gpreemptclient", json.dumps(cfg)))
    by_id = {t["id"]: t for t in rep["tasks"]}
    assert 130 <= by_id["vgg_rt"]["requests"] <= 151
    assert sum(by_id[a + "_be"]["resumes"] for a in ALGOS) > 0
    assert all(by_id[a + "_be"]["requests"] > 100 for a in ALGOS)
    # from the device time stamps: nothing behind a stop point ran, and every finished request ran
    # each tile of each kernel once over its launches (the kernels behind the last live iteration count
    # theirs without running them)
    stops = done = 0
    for e in rep["gpus"][0]["scheduleLog"]["events"]:
        if e[0] == 4:
            assert e[5] == 0, "a kernel behind the stop point ran a tile"
            stops += 1
        elif e[0] == 5:
            assert e[3] == 0, "a best-effort request did not run every tile exactly once"
            done += 1
    assert stops > 0 and done > 400
