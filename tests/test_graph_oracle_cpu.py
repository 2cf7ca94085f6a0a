"""The graph-analytics CPU oracle against independent implementations (scipy.sparse.csgraph, a
dense power iteration) and the graph-file writer against the reference's reader layout."""
import os
import subprocess
import sys

import numpy as np
import pytest

from gpreempt_b200 import graph_files
from oracle import graphs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _csr(offsets, neighbours, weights=None):
    from scipy.sparse import csr_matrix

    data = np.ones(len(neighbours)) if weights is None else weights.astype(np.float64)
    n = len(offsets) - 1
    return csr_matrix((data, neighbours.astype(np.int64), offsets.astype(np.int64)), shape=(n, n))


@pytest.fixture(scope="module", params=[(600, 12, 40, 3, 1), (1500, 30, 100, 5, 4), (257, 6, 9, 11, 2)])
def graph(request):
    vertices, degree, band, seed, components = request.param
    offsets, neighbours = graph_files.synthetic_banded(vertices, degree, band, seed, components)
    weights = graph_files.synthetic_weights(len(neighbours), seed)
    return offsets, neighbours, weights, components


def test_synthetic_graph_is_symmetric_simple_and_has_the_asked_components(graph):
    offsets, neighbours, _, components = graph
    from scipy.sparse.csgraph import connected_components

    m = _csr(offsets, neighbours)
    assert (m != m.T).nnz == 0
    assert m.diagonal().sum() == 0
    assert m.max() == 1  # no duplicate edges
    assert connected_components(m, directed=False)[0] == components


def test_bfs_levels_match_scipy(graph):
    from scipy.sparse.csgraph import shortest_path

    offsets, neighbours, _, _ = graph
    label, launches = graphs.bfs(offsets, neighbours)
    hops = shortest_path(_csr(offsets, neighbours), unweighted=True, indices=0)
    want = np.where(np.isinf(hops), graphs.INFINITY, hops).astype(np.uint32)
    assert np.array_equal(label, want)
    assert launches == int(hops[np.isfinite(hops)].max()) + 1


def test_sssp_distances_match_dijkstra(graph):
    from scipy.sparse.csgraph import dijkstra

    offsets, neighbours, weights, _ = graph
    cost, _ = graphs.sssp(offsets, neighbours, weights)
    dist = dijkstra(_csr(offsets, neighbours, weights), directed=True, indices=0)
    want = np.where(np.isinf(dist), graphs.INFINITY, dist).astype(np.uint32)
    assert np.array_equal(cost, want)


def test_cc_labels_are_the_smallest_vertex_of_each_component(graph):
    from scipy.sparse.csgraph import connected_components

    offsets, neighbours, _, components = graph
    comp, _ = graphs.cc(offsets, neighbours)
    count, member = connected_components(_csr(offsets, neighbours), directed=False)
    assert count == components
    smallest = np.full(count, len(member), np.int64)
    np.minimum.at(smallest, member, np.arange(len(member)))
    assert np.array_equal(comp, smallest[member].astype(np.uint64))


def test_pagerank_is_the_residual_push_scheme_within_its_tolerance(graph):
    """The scheme pushes (1-a) a^k P^k 1 until the pushed amount of a vertex is below the tolerance, so it
    approaches (1-a) (I - a P^T)^-1 1 from below with at most tolerance / (1-a) missing per vertex."""
    offsets, neighbours, _, _ = graph
    value, iterations = graphs.pagerank(offsets, neighbours)
    n = len(offsets) - 1
    deg = np.diff(offsets.astype(np.int64)).astype(np.float64)
    p = _csr(offsets, neighbours).toarray() / deg[:, None]  # row-stochastic
    exact = (1 - graphs.ALPHA) * np.linalg.solve(np.eye(n) - graphs.ALPHA * p.T, np.ones(n))
    assert 1 < iterations <= graphs.MAX_ITER
    assert np.all(value <= exact + 1e-4)
    assert np.max(exact - value) < graphs.TOLERANCE / (1 - graphs.ALPHA) * 1.05


def test_isolated_and_unreachable_vertices():
    # 0-1-2 chain, 3 isolated, 4-5 pair
    offsets = np.array([0, 1, 3, 4, 4, 5, 6], np.uint64)
    neighbours = np.array([1, 0, 2, 1, 5, 4], np.uint64)
    weights = np.array([7, 7, 2, 2, 1, 1], np.uint32)
    label, _ = graphs.bfs(offsets, neighbours)
    assert label.tolist() == [0, 1, 2, graphs.INFINITY, graphs.INFINITY, graphs.INFINITY]
    cost, _ = graphs.sssp(offsets, neighbours, weights)
    assert cost.tolist() == [0, 7, 9, graphs.INFINITY, graphs.INFINITY, graphs.INFINITY]
    comp, _ = graphs.cc(offsets, neighbours)
    assert comp.tolist() == [0, 0, 0, 3, 4, 4]


def test_graph_files_have_the_layout_the_reference_reads(tmp_path):
    """read_graph (src/workloads/graphcompute.cu:15-45): u64 count, u64 type, then the elements; the
    vertex file holds vertices + 1 offsets."""
    offsets, neighbours = graph_files.synthetic_banded(100, 8, 10, 1)
    weights = graph_files.synthetic_weights(len(neighbours), 1)
    prefix = str(tmp_path / "g" / "g.bel")
    graph_files.write_bel(prefix, offsets, neighbours, weights)
    col = np.fromfile(prefix + ".col", np.uint64)
    dst = np.fromfile(prefix + ".dst", np.uint64)
    assert col[0] == 101 and len(col) == 2 + 101 and col[2] == 0 and col[-1] == len(neighbours)
    assert dst[0] == len(neighbours) and np.array_equal(dst[2:], neighbours)
    raw = open(prefix + ".val", "rb").read()
    assert int(np.frombuffer(raw[:8], np.uint64)[0]) == len(weights)
    assert np.array_equal(np.frombuffer(raw[16:], np.uint32), weights)
    o, d, w = graph_files.read_bel(prefix)
    assert np.array_equal(o, offsets) and np.array_equal(d, neighbours) and np.array_equal(w, weights)
    with pytest.raises(ValueError):
        graph_files.write_bel(prefix, offsets[:-1], neighbours)


def test_graph_files_tool_writes_a_graph(tmp_path):
    prefix = str(tmp_path / "t.bel")
    res = subprocess.run([sys.executable, "-m", "gpreempt_b200.graph_files", "--out", prefix, "--vertices", "300",
                          "--degree", "10", "--band", "20"], capture_output=True, text=True, cwd=ROOT)
    assert res.returncode == 0, res.stderr
    o, d, w = graph_files.read_bel(prefix)
    assert len(o) == 301 and len(d) == len(w) > 1000


def _golden():
    import json

    with open(os.path.join(ROOT, "tests", "golden", "graph_reference.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("which", ["small", "crank"])
def test_oracle_matches_results_of_the_reference_kernels(which):
    """tests/golden/graph_reference.json holds what GraphComputeRaw::{BFS,SSSP,CC,PageRank} of the
    reference computed on a GPU for two seeded graphs (tests/golden/make_graph_golden.py): labels,
    distances and components must be identical, ranks within the tolerance of the float sums."""
    import hashlib

    entry = _golden()["graphs"][which]
    offsets, neighbours = graph_files.synthetic_banded(**entry["spec"])
    weights = graph_files.synthetic_weights(len(neighbours), entry["spec"]["seed"])
    assert len(neighbours) == entry["edges"]
    got = {"bfs": graphs.bfs(offsets, neighbours)[0], "sssp": graphs.sssp(offsets, neighbours, weights)[0],
           "cc": graphs.cc(offsets, neighbours)[0], "pagerank": graphs.pagerank(offsets, neighbours)[0]}
    for algo, want in entry["results"].items():
        arr = got[algo]
        picks = np.array(want["picks"])
        if algo == "pagerank":
            assert np.max(np.abs(arr[picks] - np.array(want["at_picks"]))) <= 1.1e-3
            assert abs(float(arr.astype(np.float64).sum()) - want["sum"]) <= 2e-4 * len(arr)
            if "values" in want:
                err = np.abs(arr - np.array(want["values"], np.float32))
                assert err.max() <= 1.1e-3 and err.mean() <= 1e-5
        else:
            assert arr[picks].astype(np.uint64).tolist() == want["at_picks"], algo
            assert hashlib.sha256(arr.astype(np.uint64).tobytes()).hexdigest() == want["sha256"], algo
            if "values" in want:
                assert arr.astype(np.uint64).tolist() == want["values"], algo


def test_graph_files_from_a_matrix_market_file(tmp_path):
    """--from-mtx: the route for a user who has the reference's dataset as SuiteSparse ships it."""
    from scipy.io import mmwrite
    from scipy.sparse import random as sparse_random

    m = sparse_random(60, 60, density=0.08, random_state=3, format="coo")
    m = ((m + m.T) > 0).astype(np.float64).tocoo()
    mmwrite(str(tmp_path / "m.mtx"), m)
    info = graph_files.write_from_mtx(str(tmp_path / "m.bel"), str(tmp_path / "m.mtx"))
    offsets, neighbours, weights = graph_files.read_bel(str(tmp_path / "m.bel"))
    csr = m.tocsr()
    csr.sort_indices()
    assert info == {"prefix": str(tmp_path / "m.bel"), "vertices": 60, "edges": int(csr.nnz)}
    assert np.array_equal(offsets, csr.indptr.astype(np.uint64))
    assert np.array_equal(neighbours, csr.indices.astype(np.uint64))
    assert len(weights) == csr.nnz and weights.min() >= 1
    comp, _ = graphs.cc(offsets, neighbours)
    from scipy.sparse.csgraph import connected_components

    assert len(np.unique(comp)) == connected_components(csr, directed=False)[0]


def test_library_refuses_broken_graph_files_before_it_needs_a_gpu(tmp_path):
    """gpx_model_open("bfs:<prefix>") reads the files first, so their errors are reported where no GPU
    is: a missing file is NotFound (3), a malformed one Fail (1), too many vertices OutOfRange (4);
    a good one gets as far as asking for the device."""
    from gpreempt_b200 import api

    def status_of(name):
        with pytest.raises(api.GpxError) as e:
            api.Model(name)
        return e.value.status, str(e.value)

    assert status_of("bfs")[0] == 3 and "needs a graph" in status_of("bfs")[1]
    assert status_of("bfs:" + str(tmp_path / "nothing.bel"))[0] == 3
    offsets, neighbours = graph_files.synthetic_banded(200, 8, 12, 1)
    weights = graph_files.synthetic_weights(len(neighbours), 1)
    good = str(tmp_path / "good.bel")
    graph_files.write_bel(good, offsets, neighbours, weights)
    st, text = status_of("sssp:" + good)
    assert st == 1 and "gpx_init" in text  # the files were accepted

    def variant(name, offs=offsets, nbs=neighbours, wts=weights, cut=None):
        prefix = str(tmp_path / name)
        # written by hand: write_bel refuses these itself
        for ext, head, arr in ((".col", len(offs), np.asarray(offs, np.uint64)), (".dst", len(nbs), np.asarray(nbs, np.uint64)),
                               (".val", len(wts), np.asarray(wts, np.uint32))):
            with open(prefix + ext, "wb") as f:
                np.array([head, 8], np.uint64).tofile(f)
                arr.tofile(f)
        if cut:
            with open(prefix + cut, "r+b") as f:
                f.truncate(16 + 8)
        return prefix

    bad_id = neighbours.copy()
    bad_id[5] = 200
    assert "points at vertex" in status_of("cc:" + variant("bad_id.bel", nbs=bad_id))[1]
    down = offsets.copy()
    down[10], down[11] = down[11], down[10]
    assert "offsets decrease" in status_of("cc:" + variant("down.bel", offs=down))[1]
    assert "offsets run from" in status_of("cc:" + variant("short.bel", nbs=neighbours[:-3], wts=weights[:-3]))[1]
    assert "shorter than its header" in status_of("cc:" + variant("cut.bel", cut=".dst"))[1]
    assert "weights for" in status_of("sssp:" + variant("few_w.bel", wts=weights[:10]))[1]
    os.remove(variant("no_w.bel") + ".val")
    assert status_of("sssp:" + str(tmp_path / "no_w.bel"))[0] == 3
    assert status_of("bfs:" + str(tmp_path / "no_w.bel"))[1].count("gpx_init") == 1  # bfs needs no weights
