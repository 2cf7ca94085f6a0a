"""The C++ classes with the reference's names (include/gpx/*.h) and the C header itself are
compiled by a real compiler: a C99 client of gpx.h, and a port of the reference's manual
preempt-and-resume test (src/tests/test-dnn-blp.cpp) written against foo::BLPExecutor.  The CPU
tests compile, link and (for the C client) run; the GPU test runs the port and compares its
output with the ctypes path bit for bit."""
import os
import subprocess

import numpy as np
import pytest

from gpreempt_b200 import build as gpx_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "gpreempt_b200", "lib")


def _compile(tmp_path, compiler, std, src, out):
    gpx_build.build()
    exe = str(tmp_path / out)
    # include/ for the C header, include/gpx for the classes with the reference's header names
    cmd = [compiler, f"-std={std}", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(ROOT, "include", "gpx"),
           os.path.join(ROOT, "tests", "cpp", src), "-o", exe, "-L", LIBDIR, "-lgpx",
           f"-Wl,-rpath,{LIBDIR}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_c99_client_compiles_links_and_runs(tmp_path):
    exe = _compile(tmp_path, "gcc", "c99", "abi_c99.c", "abi_c99")
    res = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, (res.returncode, res.stdout, res.stderr)
    assert "PASS" in res.stdout


def test_reference_named_classes_compile_and_link(tmp_path):
    _compile(tmp_path, "g++", "c++17", "test_dnn_blp.cpp", "test_dnn_blp")
    _compile(tmp_path, "g++", "c++17", "test_sci.cpp", "test_sci")
    _compile(tmp_path, "g++", "c++17", "test_graph.cpp", "test_graph")


@pytest.mark.gpu
def test_port_of_the_reference_sci_test(gpx, tmp_path):
    """src/tests/test-sci.cpp through foo::BaseExecutor / foo::BLPExecutor: drift of mass and
    energy after one miniWeather time step, and a preempted time step that ends in the same state."""
    exe = _compile(tmp_path, "g++", "c++17", "test_sci.cpp", "test_sci")
    res = subprocess.run([exe, "miniweather"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, (res.stdout, res.stderr)
    assert "d_mass:" in res.stdout and "d_te:" in res.stdout and "PASS" in res.stdout


@pytest.mark.gpu
def test_port_of_the_reference_graph_tests(gpx, tmp_path):
    """src/tests/test-graph.cpp and test-graph-blp.cpp through foo::BaseExecutor / foo::BLPExecutor
    (set_graph_path, init, execute): the result equals the CPU oracle's, and a preempted and resumed
    run ends with the same bytes."""
    from gpreempt_b200 import graph_files
    from oracle import graphs

    exe = _compile(tmp_path, "g++", "c++17", "test_graph.cpp", "test_graph")
    prefix = str(tmp_path / "g" / "g.bel")
    graph_files.write_synthetic(prefix, 20000, 64, 400, 2)
    offsets, neighbours, weights = graph_files.read_bel(prefix)
    want = {"bfs": graphs.bfs(offsets, neighbours)[0], "sssp": graphs.sssp(offsets, neighbours, weights)[0],
            "cc": graphs.cc(offsets, neighbours)[0].astype(np.uint32)}
    for algo in ("bfs", "sssp", "cc", "pagerank"):
        out = str(tmp_path / (algo + ".bin"))
        res = subprocess.run([exe, algo, prefix, out], capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, (algo, res.stdout, res.stderr)
        assert f"{algo} Compute:" in res.stdout and "PASS" in res.stdout
        if algo in want:
            assert np.array_equal(np.fromfile(out, np.uint32), want[algo]), algo
        else:
            rank = np.fromfile(out, np.float32)
            assert np.max(np.abs(rank - graphs.pagerank(offsets, neighbours)[0])) <= 1.1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("model,batch,delay_us", [("resnet_tiny", 2, 0), ("resnet50", 8, 300)])
def test_port_of_the_reference_blp_test_matches_the_ctypes_path(gpx, tmp_path, model, batch, delay_us):
    exe = _compile(tmp_path, "g++", "c++17", "test_dnn_blp.cpp", "test_dnn_blp")
    out = str(tmp_path / "heads.bin")
    res = subprocess.run([exe, model, str(batch), str(delay_us), out], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, (res.stdout, res.stderr)
    assert "PASS resumed output is bit-identical" in res.stdout
    got = np.fromfile(out, np.float32).reshape(batch, 1000)
    ex = gpx.BaseExecutor()
    ex.init(model, batch=batch, seed=1)
    ex.set_input("data", np.full((batch, 3, 224, 224), 10.0, np.float32))
    ex.execute()
    assert np.array_equal(ex.get_output("heads"), got)
    ex.clear()
