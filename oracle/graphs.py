"""ctypes wrapper of the graph-analytics CPU oracle (graph_oracle.c) - TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and bench.py's CPU baseline may import this module.  `Reference`
wraps oracle/_ref/libgraphcompute_ref.so, the reference's own CUDA source compiled unmodified
(oracle/Makefile, target `ref`); it needs a GPU and exists only where that library was built.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libgraph_oracle.so")
REF_LIB_PATH = os.path.join(_HERE, "_ref", "libgraphcompute_ref.so")
_lib = None
_u64p = ctypes.POINTER(ctypes.c_uint64)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_f32p = ctypes.POINTER(ctypes.c_float)

INFINITY = 0xFFFFFFFF
ALPHA, TOLERANCE, MAX_ITER = 0.85, 0.001, 100  # include/workloads/graphcompute.h:84-86


def build() -> str:
    src = os.path.join(_HERE, "graph_oracle.c")
    if not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libgraph_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.gro_bfs.argtypes = [ctypes.c_uint64, _u64p, _u64p, ctypes.c_uint32, _u32p]
        _lib.gro_cc.argtypes = [ctypes.c_uint64, _u64p, _u64p, _u64p]
        _lib.gro_sssp.argtypes = [ctypes.c_uint64, _u64p, _u64p, _u32p, ctypes.c_uint32, _u32p]
        _lib.gro_pagerank.argtypes = [ctypes.c_uint64, _u64p, _u64p, ctypes.c_float, ctypes.c_float, ctypes.c_int, _f32p]
    return _lib


def _graph(offsets, neighbours):
    offsets = np.ascontiguousarray(offsets, np.uint64)
    neighbours = np.ascontiguousarray(neighbours, np.uint64)
    return offsets, neighbours, len(offsets) - 1


def bfs(offsets, neighbours, src: int = 0):
    """(levels, kernel launches) of BFS::compute."""
    o, d, n = _graph(offsets, neighbours)
    label = np.empty(n, np.uint32)
    it = lib().gro_bfs(n, o.ctypes.data_as(_u64p), d.ctypes.data_as(_u64p), src, label.ctypes.data_as(_u32p))
    return label, it


def cc(offsets, neighbours):
    o, d, n = _graph(offsets, neighbours)
    comp = np.empty(n, np.uint64)
    it = lib().gro_cc(n, o.ctypes.data_as(_u64p), d.ctypes.data_as(_u64p), comp.ctypes.data_as(_u64p))
    return comp, it


def sssp(offsets, neighbours, weights, src: int = 0):
    o, d, n = _graph(offsets, neighbours)
    w = np.ascontiguousarray(weights, np.uint32)
    cost = np.empty(n, np.uint32)
    it = lib().gro_sssp(n, o.ctypes.data_as(_u64p), d.ctypes.data_as(_u64p), w.ctypes.data_as(_u32p), src,
                        cost.ctypes.data_as(_u32p))
    return cost, it


def pagerank(offsets, neighbours, alpha: float = ALPHA, tolerance: float = TOLERANCE, max_iter: int = MAX_ITER):
    o, d, n = _graph(offsets, neighbours)
    value = np.empty(n, np.float32)
    it = lib().gro_pagerank(n, o.ctypes.data_as(_u64p), d.ctypes.data_as(_u64p), alpha, tolerance, max_iter,
                            value.ctypes.data_as(_f32p))
    return value, it


def reference_available() -> bool:
    return os.path.exists(REF_LIB_PATH)


class Reference:
    """One graph workload of the reference itself on the GPU (GraphComputeRaw::*, src/workloads/graphcompute.cu)."""

    DTYPES = {"bfs": np.uint32, "sssp": np.uint32, "cc": np.uint64, "pagerank": np.float32}

    def __init__(self, algo: str, prefix: str, device: int = 0):
        self.lib = ctypes.CDLL(REF_LIB_PATH)
        self.lib.gcref_open.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_char_p]
        self.lib.gcref_vertices.restype = ctypes.c_ulonglong
        self.lib.gcref_compute.restype = ctypes.c_double
        self.lib.gcref_compute.argtypes = [ctypes.c_int]
        self.lib.gcref_result.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
        self.algo = algo
        rc = self.lib.gcref_open(device, algo.encode(), prefix.encode())
        if rc != 0:
            raise RuntimeError(f"gcref_open({algo}, {prefix}) failed with {rc}")
        self.vertices = int(self.lib.gcref_vertices())

    def compute(self, runs: int = 1) -> float:
        """Runs GraphCompute::compute `runs` times; host milliseconds of all of them."""
        ms = self.lib.gcref_compute(runs)
        if ms < 0:
            raise RuntimeError(f"gcref_compute failed with {ms}")
        return ms

    def result(self) -> np.ndarray:
        out = np.empty(self.vertices, self.DTYPES[self.algo])
        rc = self.lib.gcref_result(out.ctypes.data_as(ctypes.c_void_p), out.nbytes)
        if rc != 0:
            raise RuntimeError(f"gcref_result failed with {rc}")
        return out

    def close(self) -> None:
        self.lib.gcref_close()
