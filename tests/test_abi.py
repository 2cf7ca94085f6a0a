"""The C-ABI library loads without a GPU and exports every symbol include/gpx.h declares."""
import ctypes

import pytest

from gpreempt_b200 import binding as B
from gpreempt_b200 import build as gpx_build


@pytest.fixture(scope="module")
def lib():
    gpx_build.build()
    return B.load()


def test_every_declared_symbol_is_exported(lib):
    names = B.declared_symbols()
    assert len(names) >= 60
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in gpx.h but not exported: {missing}"


def test_every_declared_symbol_has_a_ctypes_signature(lib):
    special = {"gpx_strerror", "gpx_last_error", "gpx_host_now_ns"}
    unbound = [n for n in B.declared_symbols() if n not in B._SIGS and n not in special]
    assert not unbound, f"no ctypes signature for: {unbound}"


def test_status_codes_match_the_reference_enum(lib):
    # include/util/common.h:16-23: Succ, Fail, Timeout, NotFound, OutOfRange, Full
    want = ["Succ", "Fail", "Timeout", "NotFound", "OutOfRange", "Full"]
    assert [lib.gpx_strerror(i).decode() for i in range(6)] == want
    assert (B.SUCC, B.FAIL, B.TIMEOUT, B.NOT_FOUND, B.OUT_OF_RANGE, B.FULL) == tuple(range(6))


def test_host_clock_is_monotonic(lib):
    a = lib.gpx_host_now_ns()
    b = lib.gpx_host_now_ns()
    assert b >= a > 0


def test_argument_checks_do_not_need_a_device(lib):
    tiles = ctypes.c_int()
    assert lib.gpx_axpy_tiles(10000, 4096, ctypes.byref(tiles)) == B.SUCC
    assert tiles.value == 3
    assert lib.gpx_axpy_tiles(10000, 6, ctypes.byref(tiles)) == B.OUT_OF_RANGE
    assert b"multiple of 4" in lib.gpx_last_error()
    assert lib.gpx_set_priority(7) == B.OUT_OF_RANGE
    assert lib.gpx_set_priority(0) == B.SUCC


def test_synthetic_generator_is_counter_based(lib):
    import numpy as np

    from gpreempt_b200 import api

    a = api.synth_normal(4096, seed=1, stream=3)
    b = api.synth_normal(4096, seed=1, stream=3)
    c = api.synth_normal(2048, seed=1, stream=3)
    d = api.synth_normal(4096, seed=2, stream=3)
    assert np.array_equal(a, b) and np.array_equal(a[:2048], c)
    assert not np.array_equal(a, d)
    big = api.synth_normal(1 << 18, seed=0, stream=0)
    assert abs(float(big.mean())) < 0.01 and abs(float(big.std()) - 1.0) < 0.01
    u = api.synth_uniform(1 << 18, seed=4, stream=0, lo=-1.0, hi=1.0)
    assert u.min() >= -1.0 and u.max() < 1.0 and abs(float(u.mean())) < 0.01
