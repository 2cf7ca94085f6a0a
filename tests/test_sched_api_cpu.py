"""Host-only behaviour of the scheduler API: deadlines and failure propagation without a GPU.

The failures are made on the host: a dispatcher that was never started (stalled), a ticket nobody
issued, a dispatcher thread that cannot bind a device.  No GPU is faulted, trapped or hung.
"""
import ctypes
import time

import pytest

from gpreempt_b200 import binding as B
from gpreempt_b200 import build as gpx_build


@pytest.fixture(scope="module")
def lib():
    gpx_build.build()
    return B.load()


def _sched(lib, policy=b"gpreemptclient"):
    s = ctypes.c_void_p()
    assert lib.gpx_sched_create(0, policy, ctypes.byref(s)) == B.SUCC
    return s


def test_wait_on_a_stalled_dispatcher_times_out_and_the_request_stays_queued(lib):
    s = _sched(lib)
    c = ctypes.c_int(-1)
    assert lib.gpx_sched_attach(s, None, 0, ctypes.byref(c)) == B.SUCC  # a client without GPU work
    assert c.value == 0
    t = ctypes.c_uint64()
    assert lib.gpx_sched_enqueue(s, 0, ctypes.byref(t)) == B.SUCC and t.value == 1
    assert lib.gpx_sched_enqueue(s, 0, ctypes.byref(t)) == B.SUCC and t.value == 2
    t0 = time.perf_counter()
    assert lib.gpx_wait(s, 0, 1, 30_000_000) == B.TIMEOUT  # nobody runs the dispatcher: 30 ms deadline
    dt = time.perf_counter() - t0
    assert 0.02 < dt < 2.0
    assert b"not completed within" in lib.gpx_last_error() and b"not running" in lib.gpx_last_error()
    need = ctypes.c_size_t()
    assert lib.gpx_sched_stats(s, None, 0, ctypes.byref(need)) == B.SUCC
    buf = ctypes.create_string_buffer(need.value)
    assert lib.gpx_sched_stats(s, buf, need.value, ctypes.byref(need)) == B.SUCC
    import json

    st = json.loads(buf.value.decode())
    assert st["running"] is False and st["clients"][0]["submitted"] == 2 and st["clients"][0]["completed"] == 0
    assert lib.gpx_sched_destroy(s) == B.SUCC


def test_argument_errors(lib):
    s = _sched(lib)
    c = ctypes.c_int()
    t = ctypes.c_uint64()
    assert lib.gpx_sched_attach(s, None, 7, ctypes.byref(c)) == B.OUT_OF_RANGE
    assert lib.gpx_sched_enqueue(s, 0, ctypes.byref(t)) == B.OUT_OF_RANGE  # no such client
    assert lib.gpx_sched_attach(s, None, 1, ctypes.byref(c)) == B.SUCC
    assert lib.gpx_wait(s, 0, 5, 1000) == B.NOT_FOUND  # ticket 5 was never issued
    assert lib.gpx_sched_hint(s, 3, 1) == B.OUT_OF_RANGE
    assert lib.gpx_sched_destroy(s) == B.SUCC
    s2 = ctypes.c_void_p()
    assert lib.gpx_sched_create(0, b"nosuchclient", ctypes.byref(s2)) == B.NOT_FOUND


def test_queue_capacity_is_the_reference_queue_capacity(lib):
    s = _sched(lib, b"baseclient")
    c = ctypes.c_int()
    assert lib.gpx_sched_attach(s, None, 1, ctypes.byref(c)) == B.SUCC
    t = ctypes.c_uint64()
    for _ in range(10000):
        assert lib.gpx_sched_enqueue(s, 0, ctypes.byref(t)) == B.SUCC
    assert lib.gpx_sched_enqueue(s, 0, ctypes.byref(t)) == B.FULL  # include/threadsafe_queue.h:14
    assert lib.gpx_sched_destroy(s) == B.SUCC


def test_a_dispatcher_that_cannot_start_fails_the_waiters(lib):
    """Without a usable device the dispatcher thread stops with an error; a waiting client gets
    GPX_FAIL with the reason instead of waiting out its deadline, and shutdown reports it too."""
    count = ctypes.c_int()
    if lib.gpx_device_count(ctypes.byref(count)) == B.SUCC and count.value > 0:
        pytest.skip("a device is present: the dispatcher starts normally here")
    s = _sched(lib)
    c = ctypes.c_int()
    assert lib.gpx_sched_attach(s, None, 0, ctypes.byref(c)) == B.SUCC
    t = ctypes.c_uint64()
    assert lib.gpx_sched_enqueue(s, 0, ctypes.byref(t)) == B.SUCC
    assert lib.gpx_sched_run(s) == B.SUCC
    assert lib.gpx_wait(s, 0, t.value, 5_000_000_000) == B.FAIL
    assert b"dispatcher failed" in lib.gpx_last_error()
    assert lib.gpx_sched_shutdown(s) == B.FAIL
    assert lib.gpx_sched_destroy(s) == B.SUCC
