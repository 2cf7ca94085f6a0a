"""Parity and preemption tests of the fp32 axpy kernel, through the C ABI on the GPU."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

A = 1.0009765625


def _inputs(gpx, n, seed=4):
    x = gpx.synth_uniform(n, seed, 0)
    y = gpx.synth_uniform(n, seed, 1)
    return x, y


@pytest.mark.parametrize("n", [1, 3, 4, 1000, 4096, 4097, 12345, 1 << 20, (1 << 22) + 5])
def test_axpy_bit_exact_vs_oracle(gpx, oracle, n):
    x, y = _inputs(gpx, n)
    dx, dy = gpx.DeviceBuffer.from_numpy(x), gpx.DeviceBuffer.from_numpy(y)
    gpx.axpy(A, dx, dy, n)  # static schedule (latency-critical form)
    got = dy.download(np.float32, n)
    want = oracle.axpy(A, x, y)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    dx.free(), dy.free()


def test_axpy_empty_and_bad_arguments(gpx):
    import ctypes

    from gpreempt_b200 import binding as B

    lib = B.load()
    assert lib.gpx_axpy_f32(ctypes.c_float(1.0), None, None, 0, 0, None, None) == B.SUCC
    buf = gpx.DeviceBuffer(1024)
    st = lib.gpx_axpy_f32(ctypes.c_float(1.0), ctypes.c_void_p(buf.ptr.value + 4), buf.ptr, 16, 0,
                          None, None)
    assert st == B.FAIL and b"aligned" in lib.gpx_last_error()
    buf.free()


@pytest.mark.parametrize("transport", [0, 1])
def test_axpy_preemptible_uninterrupted_matches(gpx, oracle, transport):
    n = (1 << 22) + 77
    x, y = _inputs(gpx, n, 14)
    dx, dy = gpx.DeviceBuffer.from_numpy(x), gpx.DeviceBuffer.from_numpy(y)
    word = gpx.PreemptWord(transport)
    ctx = gpx.BlpContext(word)
    s = gpx.Stream(1)
    gpx.axpy(A, dx, dy, n, ctx, s)
    s.sync()
    st = ctx.read()
    tiles = gpx.axpy_tiles(n)
    assert st["stop_index"] == -1
    assert st["tiles_run"] == tiles
    assert st["cursor"] >= tiles
    assert st["t_end"] > st["t_start"]
    assert np.array_equal(dy.download(np.float32, n), oracle.axpy(A, x, y))
    for o in (dx, dy, ctx, word, s):
        (o.free if hasattr(o, "free") else o.destroy)()


@pytest.mark.parametrize("transport", [0, 1])
def test_axpy_preempt_resume_is_bit_identical(gpx, oracle, transport):
    """Raise the word at random times, drain, clear, resume; every tile runs exactly once."""
    n = 1 << 27  # 512 MiB per vector: ~0.25 ms of kernel at full HBM bandwidth
    x, y = _inputs(gpx, n, 24)
    want = oracle.axpy(A, x, y)
    dx = gpx.DeviceBuffer.from_numpy(x)
    dy = gpx.DeviceBuffer(n * 4)
    word = gpx.PreemptWord(transport)
    ctx = gpx.BlpContext(word, kernel_id=7)
    s = gpx.Stream(1)
    tiles = gpx.axpy_tiles(n)
    rng = np.random.default_rng(99 + transport)
    preempted_runs = 0
    for trial in range(12):
        dy.upload(y)
        ctx.reset()
        word.clear()
        gpx.device_sync() if hasattr(gpx, "device_sync") else None
        launches = 0
        total_run = 0
        delay_us = float(rng.uniform(0, 300))
        while True:
            gpx.axpy(A, dx, dy, n, ctx, s)
            launches += 1
            if launches <= 3:
                t0 = time.perf_counter()
                while (time.perf_counter() - t0) * 1e6 < delay_us:
                    pass
                word.raise_()
            s.sync()
            st = ctx.read()
            word.clear()
            if transport == 1:
                time.sleep(0.001)  # the clear travels on its own stream; let it land
            if st["stop_index"] == -1:
                break
            assert st["stop_index"] == 7
            ctx.rearm()
            preempted_runs += 1
            assert launches < 50
        st = ctx.read()
        assert st["tiles_run"] == tiles, "every tile must run exactly once across resumes"
        got = dy.download(np.float32, n)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert preempted_runs > 0, "no launch was ever preempted; the test did not exercise resume"
    for o in (dx, dy, ctx, word, s):
        (o.free if hasattr(o, "free") else o.destroy)()


def test_axpy_launched_with_word_raised_does_nothing(gpx):
    n = 1 << 20
    x, y = _inputs(gpx, n, 34)
    dx, dy = gpx.DeviceBuffer.from_numpy(x), gpx.DeviceBuffer.from_numpy(y)
    word = gpx.PreemptWord(0)
    ctx = gpx.BlpContext(word, kernel_id=3)
    word.raise_()
    gpx.axpy(A, dx, dy, n, ctx)
    st = ctx.read()
    assert st["stop_index"] == 3 and st["cursor"] == 0 and st["tiles_run"] == 0
    assert np.array_equal(dy.download(np.float32, n), y)
    for o in (dx, dy, ctx, word):
        (o.free if hasattr(o, "free") else o.destroy)()


def test_block_kernel_is_bounded_and_releasable(gpx):
    """The wait kernel reports Timeout when nothing releases it and Succ when the host does."""
    import ctypes

    from gpreempt_b200 import binding as B

    lib = B.load()
    word = gpx.PreemptWord(0)
    status = gpx.DeviceBuffer(64)
    s = gpx.Stream(0)
    t0 = time.perf_counter()
    gpx.check(lib.gpx_block_launch(word.dptr, status.ptr, 20_000_000, s.handle))  # 20 ms
    s.sync()
    dt = time.perf_counter() - t0
    assert status.download(np.int32, 1)[0] == B.TIMEOUT
    assert 0.015 < dt < 1.0
    gpx.check(lib.gpx_block_launch(word.dptr, status.ptr, 1_000_000_000, s.handle))
    time.sleep(0.002)
    word.raise_()
    s.sync()
    assert status.download(np.int32, 1)[0] == B.SUCC
    assert lib.gpx_block_launch(word.dptr, status.ptr, 5_000_000_000, s.handle) == B.OUT_OF_RANGE
    gpx.check(lib.gpx_noop_launch(s.handle))
    s.sync()
    off, unc = gpx.clock_offset_ns()
    assert unc >= 0
    for o in (status, word, s):
        (o.free if hasattr(o, "free") else o.destroy)()
