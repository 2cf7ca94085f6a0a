"""The GEMM entry point that allocates nothing (gpx_gemm_bf16_static).

It exists for callers that cannot allocate device memory (memory handed out once by an
external pool, a thread that must stay out of the allocator, places where allocation is not
permitted): its progress slots and spill area sit in a static device array inside the library.
The test calls it through the C ABI twice in a row, with different operands, and requires each
result to equal the existing entry point's (gpx_gemm_bf16 with a caller-allocated context) bit
for bit — the same kernel runs, so the tolerance is zero.  Collected last, so a run that stops
at the first failure has already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _operands(gpx, oracle, m, n, k, seed):
    a = oracle.f32_to_bf16(gpx.synth_uniform(m * k, seed, 0).reshape(m, k))
    b = oracle.f32_to_bf16(gpx.synth_uniform(n * k, seed, 1).reshape(n, k))
    return a, b


def test_static_scratch_gemm_matches_allocating_entry_point_twice_in_a_row(gpx, oracle):
    s = gpx.Stream(1)
    ctx = gpx.GemmContext()
    # two different products back to back: the second must not see the first one's progress slots
    for call, (m, n, k, seed) in enumerate([(1024, 1024, 512, 21), (2048, 1024, 192, 22)]):
        a, b = _operands(gpx, oracle, m, n, k, seed)
        da, db = gpx.DeviceBuffer.from_numpy(a), gpx.DeviceBuffer.from_numpy(b)
        want_buf, got_buf = gpx.DeviceBuffer(m * n * 2), gpx.DeviceBuffer(m * n * 2)
        want_buf.zero(), got_buf.zero()
        ctx.reset()
        gpx.gemm_bf16(da, db, want_buf, m, n, k, ctx, None, s)
        s.sync()
        assert ctx.status() == (0, 0)
        gpx.gemm_bf16_static(da, db, got_buf, m, n, k, False, None, s)
        s.sync()
        assert gpx.gemm_static_status() == (0, 0)
        want = want_buf.download(np.uint16, m * n)
        got = got_buf.download(np.uint16, m * n)
        assert np.array_equal(got, want), f"call {call}: static-scratch result differs"
        # and the product is right, not merely equal: sampled check against the oracle
        rng = np.random.default_rng(call)
        rows = rng.integers(0, m, 256).astype(np.int32)
        cols = rng.integers(0, n, 256).astype(np.int32)
        exact = oracle.gemm_bf16_nt_samples(a, b, rows, cols)
        vals = oracle.bf16_to_f32(got.reshape(m, n)[rows, cols]).astype(np.float64)
        assert np.max(np.abs(vals - exact)) <= 2e-2 * np.max(np.abs(exact))
        for o in (da, db, want_buf, got_buf):
            o.free()
    ctx.free(), s.destroy()


def test_static_scratch_gemm_resumes_after_a_raised_word(gpx, oracle):
    m, n, k = 1024, 1024, 2048
    a, b = _operands(gpx, oracle, m, n, k, 23)
    da, db = gpx.DeviceBuffer.from_numpy(a), gpx.DeviceBuffer.from_numpy(b)
    want_buf, got_buf = gpx.DeviceBuffer(m * n * 2), gpx.DeviceBuffer(m * n * 2)
    s = gpx.Stream(1)
    ctx = gpx.GemmContext()
    gpx.gemm_bf16(da, db, want_buf, m, n, k, ctx, None, s)
    s.sync()
    word = gpx.PreemptWord(1)
    blp = gpx.BlpContext(word, kernel_id=4)
    got_buf.zero()
    word.raise_()
    gpx.device_sync()
    gpx.gemm_bf16_static(da, db, got_buf, m, n, k, False, blp, s)  # drains at once: word is up
    s.sync()
    assert blp.read()["stop_index"] == 4
    word.clear()
    gpx.device_sync()
    blp.rearm()
    gpx.gemm_bf16_static(da, db, got_buf, m, n, k, True, blp, s)   # resume from the saved slots
    s.sync()
    st = blp.read()
    assert st["stop_index"] == -1 and st["cursor"] == gpx.gemm_tiles(m, n)
    assert gpx.gemm_static_status() == (0, 0)
    assert np.array_equal(got_buf.download(np.uint16, m * n), want_buf.download(np.uint16, m * n))
    for o in (da, db, want_buf, got_buf, ctx, blp, word, s):
        (o.free if hasattr(o, "free") else o.destroy)()


def test_static_scratch_gemm_spills_and_reloads_accumulators_mid_tile(gpx, oracle):
    """The path that makes the static array matter: the word goes up while every CTA is in the
    middle of its only tile, so each one saves its fp32 accumulators and K position into the
    array and a `resume=1` call reloads them.  The product sits at the 64-tile limit with a long
    K, so a tile takes the whole kernel; afterwards a fresh product of another shape (resume=0)
    must not be disturbed by what the first one left in the array."""
    import time

    m, n, k = 2048, 1024, 16384
    a, b = _operands(gpx, oracle, m, n, k, 24)
    da, db = gpx.DeviceBuffer.from_numpy(a), gpx.DeviceBuffer.from_numpy(b)
    want_buf, got_buf = gpx.DeviceBuffer(m * n * 2), gpx.DeviceBuffer(m * n * 2)
    s = gpx.Stream(1)
    ctx = gpx.GemmContext()
    tiles = gpx.gemm_tiles(m, n)
    assert tiles == 64
    gpx.gemm_bf16(da, db, want_buf, m, n, k, ctx, None, s)
    s.sync()
    t0 = time.perf_counter()
    ctx.reset()
    gpx.gemm_bf16(da, db, want_buf, m, n, k, ctx, None, s)
    s.sync()
    run_us = (time.perf_counter() - t0) * 1e6
    assert ctx.status() == (0, 0)
    want = want_buf.download(np.uint16, m * n)

    word = gpx.PreemptWord(1)
    blp = gpx.BlpContext(word, kernel_id=6)
    mid_tile_stops = 0
    for trial, frac in enumerate((0.3, 0.5, 0.2, 0.6)):
        got_buf.zero()
        blp.reset()
        word.clear()
        gpx.device_sync()
        resume = False
        rounds = 0
        while True:
            gpx.gemm_bf16_static(da, db, got_buf, m, n, k, resume, blp, s)
            if rounds < 3:
                t0 = time.perf_counter()
                while (time.perf_counter() - t0) * 1e6 < run_us * frac:
                    pass
                word.raise_()
            s.sync()
            word.clear()
            gpx.device_sync()
            st = blp.read()
            assert gpx.gemm_static_status() == (0, 0)
            rounds += 1
            if st["stop_index"] == -1:
                break
            assert st["stop_index"] == 6
            # One tile per CTA: a launch that ran for a while and completed no tile can only have
            # left its progress in the accumulators it saved.
            if st["cursor"] < tiles and st["t_seen"] - st["t_start"] > 5_000:
                mid_tile_stops += 1
            blp.rearm()
            resume = True
            assert rounds < 20
        st = blp.read()
        assert st["cursor"] == tiles
        assert np.array_equal(got_buf.download(np.uint16, m * n), want), f"trial {trial}: resumed result differs"
    assert mid_tile_stops > 0, "no launch was ever stopped in the middle of its tiles"

    # a fresh product of another shape right after: the header-only clear of resume=0 must do
    m2, n2, k2 = 1024, 512, 320
    a2, b2 = _operands(gpx, oracle, m2, n2, k2, 25)
    da2, db2 = gpx.DeviceBuffer.from_numpy(a2), gpx.DeviceBuffer.from_numpy(b2)
    want2, got2 = gpx.DeviceBuffer(m2 * n2 * 2), gpx.DeviceBuffer(m2 * n2 * 2)
    ctx.reset()
    gpx.gemm_bf16(da2, db2, want2, m2, n2, k2, ctx, None, s)
    gpx.gemm_bf16_static(da2, db2, got2, m2, n2, k2, False, None, s)
    s.sync()
    assert gpx.gemm_static_status() == (0, 0)
    assert np.array_equal(got2.download(np.uint16, m2 * n2), want2.download(np.uint16, m2 * n2))
    for o in (da, db, want_buf, got_buf, da2, db2, want2, got2, ctx, blp, word, s):
        (o.free if hasattr(o, "free") else o.destroy)()


def test_static_scratch_gemm_rejects_products_beyond_its_limit(gpx):
    from gpreempt_b200 import binding as B

    buf = gpx.DeviceBuffer(1 << 20)
    with pytest.raises(gpx.GpxError) as e:
        gpx.gemm_bf16_static(buf, buf, buf, 8192, 8192, 64)  # 64 x 32 = 2048 tiles > 64
    assert e.value.status == B.OUT_OF_RANGE
    assert "at most 64 output tiles" in str(e.value)
    buf.free()
