"""Parity and K-granular preempt/resume of the tcgen05 bf16 GEMM, through the C ABI."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

# bf16 output of an fp32-accumulated product: the parity contract allows 2e-2 relative to the
# largest reference magnitude; the bound used here is much tighter (one bf16 rounding of the
# exact value plus fp32 accumulation noise).
REL_TOL_BF16 = 2e-2


def _operands(gpx, oracle, m, n, k, seed=3):
    a = oracle.f32_to_bf16(gpx.synth_uniform(m * k, seed, 0).reshape(m, k))
    b = oracle.f32_to_bf16(gpx.synth_uniform(n * k, seed, 1).reshape(n, k))
    return a, b


def _check(oracle, got_bits, exact):
    got = oracle.bf16_to_f32(got_bits).astype(np.float64)
    scale = float(np.max(np.abs(exact)))
    err = np.abs(got - exact)
    assert float(err.max()) <= REL_TOL_BF16 * scale
    # tight bound: half a bf16 ulp of the value plus accumulation noise
    tight = np.abs(exact) * 2.0 ** -8 + scale * 1e-5
    assert np.all(err <= tight), f"max excess {float((err - tight).max())}"


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 192),
                                   (1024, 1024, 1024), (2048, 768, 320)])
def test_gemm_matches_oracle(gpx, oracle, m, n, k):
    a, b = _operands(gpx, oracle, m, n, k)
    da, db = gpx.DeviceBuffer.from_numpy(a), gpx.DeviceBuffer.from_numpy(b)
    dc = gpx.DeviceBuffer(m * n * 2)
    dc.zero()
    ctx = gpx.GemmContext()
    s = gpx.Stream(1)
    gpx.gemm_bf16(da, db, dc, m, n, k, ctx, None, s)
    s.sync()
    assert ctx.status() == (0, 0)
    got = dc.download(np.uint16, m * n).reshape(m, n)
    _check(oracle, got, oracle.gemm_bf16_nt(a, b))
    for o in (da, db, dc, ctx, s):
        (o.free if hasattr(o, "free") else o.destroy)()


def test_gemm_rejects_bad_shapes(gpx):
    from gpreempt_b200 import binding as B

    buf = gpx.DeviceBuffer(1 << 20)
    ctx = gpx.GemmContext()
    with pytest.raises(gpx.GpxError) as e:
        gpx.gemm_bf16(buf, buf, buf, 100, 256, 64, ctx)
    assert e.value.status == B.OUT_OF_RANGE
    with pytest.raises(gpx.GpxError) as e:
        gpx.gemm_bf16(buf, buf, buf, 128, 256, 65, ctx)
    assert e.value.status == B.OUT_OF_RANGE
    buf.free(), ctx.free()


@pytest.mark.parametrize("size", [4096, 8192])
def test_gemm_preempt_resume_is_bit_identical(gpx, oracle, size):
    m = n = k = size
    a, b = _operands(gpx, oracle, m, n, k, seed=3)
    da, db = gpx.DeviceBuffer.from_numpy(a), gpx.DeviceBuffer.from_numpy(b)
    dc = gpx.DeviceBuffer(m * n * 2)
    ctx = gpx.GemmContext()
    s = gpx.Stream(1)
    word = gpx.PreemptWord(1)
    blp = gpx.BlpContext(word, kernel_id=11)
    tiles = gpx.gemm_tiles(m, n)

    # uninterrupted reference run (also timed, to place the triggers)
    dc.zero()
    gpx.gemm_bf16(da, db, dc, m, n, k, ctx, blp, s)
    s.sync()
    t0 = time.perf_counter()
    ctx.reset(), blp.reset()
    gpx.gemm_bf16(da, db, dc, m, n, k, ctx, blp, s)
    s.sync()
    run_us = (time.perf_counter() - t0) * 1e6
    assert ctx.status() == (0, 0)
    st = blp.read()
    assert st["stop_index"] == -1 and st["cursor"] == tiles and st["tiles_run"] == tiles
    want = dc.download(np.uint16, m * n)

    # sampled parity of the full-size product against the oracle
    rng = np.random.default_rng(5)
    rows = rng.integers(0, m, 2048).astype(np.int32)
    cols = rng.integers(0, n, 2048).astype(np.int32)
    exact = oracle.gemm_bf16_nt_samples(a, b, rows, cols)
    _check(oracle, want.reshape(m, n)[rows, cols], exact)

    stops = 0
    for trial in range(6):
        dc.zero()
        ctx.reset(), blp.reset()
        word.clear()
        time.sleep(0.001)
        rounds = 0
        while True:
            gpx.gemm_bf16(da, db, dc, m, n, k, ctx, blp, s)
            if rounds < 5:
                delay = float(rng.uniform(0, run_us * 0.6))
                t0 = time.perf_counter()
                while (time.perf_counter() - t0) * 1e6 < delay:
                    pass
                word.raise_()
            s.sync()
            word.clear()
            time.sleep(0.0005)
            st = blp.read()
            rounds += 1
            assert ctx.status() == (0, 0)
            if st["stop_index"] == -1:
                break
            assert st["stop_index"] == 11
            stops += 1
            blp.rearm()
            assert rounds < 40
        st = blp.read()
        assert st["cursor"] == tiles and st["tiles_run"] == tiles
        got = dc.download(np.uint16, m * n)
        assert np.array_equal(got, want), f"trial {trial}: resumed result differs"
    assert stops > 0, "never preempted"
    for o in (da, db, dc, ctx, s, word, blp):
        (o.free if hasattr(o, "free") else o.destroy)()
