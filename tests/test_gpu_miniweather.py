"""miniWeather (the reference's scientific best-effort workload) on the GPU: parity with the CPU
oracle and with the reference's own kernels, conservation, and preempt/resume bit-exactness."""
import json
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

# Float arithmetic, so a tolerance.  The horizontal momentum flux carries the full pressure
# (~1e5 Pa, one float ulp = 0.0078) and its difference is scaled by dt/dx = 1/300 at the
# reference's grid spacing, so two correct evaluations that round differently (fused multiply-adds
# on the GPU, none in the oracle) differ by ~3e-5 per semi-discrete step in rho*u; the other
# variables have fluxes of order 1-100 and agree far closer.  Bounds per time step, absolute:
ATOL_PER_STEP = {0: 2e-6, 1: 6e-4, 2: 6e-4, 3: 2e-4}


def _mw():
    from oracle import miniweather as mw

    mw.build()
    return mw


def _check_close(got, want, steps, what):
    from oracle.miniweather import interior

    for v in range(4):
        err = float(np.max(np.abs(interior(got)[v].astype(np.float64) - interior(want)[v])))
        assert err <= ATOL_PER_STEP[v] * steps, f"{what}: variable {v} differs by {err:.3e} after {steps} step(s)"


@pytest.mark.parametrize("name,nx,nz", [("miniweather_tiny", 320, 160), ("miniweather_200x104", 200, 104),
                                        ("miniweather", 3200, 1600)])
def test_initial_state_and_time_steps_match_oracle(gpx, name, nx, nz):
    mw = _mw()
    ex = gpx.BaseExecutor()
    ex.init(name)
    orc = mw.Oracle(nx, nz)
    assert ex.get_kernel_num() == 12
    # sci_init: same libm on both sides, so the initial fields agree bit for bit
    assert np.array_equal(ex.model.get("state"), orc.state)
    assert np.array_equal(ex.model.get("state_tmp"), orc.state)
    for f in ("hy_dens_cell", "hy_dens_theta_cell", "hy_dens_int", "hy_dens_theta_int", "hy_pressure_int"):
        assert np.array_equal(ex.model.get(f).ravel(), orc.field(f)), f
    m0, e0 = ex.model.reductions()
    assert (m0, e0) == orc.reductions()
    for step in (1, 2):
        ex.execute()
        orc.timestep()
        _check_close(ex.model.get("state"), orc.state, step, f"{name} state")
    # Halo cells of `state` (the forcing array of the first stage only, as in the reference): the
    # wrapped columns, the density rows the reference's vertical halo launch covers, and rows it
    # never writes, which still hold the initial values.  `state_tmp` is scratch and not compared:
    # the library's second stage writes a third buffer.
    got, want = ex.model.get("state"), orc.state
    assert np.allclose(got[:, 2:-2, :2], want[:, 2:-2, :2], atol=2e-3)
    assert np.allclose(got[:, 2:-2, -2:], want[:, 2:-2, -2:], atol=2e-3)
    assert np.allclose(got[0, :2, 2:-2], want[0, :2, 2:-2], atol=1e-5)
    assert np.allclose(got[0, -2:, 2:-2], want[0, -2:, 2:-2], atol=1e-5)
    assert np.array_equal(got[3, :2, 2:-2], want[3, :2, 2:-2])
    assert np.array_equal(got[2, -2:, 2:-2], want[2, -2:, 2:-2])
    m1, e1 = ex.model.reductions()
    assert abs(m1 - m0) / m0 < 1e-8 and abs(e1 - e0) / e0 < 1e-4   # float rounding; energy is not conserved exactly
    # starting over
    ex.model.init_random(0)
    assert np.array_equal(ex.model.get("state"), orc.__class__(nx, nz).state)
    ex.clear()


def test_matches_the_reference_kernels(gpx):
    """Against the reference's own CUDA source (compiled unmodified into oracle/_ref): the
    library's kernels and the CPU oracle after 1 and 3 time steps on the 3200 x 1600 grid."""
    mw = _mw()
    if not mw.reference_available():
        pytest.skip("oracle/_ref/libminiweather_ref.so was not built (make -C oracle ref)")
    ref = mw.Reference(0)
    ex = gpx.BaseExecutor()
    ex.init("miniweather")
    orc = mw.Oracle(ref.nx, ref.nz)
    assert ref.dt == orc.dt
    assert np.array_equal(ref.state(0), orc.state), "initial state of the oracle differs from the reference's"
    assert np.array_equal(ref.state(0), ex.model.get("state"))
    assert ref.reductions() == orc.reductions() == ex.model.reductions()
    done = 0
    for steps in (1, 3):
        n = steps - done
        ref.timestep(n)
        orc.timestep(n)
        for _ in range(n):
            ex.execute()
        done = steps
        want = ref.state(0)
        _check_close(orc.state, want, steps, "oracle vs reference")
        got = ex.model.get("state")
        _check_close(got, want, steps, "library vs reference")
        # The library's kernels execute the reference's operations with the same roundings: every
        # cell of every variable is identical, not merely close.
        assert np.array_equal(mw.interior(got), mw.interior(want)), f"not bit-identical after {steps} step(s)"
        assert np.array_equal(got[:, 2:-2, :], want[:, 2:-2, :])          # wrapped columns too
        assert np.array_equal(got[0, :, 2:-2], want[0, :, 2:-2])          # density halo rows
        rm, re_ = ref.reductions()
        gm, ge = ex.model.reductions()
        assert abs(gm - rm) / rm < 1e-10 and abs(ge - re_) / re_ < 1e-8
    ref.close()
    ex.clear()


def test_preempt_resume_bit_identical(gpx):
    """execute, raise the word mid-run, drain, clear, resume (src/tests/test-dnn-blp.cpp:36-43 for
    this workload): three time steps equal the uninterrupted run bit for bit, every tile ran once."""
    base = gpx.BaseExecutor()
    base.init("miniweather")
    for _ in range(3):
        base.execute()
    want = base.model.get("state")
    want_tmp = base.model.get("state_tmp")

    word = gpx.PreemptWord(0)
    ex = gpx.BLPExecutor()
    ex.init("miniweather")
    ex.set_word(word)
    ex.enable_trace(True)
    s = gpx.Stream(1)
    nk = ex.get_kernel_num()
    tiles = np.array([ex.model.get_kernel_info(i)["total_tiles"] for i in range(nk)])
    t0 = time.perf_counter()
    ex.execute(s)
    s.sync()
    run_us = (time.perf_counter() - t0) * 1e6
    trace = ex.read_trace()
    assert np.array_equal(trace[:, 3].astype(np.int64), tiles)
    rng = np.random.default_rng(5)
    stops_seen = 0
    for trial in range(4):
        ex.model.init_random(0)
        for step in range(3):
            word.clear()
            time.sleep(0.001)
            ex.execute(s)
            rounds = 0
            while True:
                if rounds < 5:
                    delay = float(rng.uniform(0, run_us / 3))
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
                assert 0 <= stop < nk and rounds < 80
            s.sync()
            assert np.all(ex.read_cursors() >= tiles)
        assert np.array_equal(ex.model.get("state"), want), f"trial {trial}"
        assert np.array_equal(ex.model.get("state_tmp"), want_tmp), f"trial {trial}"
    assert stops_seen > 0, "no run was ever preempted"
    base.clear(), ex.clear(), word.destroy(), s.destroy()


def test_graph_capture_and_data_calls(gpx):
    """Executor::capture_graph works for the workload, it has no request data
    (Executor::get_data_size returns 0 for it, src/executor.cpp:87-97) and cannot be exported."""
    a, b = gpx.BaseExecutor(), gpx.BaseExecutor()
    a.init("miniweather_tiny")
    b.init("miniweather_tiny")
    s = gpx.Stream(0)
    b.capture_graph(s)
    for _ in range(4):
        a.execute()
        b.execute(s)
    s.sync()
    assert np.array_equal(a.model.get("state"), b.model.get("state"))
    with pytest.raises(gpx.GpxError):
        a.model.find_storage_idx("data")
    with pytest.raises(gpx.GpxError):
        a.model.export_json()
    with pytest.raises(gpx.GpxError):
        gpx.Model("resnet_tiny").reductions()
    a.clear(), b.clear(), s.destroy()


def test_best_effort_tenant_under_a_latency_critical_model(gpx):
    """The shape of the reference's config/Y.json: a closed-loop miniweather tenant under a
    latency-critical DNN, preempted and resumed by the dispatcher."""
    cfg = {"time": 1.0, "seed": 3, "warmup": 2, "standalone": 2, "tasks": [
        {"id": "vgg_rt", "load": {"type": "periodic", "priority": 0, "frequency": 100},
         "client": {"name": "vgg_rt", "model_name": "vgg", "priority": 0, "batch_size": 1,
                    "use_cuda_graph": True, "preprocess_time": 200}},
        {"id": "miniweather_be", "load": {"type": "periodic", "priority": 0, "frequency": 150},
         "client": {"name": "miniweather_be", "model_name": "miniweather", "priority": 1, "batch_size": 1,
                    "use_cuda_graph": True, "preprocess_time": 0}}]}
    rep = json.loads(gpx.run_workload("gpreemptclient", json.dumps(cfg)))
    by_id = {t["id"]: t for t in rep["tasks"]}
    assert by_id["miniweather_be"]["requests"] > 50
    assert 90 <= by_id["vgg_rt"]["requests"] <= 101
    assert rep["gpus"][0]["wordRaises"] > 0 and by_id["miniweather_be"]["resumes"] > 0
    assert by_id["miniweather_be"]["in_bytes"] == 0


def test_mass_and_energy_drift_as_the_reference_prints_them(gpx):
    """src/tests/test-sci.cpp:10-21: initialise, take the reductions, run one time step, print the
    relative change of mass and total energy.  The figures of the reference's own kernels are in
    tests/golden/miniweather_reference.json."""
    import os

    with open(os.path.join(os.path.dirname(__file__), "golden", "miniweather_reference.json")) as fp:
        golden = json.load(fp)
    ex = gpx.BaseExecutor()
    ex.init("miniweather")
    mass0, te0 = ex.model.reductions()
    ex.execute()
    mass, te = ex.model.reductions()
    d_mass, d_te = (mass - mass0) / mass0, (te - te0) / te0
    g0, g1 = golden["steps"]["0"], golden["steps"]["1"]
    assert (mass0, te0) == (g0["mass"], g0["te"])
    assert (mass, te) == (g1["mass"], g1["te"])          # same cells, same sum order: same doubles
    assert d_mass == (g1["mass"] - g0["mass"]) / g0["mass"] and abs(d_mass) < 1e-9
    assert d_te == (g1["te"] - g0["te"]) / g0["te"] and abs(d_te) < 1e-7
    ex.clear()
