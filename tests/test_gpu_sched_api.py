"""The scheduler API driven by client threads of the caller: the counterpart of the reference's
REEF client loop (new_task / wait_task, src/reef-client/reefclient.cpp:105-110)."""
import threading
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _data(gpx, batch, seed=0):
    return gpx.synth_normal(batch * 3 * 224 * 224, seed, 0).reshape(batch, 3, 224, 224)


def test_two_client_threads_share_one_gpu_through_the_scheduler(gpx):
    """A latency-critical thread and a best-effort thread submit through one scheduler under the
    GP policy.  Every request completes with the result of a solo run (bit for bit, although
    the best-effort forwards are preempted and resumed), the word was raised, the best-effort
    executor was resumed, and the statistics count every request."""
    hp_ref = gpx.BaseExecutor()
    hp_ref.init("resnet_tiny", batch=1, seed=1)
    hp_data = _data(gpx, 1, seed=3)
    hp_ref.set_input("data", hp_data)
    hp_ref.execute()
    hp_want = hp_ref.get_output("heads")
    be_ref = gpx.BaseExecutor()
    be_ref.init("resnet50", batch=16, seed=1)
    be_data = _data(gpx, 16, seed=4)
    be_ref.set_input("data", be_data)
    be_ref.execute()
    be_want = be_ref.get_output("heads")

    hp = gpx.BaseExecutor()
    hp.init("resnet_tiny", batch=1, seed=1)
    be = gpx.BLPExecutor()
    be.init("resnet50", batch=16, seed=1)
    sched = gpx.Scheduler(0, "gpreemptclient")
    c_hp = sched.attach(hp, 0)
    c_be = sched.attach(be, 1)
    hp.capture_graph(sched.client_stream(c_hp))
    hp.set_input("data", hp_data)
    be.set_input("data", be_data)
    gpx.device_sync()
    sched.run()

    errors = []
    hp_done, be_done = [0], [0]
    stop = threading.Event()

    def hp_client():
        try:
            gpx.init_cuda(0)
            while not stop.is_set():
                t = sched.new_task(c_hp)
                sched.wait_task(c_hp, t, 10.0)
                if not np.array_equal(hp.get_output("heads"), hp_want):
                    errors.append("latency-critical result differs")
                hp_done[0] += 1
                time.sleep(0.002)
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))

    def be_client():
        try:
            gpx.init_cuda(0)
            for _ in range(40):
                t = sched.new_task(c_be)
                sched.wait_task(c_be, t, 20.0)
                if not np.array_equal(be.get_output("heads"), be_want):
                    errors.append("best-effort result differs after preemption")
                be_done[0] += 1
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))
        finally:
            stop.set()

    th = [threading.Thread(target=hp_client), threading.Thread(target=be_client)]
    for t in th:
        t.start()
    for t in th:
        t.join()
    st = sched.stats()
    sched.shutdown()
    assert not errors, errors[:3]
    assert be_done[0] == 40 and hp_done[0] > 5
    assert st["wordRaises"] > 0 and st["beResumes"] > 0
    assert st["clients"][c_hp]["completed"] == hp_done[0]
    assert st["clients"][c_be]["completed"] == 40
    assert st["kernelDrain(us)"]["count"] > 0 and st["kernelDrain(us)"]["p99"] < 100.0
    assert be.error() == (0, 0)
    sched.destroy()
    for e in (hp_ref, be_ref, hp, be):
        e.clear()


def test_queued_tickets_run_in_order_and_a_short_deadline_reports_timeout(gpx):
    from gpreempt_b200 import binding as B

    be = gpx.BaseExecutor()
    be.init("resnet50", batch=16, seed=1)
    be.set_input("data", _data(gpx, 16))
    sched = gpx.Scheduler(0, "baseclient")
    c = sched.attach(be, 1)
    probe = sched.attach(None, 0)  # a client without GPU work: measures the dispatch path only
    gpx.device_sync()
    sched.run()
    tickets = [sched.new_task(c) for _ in range(8)]
    assert tickets == list(range(1, 9))
    with pytest.raises(gpx.GpxError) as e:
        sched.wait_task(c, tickets[-1], 1e-5)  # 10 us: eight forwards cannot have finished
    assert e.value.status == B.TIMEOUT
    sched.wait_task(c, tickets[-1], 20.0)      # the request stayed queued and completes
    for t in tickets:
        sched.wait_task(c, t, 1.0)
    t = sched.new_task(probe)
    sched.wait_task(probe, t, 5.0)
    st = sched.stats()
    assert st["clients"][c]["completed"] == 8 and st["clients"][probe]["completed"] == 1
    assert st["wordRaises"] == 0
    sched.shutdown()
    sched.destroy()
    be.clear()


def test_hint_raises_the_word_before_the_request_arrives(gpx):
    hp = gpx.BaseExecutor()
    hp.init("resnet_tiny", batch=1, seed=1)
    be = gpx.BLPExecutor()
    be.init("resnet50", batch=16, seed=1)
    hp.set_input("data", _data(gpx, 1))
    be.set_input("data", _data(gpx, 16))
    sched = gpx.Scheduler(0, "gpreemptclient")
    c_hp, c_be = sched.attach(hp, 0), sched.attach(be, 1)
    gpx.device_sync()
    sched.run()
    tb = sched.new_task(c_be)
    time.sleep(0.0005)
    sched.hint(c_hp, True)        # DeamonHint: the request is about to come
    time.sleep(0.002)
    raises_after_hint = sched.stats()["wordRaises"]
    t = sched.new_task(c_hp)
    sched.wait_task(c_hp, t, 10.0)
    sched.wait_task(c_be, tb, 20.0)
    st = sched.stats()
    assert raises_after_hint >= 1, "the hint did not raise the word"
    assert st["clients"][c_hp]["completed"] == 1 and st["clients"][c_be]["completed"] == 1
    sched.shutdown()
    sched.destroy()
    hp.clear(), be.clear()
