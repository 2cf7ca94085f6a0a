#!/usr/bin/env python
"""Headline benchmark: two tenants on one GPU (per rank).

Workload (the reference's A-type contention config, config/A.json, at the sizes the baseline
names): a latency-critical ResNet-50 batch-1 fp32 client with Poisson arrivals at 100 req/s and
a best-effort ResNet-50 batch-32 fp32 client that resubmits continuously.  A "step" is 50
best-effort batches (1 600 inferences, about 0.1 s) executed while the latency-critical load keeps
arriving, so that any number of steps spans real contention (about ten latency-critical arrivals
and preemptions per step).

    python bench.py --gpus N --steps K --warmup W          # this library, one rank per GPU
    python bench.py --impl reference --steps K --warmup W  # CPU port of the same forward

Rank 0 prints ONE JSON line.  `value` is the whole-job best-effort throughput (inf/s) under
contention with inputs resident in HBM; `e2e` is the same with every request's input copied
from pinned host memory and its result copied back inside the timed region; `e2e` also carries
the rest of the metric: latency-critical p50/p99 under contention (the 10 s run the baseline
configuration names) and alone, best-effort throughput alone, and the preemption latencies.  No
number here is produced on the CPU oracle except the `cpu_baseline` object.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BE_BATCH = 32
BATCHES_PER_STEP = 50
LATENCY_RUN_S = 10.0
HP_RATE = 100.0
WORKLOAD = ("configs[1]: HP ResNet-50 b1 fp32 Poisson 100 req/s vs BE ResNet-50 b32 fp32 closed loop, "
            "one scheduler per GPU (replicas)")
REF_IMAGES_PER_STEP = 8      # bounded sample of a step for the CPU arm
MICROBENCH_TRIGGERS = 1000
MICROBENCH_AXPY_ELEMS = 1 << 30


def workload_config(device: int, steps: int, warmup: int, resident: bool, hp: bool = True,
                    be: bool = True, seconds: float = 600.0) -> dict:
    tasks = []
    if hp:
        tasks.append({
            "id": "resnet50_rt",
            "load": {"type": "poisson", "priority": 0, "frequency": HP_RATE},
            "client": {"name": "resnet50_rt", "model_name": "resnet50", "priority": 0,
                       "batch_size": 1, "use_cuda_graph": True, "preprocess_time": 0},
        })
    if be:
        tasks.append({
            "id": "resnet50_be",
            "load": ({"type": "continuous", "priority": 1, "max_requests": steps} if steps > 0 else
                     {"type": "continuous", "priority": 1}),
            "client": {"name": "resnet50_be", "model_name": "resnet50", "priority": 1,
                       "batch_size": BE_BATCH, "use_cuda_graph": True, "preprocess_time": 0},
        })
    # With host copies the best-effort tenant double-buffers its input: the next batch is staged
    # in pieces while the current one runs, and copyInput becomes a device-to-device copy.
    cfg = {"time": seconds, "device": device, "seed": 2, "warmup": warmup, "standalone": 5,
           "resident_inputs": resident, "prefetch_inputs": not resident, "tasks": tasks}
    if be and steps > 0:
        cfg["end_when"] = "resnet50_be"
    return cfg


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device = device
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.device)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def measured_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fp:
            return json.load(fp), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def ncu_traffic_bytes() -> tuple[float | None, str]:
    """DRAM read + write bytes of the convolution launches of one best-effort forward, from the
    committed ncu summary (the `dram_bytes_per_step:` line that its capture command produced).
    None when the summary is absent; the number is a capture, not measured by this run."""
    path = os.path.join(ROOT, "profiles", "cgemm_tcgen05_resnet50_b32_dram_traffic.md")
    try:
        with open(path) as fp:
            for line in fp:
                if line.startswith("dram_bytes_per_step:"):
                    return float(line.split(":", 1)[1].split()[0]), os.path.relpath(path, ROOT)
    except OSError:
        pass
    return None, ""


def conv_roofline(api, device: int) -> dict:
    """Per-layer device time of one best-effort forward, measured with CUDA events on the
    launching stream, and the algorithmic FLOP rate of the convolution kernels."""
    ex = api.BLPExecutor()
    ex.init("resnet50", batch=BE_BATCH, seed=1)
    word = api.PreemptWord(1)
    ex.set_word(word)
    s = api.Stream(1)
    data = api.synth_normal(BE_BATCH * 3 * 224 * 224, 0).reshape(BE_BATCH, 3, 224, 224)
    ex.set_input("data", data)
    nk = ex.get_kernel_num()
    infos = [ex.model.get_kernel_info(i) for i in range(nk)]
    for _ in range(3):
        ex.execute(s)
    s.sync()
    events = [api.Event() for _ in range(nk + 1)]
    reps = 5
    per_kernel = [0.0] * nk
    for _ in range(reps):
        # relaunch every kernel with fresh cursors, an event between each pair
        ex.reset_cursors(s)
        events[0].record(s)
        for i in range(nk):
            ex.launch_kernel(i, s)
            events[i + 1].record(s)
        events[nk].sync()
        for i in range(nk):
            per_kernel[i] += events[i].elapsed_ms(events[i + 1]) / reps
    assert ex.error() == (0, 0), ex.error()
    # tensor-core convolutions run CTAs of more than 256 threads; everything else is a CUDA-core kernel
    tc = [i for i in range(nk) if infos[i]["launch_params"][3] > 256]
    dominant = tc if tc else [i for i in range(nk) if "pool" not in infos[i]["name"]]
    flops = sum(infos[i]["flops"] for i in dominant)
    ms = sum(per_kernel[i] for i in dominant)
    total_ms = sum(per_kernel)
    top = sorted(((per_kernel[i], infos[i]["name"]) for i in range(nk)), reverse=True)[:3]
    ex.clear(), word.destroy(), s.destroy()
    for e in events:
        e.destroy()
    return {"conv_flops_per_step": flops, "conv_ms_per_step": ms, "all_kernels_ms_per_step": total_ms,
            "conv_launches_per_step": len(dominant), "tensor_core": bool(tc),
            "conv_bytes_per_step": sum(infos[i]["bytes"] for i in dominant),
            "share_of_step": ms / total_ms if total_ms else 0.0,
            "layers": [(infos[i]["flops"], infos[i]["bytes"]) for i in range(nk)],
            "top": [[round(t, 4), n] for t, n in top]}


def _seeded_params(orc, shapes, std=None):
    import numpy as np

    rng = np.random.default_rng(1)
    params = {}
    for name, shape in shapes.items():
        if name.endswith("weight") and len(shape) > 1:
            fan_in = int(np.prod(shape[1:]))
            params[name] = (rng.standard_normal(shape) * (std or np.sqrt(2.0 / fan_in))).astype(np.float32)
        else:
            params[name] = (rng.standard_normal(shape) * 0.01).astype(np.float32)
    return params


def cpu_baseline(seconds: float = 10.0) -> dict:
    """The oracle's fp32 forward (a port, not the reference's TVM build) timed on host cores: the
    benchmark's model for about `seconds`, then one-thread and other-model figures on short samples."""
    import numpy as np
    from oracle import oracle as orc

    orc.build()
    rng = np.random.default_rng(1)
    params = _seeded_params(orc, orc.resnet_param_shapes())
    data = rng.standard_normal((1, 3, 224, 224)).astype(np.float32)
    orc.forward("resnet50", params, data, fast=True)  # warm-up
    t0 = time.perf_counter()
    images = 0
    while time.perf_counter() - t0 < seconds:
        orc.forward("resnet50", params, data, fast=True)
        images += 1
    dt = time.perf_counter() - t0
    others = {}

    def timed(fn, reps):
        fn()
        t = time.perf_counter()
        for _ in range(reps):
            fn()
        return (time.perf_counter() - t) / reps

    try:
        others["mobilenet_v2_b1_inf_s"] = 1.0 / timed(lambda: orc.forward(
            "mobilenet_v2", _seeded_params(orc, orc.mobilenet_v2_param_shapes()), data, fast=True), 5)
        dn = _seeded_params(orc, orc.densenet_param_shapes())
        others["densenet201_b1_inf_s"] = 1.0 / timed(lambda: orc.forward("densenet201", dn, data, fast=True), 3)
        bp = _seeded_params(orc, orc.bert_param_shapes(), 0.02)
        ids = rng.integers(0, 30522, (1, 128)).astype(np.int64)
        others["bert_base_s128_b1_inf_s"] = 1.0 / timed(lambda: orc.bert_forward(bp, ids), 2)
        x = rng.standard_normal(1 << 26).astype(np.float32)
        y = rng.standard_normal(1 << 26).astype(np.float32)
        others["axpy_2p26_gb_s"] = 12.0 * (1 << 26) / timed(lambda: orc.axpy(1.0009765625, x, y), 3) / 1e9
        a = orc.f32_to_bf16(rng.uniform(-1, 1, (1024, 1024)).astype(np.float32))
        others["gemm_bf16_1024_gflop_s"] = 2.0 * 1024 ** 3 / timed(lambda: orc.gemm_bf16_nt_fast(a, a), 2) / 1e9
        from oracle import miniweather as mw

        sim = mw.Oracle(3200, 1600)
        others["miniweather_3200x1600_cpu_oracle_ms_per_time_step"] = timed(sim.timestep, 2) * 1e3
        if mw.reference_available():
            # the reference's own CUDA source for this workload, compiled unmodified (oracle/Makefile)
            ref = mw.Reference(0)
            ref.timestep(2)
            others["miniweather_3200x1600_reference_kernels_ms_per_time_step"] = ref.time_steps(20) / 20
            ref.close()
        others.update(_graph_cpu_figures())
    except Exception as e:  # noqa: BLE001 - the side figures must not cost the run its line
        others["error"] = repr(e)
    return {"value": images / dt, "unit": "inf/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{images} ResNet-50 fp32 batch-1 forwards of the CPU oracle "
                      f"(fp32 accumulate, OpenMP, every core), {dt:.1f} s",
            "other_samples": others}


def run_reference(args, rank: int) -> None:
    """Reference arm: the reference's arithmetic cannot be built here (TVM-generated kernels are
    absent from its tree), so the CPU port of the same forward is timed, one image per step."""
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1; the CPU arm uses every host core.
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())
    import numpy as np
    from oracle import oracle as orc

    orc.build()
    rng = np.random.default_rng(1)
    params = _seeded_params(orc, orc.resnet_param_shapes())
    data = rng.standard_normal((1, 3, 224, 224)).astype(np.float32)
    for _ in range(max(1, min(args.warmup, 3))):
        orc.forward("resnet50", params, data, fast=True)
    t0 = time.perf_counter()
    for _ in range(args.steps * REF_IMAGES_PER_STEP):
        orc.forward("resnet50", params, data, fast=True)
    dt = time.perf_counter() - t0
    value = args.steps * REF_IMAGES_PER_STEP / dt
    sample = (f"each step = {REF_IMAGES_PER_STEP} of the {BATCHES_PER_STEP * BE_BATCH} images of a step "
              "(ResNet-50 fp32 forward on the CPU, every host core)")
    line = {
        "impl": "reference", "metric": "be_throughput_under_hp_contention", "value": value,
        "unit": "inf/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "be_batch": BE_BATCH, "hp_rate_hz": HP_RATE, "note": sample},
        "cpu_baseline": {"value": value, "unit": "inf/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "inf/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _graph_cpu_figures() -> dict:
    """The graph workloads on the host: the sequential CPU oracle and, where it was built, the
    reference's own CUDA source (compiled unmodified, oracle/Makefile) on the same synthetic graph."""
    import tempfile
    import time as _time

    from gpreempt_b200 import graph_files
    from oracle import graphs

    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        prefix = os.path.join(tmp, "crank", "crank.bel")
        graph_files.write_synthetic(prefix)
        offsets, neighbours, weights = graph_files.read_bel(prefix)
        runs = {"bfs": lambda: graphs.bfs(offsets, neighbours), "sssp": lambda: graphs.sssp(offsets, neighbours, weights),
                "cc": lambda: graphs.cc(offsets, neighbours), "pagerank": lambda: graphs.pagerank(offsets, neighbours)}
        for algo, run in runs.items():
            t0 = _time.perf_counter()
            run()
            out[f"graph_{algo}_cpu_oracle_ms_per_run"] = (_time.perf_counter() - t0) * 1e3
            if graphs.reference_available():
                ref = graphs.Reference(algo, prefix)
                ref.compute(2)
                out[f"graph_{algo}_reference_kernels_ms_per_run"] = ref.compute(10) / 10
                ref.close()
    return out


def miniweather_figures(api, hbm_gbs: float) -> dict:
    """The scientific best-effort workload (the reference's config/Y.json tenant): device time of one
    time step of the 3200 x 1600 grid, replayed from a CUDA graph, and its share of HBM bandwidth
    (12 kernels, each reads two state arrays and writes one: 2.95 GB per time step)."""
    ex = api.BaseExecutor()
    ex.init("miniweather")
    s = api.Stream(0)
    ex.capture_graph(s)
    for _ in range(3):
        ex.execute(s)
    s.sync()
    e0, e1 = api.Event(), api.Event()
    e0.record(s)
    for _ in range(20):
        ex.execute(s)
    e1.record(s)
    s.sync()
    ms = e0.elapsed_ms(e1) / 20
    nbytes = sum(ex.model.get_kernel_info(i)["bytes"] for i in range(ex.get_kernel_num()))
    ex.clear()
    s.destroy()
    return {"ms_per_time_step": ms, "kernels": 12, "algorithmic_gb": nbytes / 1e9,
            "achieved_gb_s": nbytes / (ms * 1e-3) / 1e9, "hbm_frac": nbytes / (ms * 1e-3) / 1e9 / hbm_gbs}


def graph_workload_figures(api) -> dict:
    """The graph-analytics best-effort workloads (the reference's config/Z.json tenants) on a seeded
    synthetic graph of the size of the reference's dataset (52 804 vertices, ~10 million edges; the
    dataset itself is not available): device time of one run to the fixed point, replayed from a CUDA
    graph, with the number of iterations it took."""
    import tempfile

    from gpreempt_b200 import graph_files

    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        prefix = os.path.join(tmp, "crank", "crank.bel")
        info = graph_files.write_synthetic(prefix)
        out["graph"] = {"vertices": info["vertices"], "edges": info["edges"], "data": "synthetic banded, seed 1"}
        for algo in ("bfs", "sssp", "cc", "pagerank"):
            ex = api.BaseExecutor()
            ex.set_graph_path(prefix)
            ex.init(algo)
            s = api.Stream(0)
            ex.capture_graph(s)
            for _ in range(3):
                ex.execute(s)
            s.sync()
            e0, e1 = api.Event(), api.Event()
            e0.record(s)
            for _ in range(20):
                ex.execute(s)
            e1.record(s)
            s.sync()
            out[algo] = {"ms_per_run": e0.elapsed_ms(e1) / 20, "iterations": ex.model.graph_info()["live_iterations"],
                         "kernels": ex.get_kernel_num()}
            ex.clear()
            s.destroy()
    return out


def model_roofline_ms(layers, peak_tflops: float, hbm_gbs: float) -> float:
    """Sum over the kernels of one forward of max(FLOP / tensor peak, bytes / HBM bandwidth)."""
    return sum(max(f / (peak_tflops * 1e12), b / (hbm_gbs * 1e9)) for f, b in layers) * 1e3


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="gpx", choices=["gpx", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--latency-seconds", type=float, default=LATENCY_RUN_S)
    ap.add_argument("--triggers", type=int, default=MICROBENCH_TRIGGERS)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    from gpreempt_b200 import api, dist
    from gpreempt_b200 import binding as B
    import ctypes

    group = dist.init(world, rank)
    device = local_rank if world > 1 else 0
    # Each rank's dispatcher and two client threads get cores of their own when the host has
    # enough of them; otherwise nothing is pinned (two ranks pinned to one core stall each other).
    per_rank = (os.cpu_count() or 1) // max(world, 1)
    os.environ.setdefault("GPX_CORE_BASE", str(min(4, per_rank) * local_rank) if per_rank >= 3 else "-1")
    api.init_cuda(device)

    def launches() -> int:
        c = ctypes.c_uint64()
        B.check(B.load().gpx_launch_count(ctypes.byref(c)))
        return c.value

    batches = args.steps * BATCHES_PER_STEP          # best-effort batches of the timed region
    warm_batches = args.warmup * BATCHES_PER_STEP    # untimed: the driver's warm-up steps
    # solo runs: latency-critical alone (rtonlyclient) and best-effort alone
    hp_solo = json.loads(api.run_workload(
        "rtonlyclient", json.dumps(workload_config(device, 0, 5, False, be=False, seconds=5.0))))
    be_solo = json.loads(api.run_workload(
        "baseclient", json.dumps(workload_config(device, max(200, batches // 4), warm_batches, True, hp=False))))

    sampler = ClockSampler(device)
    dist.barrier(group)
    api.device_sync()
    sampler.start()
    l0 = launches()
    t0 = time.perf_counter()
    resident = json.loads(api.run_workload(
        "gpreemptclient", json.dumps(workload_config(device, batches, warm_batches, True))))
    api.device_sync()
    t1 = time.perf_counter()
    l1 = launches()
    e2e = json.loads(api.run_workload(
        "gpreemptclient", json.dumps(workload_config(device, batches, warm_batches, False))))
    api.device_sync()
    dist.barrier(group)
    clocks = sampler.stop()
    # The latency statistics of the configuration: the same contention workload for the 10 s it
    # names (about 1000 latency-critical requests), host copies included.
    lat = json.loads(api.run_workload(
        "gpreemptclient", json.dumps(workload_config(device, 0, 5, False, seconds=args.latency_seconds))))

    def task(rep, tid):
        return next(t for t in rep["tasks"] if t["id"] == tid)

    be_r, be_e = task(resident, "resnet50_be"), task(e2e, "resnet50_be")
    hp_r, hp_e = task(resident, "resnet50_rt"), task(e2e, "resnet50_rt")
    # device-timed span of exactly K steps (CUDA events on the best-effort stream)
    ms_resident = be_r["deviceSpan(ms)"]
    ms_e2e = be_e["deviceSpan(ms)"]
    worst_resident = dist.max_over_ranks(group, ms_resident)
    worst_e2e = dist.max_over_ranks(group, ms_e2e)
    total_inf = world * batches * BE_BATCH

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        roof = conv_roofline(api, device)
        # flag-to-drain latency and bit-exact resume of the stand-alone best-effort kernels, at the
        # sizes the microbenchmark configuration names (GEMM 8192^3; axpy over 4 GiB vectors)
        microbench = {}
        for kind, size in (("gemm", 8192), ("axpy", MICROBENCH_AXPY_ELEMS)):
            r = api.preempt_microbench(kind, size, args.triggers, seed=5)
            microbench[kind] = {k: r[k] for k in ("triggers", "preempted", "mismatches", "kernel_ms",
                                                  "drain_us_p50", "drain_us_p99", "drain_us_max",
                                                  "seen_us_p50", "late_starts", "raise_call_us_max",
                                                  "drain_after_return_us_max")}
        tflops = roof["conv_flops_per_step"] / (roof["conv_ms_per_step"] * 1e-3) / 1e12
        peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        hbm = peaks["hbm_gbs"]
        batch_ms = worst_resident / batches
        model_ms = model_roofline_ms(roof["layers"], peak, hbm)
        traffic, traffic_src = ncu_traffic_bytes()
        lat_hp, lat_be = task(lat, "resnet50_rt"), task(lat, "resnet50_be")
        solo_hp = task(hp_solo, "resnet50_rt")
        hp_p99 = lat_hp["totalLatency(us)"].get("p99", 0) / 1e3
        hp_solo_p99 = solo_hp["totalLatency(us)"].get("p99", 0) / 1e3
        be_solo_inf = task(be_solo, "resnet50_be")["throughput(inf/s)"]
        value = total_inf / (worst_resident * 1e-3)
        line = {
            "metric": "be_throughput_under_hp_contention",
            "value": value,
            "unit": "inf/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": worst_resident / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f32",
            "data": "synthetic",
            "gpu_launches": l1 - l0,
            "config": {
                "workload": WORKLOAD,
                "be_batch": BE_BATCH, "hp_rate_hz": HP_RATE, "policy": "gpreemptclient (in-kernel yield)",
                "step": f"{BATCHES_PER_STEP} best-effort batches ({BATCHES_PER_STEP * BE_BATCH} inferences) "
                        "under latency-critical Poisson load",
                "l2": "every batch streams 3 GB of layer traffic (weights + activations), larger than L2",
                "e2e": "pinned host input copied in and result copied out on every request; the "
                       "best-effort tenant stages its next input while the current batch runs",
                "latency_run": f"{args.latency_seconds:g} s of the same workload with host copies",
                "microbench": f"configs[2]: {args.triggers} triggers each, bf16 GEMM 8192^3 and fp32 axpy over "
                              f"{MICROBENCH_AXPY_ELEMS * 4 // (1 << 30)} GiB vectors",
            },
            "roofline": {
                "bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s",
                "frac": tflops / peak,
                "traffic": traffic if roof["tensor_core"] else None,
                "traffic_source": f"ncu capture summarised in {traffic_src} (not measured by this run)" if traffic else None,
                "algorithmic_bytes": roof["conv_bytes_per_step"],
                "kernel": ("cgemm_tcgen05_kernel (split-bf16 tensor-core convolution, 3 bf16 MMAs per "
                           "fp32 MAC, best-effort batch 32)") if roof["tensor_core"] else
                          "conv_simt_kernel (fp32 FFMA convolution, best-effort batch 32)",
                "share_of_step": roof["share_of_step"],
                "peak_source": f"bf16_tflops_sustained of {peak_kind} peaks; fp32 work is counted once (2 FLOP "
                               "per multiply-add) against the bf16 peak although it costs three bf16 "
                               "products, the stricter choice (no TF32 peak is measured)",
                "launches_per_step": roof["conv_launches_per_step"] * BATCHES_PER_STEP,
                "ms_per_batch_all_kernels": roof["all_kernels_ms_per_step"],
                "top_kernels_ms": roof["top"],
                "model_roofline_ms_per_batch": model_ms,
                "model_frac": model_ms / batch_ms,
                "model_frac_note": "sum over the kernels of one batch of max(FLOP / peak, bytes / measured HBM "
                                   f"bandwidth {hbm:g} GB/s), divided by the measured time per batch under contention",
            },
            "clocks": clocks,
            "e2e": {
                "value": total_inf / (worst_e2e * 1e-3), "unit": "inf/s",
                "h2d_bytes_per_step": be_e["in_bytes"] * BATCHES_PER_STEP,
                "d2h_bytes_per_step": be_e["out_bytes"] * BATCHES_PER_STEP,
                "ms_per_step": worst_e2e / args.steps,
                # the rest of the metric, measured with host copies
                "hp_p50_ms": lat_hp["totalLatency(us)"].get("p50", 0) / 1e3,
                "hp_p99_ms": hp_p99,
                "hp_requests": lat_hp["requests"],
                "hp_solo_p50_ms": solo_hp["totalLatency(us)"].get("p50", 0) / 1e3,
                "hp_solo_p99_ms": hp_solo_p99,
                "hp_p99_over_solo": hp_p99 / hp_solo_p99 if hp_solo_p99 else None,
                "hp_p99_ms_in_timed_region": hp_e["totalLatency(us)"].get("p99", 0) / 1e3,
                "hp_requests_in_timed_region": hp_e["requests"],
                "be_solo_inf_s": be_solo_inf,
                "be_over_solo": value / world / be_solo_inf if be_solo_inf else None,
                "be_inf_s_in_latency_run": lat_be["throughput(inf/s)"],
                "be_resumes_in_timed_region": e2e["gpus"][0]["beResumes"],
                "preempt_flag_to_drain_p99_us": {k: v["drain_us_p99"] for k, v in microbench.items()},
                "kernel_drain_p99_us": lat["gpus"][0]["kernelDrain(us)"].get("p99"),
                "kernel_drain_p50_us": lat["gpus"][0]["kernelDrain(us)"].get("p50"),
                "host_observed_preempt_p99_us": lat["gpus"][0]["preemptLatency(us)"].get("p99"),
                "resume_mismatches": sum(v["mismatches"] for v in microbench.values()),
            },
            "preempt_microbench": microbench,
            "wall_s_resident_run": t1 - t0,
        }
        if world == 1:
            line["other_workloads"] = {"miniweather_3200x1600": miniweather_figures(api, hbm)}
            try:
                line["other_workloads"]["graph_analytics"] = graph_workload_figures(api)
            except Exception as e:  # noqa: BLE001 - a side figure must not cost the run its line
                line["other_workloads"]["graph_analytics"] = {"error": repr(e)}
        if not args.no_cpu_baseline and world == 1:  # reported at N=1 only
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), flush=True)
    dist.finish(group)


if __name__ == "__main__":
    main()
