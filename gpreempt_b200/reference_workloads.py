"""The reference's own evaluation workloads A, B, C, D, E, Y and Z (its Fig. 4-6) on this library.

    python -m gpreempt_b200.reference_workloads [--seconds 10] [--only A,B]

Each workload is the task list of the reference's config/<name>.json (same model names, periodic
rates, priorities, 200 us of simulated pre-processing, batch 1, fp32), written here from those
parameters.  For each one the latency-critical task runs alone (the reference's LCO client) and
then with its best-effort tenants under `gpreemptclient` (GP); the line printed per workload
gives the mean end-to-end latency of the latency-critical task in both runs (the figure the
reference plots: DISB's avgTotalLatency, pre-processing included), what the contention adds, and
the best-effort throughput in requests per second summed over the best-effort tasks.

Z runs the graph-analytics tenants; its dataset (crankseg_1) ships with neither repository, so
the files are written to a scratch directory from the seeded synthetic graph of the same size
(gpreempt_b200.graph_files), unless --graph names the prefix of existing .col/.dst/.val files.

--config FILE runs a task file in the reference's schema as it is (its config/REAL.json with the
recorded arrival traces, for instance) through the same two clients, for the file's own "time"
unless --seconds is given.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile

from . import api


def _task(tid: str, model: str, priority: int, hz: float, preprocess_us: int = 200,
          load: str = "periodic", graph_path: str | None = None) -> dict:
    client = {"name": tid, "model_name": model, "priority": priority, "batch_size": 1,
              "use_cuda_graph": graph_path is None, "preprocess_time": preprocess_us}
    if graph_path is not None:
        client["graph_path"] = graph_path
    return {"id": tid, "load": {"type": load, "priority": 0, "frequency": hz}, "client": client}


_FIVE = ("resnet152", "densenet", "vgg", "inception", "bert")

WORKLOADS = {
    # config/A.json, B.json: VGG latency-critical against ResNet-152 best-effort, 100 and 220 Hz each
    "A": [_task("vgg_rt", "vgg", 0, 100), _task("resnet152_be", "resnet152", 1, 100)],
    "B": [_task("vgg_rt", "vgg", 0, 220), _task("resnet152_be", "resnet152", 1, 220)],
    # config/C.json: one latency-critical task against five best-effort models at 100 Hz
    "C": [_task("vgg_rt", "vgg", 0, 100)] + [_task(m + "_be", m, 1, 100) for m in _FIVE],
    # config/D.json, E.json: five latency-critical models at 20 Hz against the same five as
    # best-effort tenants at 100 Hz; periodic arrivals in D, Poisson arrivals in E
    "D": [_task(m + "_rt", m, 0, 20) for m in _FIVE] + [_task(m + "_be", m, 1, 100) for m in _FIVE],
    "E": [_task(m + "_rt", m, 0, 20, load="poisson") for m in _FIVE]
         + [_task(m + "_be", m, 1, 100, load="poisson") for m in _FIVE],
    # config/Y.json: the scientific tenant (no pre-processing) at 150 Hz
    "Y": [_task("vgg_rt", "vgg", 0, 100), _task("miniweather_be", "miniweather", 1, 150, 0)],
    # config/Z.json: bfs, sssp, pagerank and cc on one graph at 100 Hz each (no CUDA graph, as there)
    "Z": [_task("vgg_rt", "vgg", 0, 100)] + [_task(a + "_be", a, 1, 100, graph_path="")
                                             for a in ("bfs", "sssp", "pagerank", "cc")],
}


def run(name: str, seconds: float, graph: str = "") -> dict:
    tasks = json.loads(json.dumps(WORKLOADS[name]))
    if any("graph_path" in t["client"] for t in tasks):
        with tempfile.TemporaryDirectory() as tmp:
            if not graph:
                from . import graph_files

                graph = os.path.join(tmp, "crank", "crank.bel")
                graph_files.write_synthetic(graph)
            for t in tasks:
                if "graph_path" in t["client"]:
                    t["client"]["graph_path"] = os.path.abspath(graph)
            return _run(name, tasks, seconds)
    return _run(name, tasks, seconds)


def _run(name: str, tasks: list, seconds: float) -> dict:
    cfg = {"time": seconds, "seed": 1, "warmup": 3, "standalone": 3, "tasks": tasks}
    alone = json.loads(api.run_workload("rtonlyclient", json.dumps(cfg)))
    both = json.loads(api.run_workload("gpreemptclient", json.dumps(cfg)))
    # The reference plots one latency per workload: the mean over every latency-critical request.
    def lc_mean_us(report: dict) -> float:
        lcs = [t for t in report["tasks"] if t["priority"] == 0 and t["requests"]]
        return sum(t["avgTotalLatency(us)"] * t["requests"] for t in lcs) / sum(t["requests"] for t in lcs)

    lc = [t for t in both["tasks"] if t["priority"] == 0]
    be = [t for t in both["tasks"] if t["priority"] != 0]
    return {
        "workload": name,
        "lc_mean_ms_alone": lc_mean_us(alone) / 1e3,
        "lc_mean_ms_contended": lc_mean_us(both) / 1e3,
        "lc_added_us": lc_mean_us(both) - lc_mean_us(alone),
        "lc_p99_ms_contended": max(t["totalLatency(us)"]["p99"] for t in lc) / 1e3,
        "lc_requests": sum(t["requests"] for t in lc),
        "be_req_per_s": sum(t["avgThroughput(req/s)"] for t in be),
        "be_dropped_arrivals": sum(t["droppedArrivals"] for t in be),
        "kernel_drain_p99_us": both["gpus"][0]["kernelDrain(us)"].get("p99"),
    }


def run_file(path: str, seconds: float | None) -> dict:
    with open(path) as f:
        cfg = json.load(f)
    return _run(os.path.splitext(os.path.basename(path))[0], cfg["tasks"],
                seconds if seconds is not None else float(cfg.get("time", 10.0)))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--seconds", type=float, default=None, help="length of each run (default 10, or the file's time)")
    ap.add_argument("--config", default="", help="a task file in the reference's schema, run instead of --only")
    ap.add_argument("--only", default="A,B,C,D,E,Y,Z")
    ap.add_argument("--graph", default="", help="prefix of the graph files of workload Z")
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args()
    names = [n for n in a.only.split(",") if n]
    for n in names:
        if n not in WORKLOADS:
            ap.error(f"unknown workload {n!r} (have {', '.join(WORKLOADS)})")
    api.init_cuda(a.device)
    if a.config:
        print(json.dumps(run_file(a.config, a.seconds)), flush=True)
        return
    for n in names:
        print(json.dumps(run(n, a.seconds if a.seconds is not None else 10.0, a.graph)), flush=True)


if __name__ == "__main__":
    main()
