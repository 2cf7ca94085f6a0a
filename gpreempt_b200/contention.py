"""Contention report for a client configuration: `python -m gpreempt_b200.contention config/C3_bert_vs_vgg16.json`.

Runs the configuration three times on one GPU, as the reference's evaluation does with its
clients (src/common-clients/rtonlyclient.cpp:130-141 for the latency-critical tasks alone,
src/common-clients/baseclient.cpp for tasks without preemption, src/cuda-clients/gpreemptclient.cpp
for the preemptive policy): the latency-critical tasks alone, the best-effort tasks alone, and
all of them under the chosen policy.  Prints one JSON object: per latency-critical task p50 / p99
alone and under contention and their ratio, per best-effort task the inference rate alone and
under contention and their ratio, and the device-side drain time of preempted kernels.
"""
from __future__ import annotations

import argparse
import copy
import json

from . import api


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("config")
    ap.add_argument("--client", default="gpreemptclient")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--seconds", type=float, default=0.0, help="override the configuration's run time")
    args = ap.parse_args()
    cfg = json.load(open(args.config))
    cfg["device"] = args.device
    if args.seconds > 0:
        cfg["time"] = args.seconds
    api.init_cuda(args.device)

    def is_hp(t):
        return t["client"].get("priority", 1) == 0

    def run(client, tasks):
        c = copy.deepcopy(cfg)
        c["tasks"] = tasks
        rep = json.loads(api.run_workload(client, json.dumps(c)))
        return {t["id"]: t for t in rep["tasks"]}, rep["gpus"][0]

    hp_tasks = [t for t in cfg["tasks"] if is_hp(t)]
    be_tasks = [t for t in cfg["tasks"] if not is_hp(t)]
    hp_alone, _ = run("baseclient", hp_tasks) if hp_tasks else ({}, None)
    be_alone, _ = run("baseclient", be_tasks) if be_tasks else ({}, None)
    both, gpu = run(args.client, cfg["tasks"])

    out = {"config": args.config, "client": args.client, "seconds": cfg["time"], "latency_critical": {},
           "best_effort": {}}
    for t in hp_tasks:
        a, b = hp_alone[t["id"]], both[t["id"]]
        la, lb = a["totalLatency(us)"], b["totalLatency(us)"]
        out["latency_critical"][t["id"]] = {
            "requests": b["requests"],
            "alone_p50_us": la.get("p50"), "alone_p99_us": la.get("p99"),
            "contended_p50_us": lb.get("p50"), "contended_p99_us": lb.get("p99"),
            "p99_ratio": (lb.get("p99") / la.get("p99")) if la.get("p99") else None,
        }
    for t in be_tasks:
        a, b = be_alone[t["id"]], both[t["id"]]
        out["best_effort"][t["id"]] = {
            "alone_inf_per_s": a["throughput(inf/s)"], "contended_inf_per_s": b["throughput(inf/s)"],
            "ratio": b["throughput(inf/s)"] / a["throughput(inf/s)"] if a["throughput(inf/s)"] else None,
        }
    if be_tasks and len(be_tasks) > 1:
        # tenants that share the GPU alone already split it: compare the sums as well
        sa = sum(be_alone[t["id"]]["throughput(inf/s)"] for t in be_tasks)
        sb = sum(both[t["id"]]["throughput(inf/s)"] for t in be_tasks)
        out["best_effort_sum_ratio"] = sb / sa if sa else None
    out["kernel_drain_us"] = gpu["kernelDrain(us)"]
    out["word_raises"] = gpu["wordRaises"]
    out["be_resumes"] = gpu["beResumes"]
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
