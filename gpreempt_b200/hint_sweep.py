"""Hint-based pre-preemption sweep: `python -m gpreempt_b200.hint_sweep`.

The reference raises its preemption early: a hint sent `preprocess_time - SWITCH_TIME` into the
data-prepare phase lets the best-effort context be switched out before the latency-critical
kernels are submitted (src/cuda-clients/gpreemptclient.cpp:21,203-219,267-291; the trade-off is
the paper's Fig. 7).  This sweep runs the contention workload (latency-critical ResNet-50 b1,
Poisson arrivals, `preprocess_time` on the host; best-effort ResNet-50 b32 closed loop) with the
hint off, raised when the input copy begins (lead 0) and raised `lead` microseconds before the
end of the prepare phase, and prints one JSON line per point: latency-critical inference latency
(submission to completion) and end-to-end latency, and what the reservation costs the best-effort
tenant.
"""
from __future__ import annotations

import argparse
import json

from . import api


def config(device: int, seconds: float, rate: float, preprocess_us: int, hint: bool, lead_us: int,
           be_batch: int) -> dict:
    return {
        "time": seconds, "seed": 2, "device": device, "preempt_hint": hint, "hint_lead_us": lead_us,
        "tasks": [
            {"id": "resnet50_rt", "load": {"type": "poisson", "priority": 0, "frequency": rate},
             "client": {"name": "resnet50_rt", "model_name": "resnet50", "priority": 0, "batch_size": 1,
                        "use_cuda_graph": True, "preprocess_time": preprocess_us}},
            {"id": "resnet50_be", "load": {"type": "continuous", "priority": 1},
             "client": {"name": "resnet50_be", "model_name": "resnet50", "priority": 1, "batch_size": be_batch,
                        "use_cuda_graph": True, "preprocess_time": 0}},
        ],
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--seconds", type=float, default=4.0)
    ap.add_argument("--rate", type=float, default=100.0)
    ap.add_argument("--preprocess-us", type=int, default=300)
    ap.add_argument("--be-batch", type=int, default=32)
    ap.add_argument("--leads", default="0,50,100,200,300")
    args = ap.parse_args()
    api.init_cuda(args.device)
    points = [("off", False, 0)] + [(f"lead {l} us", True, int(l)) for l in args.leads.split(",")]
    for label, hint, lead in points:
        rep = json.loads(api.run_workload("gpreemptclient", json.dumps(
            config(args.device, args.seconds, args.rate, args.preprocess_us, hint, lead, args.be_batch))))
        tasks = {t["id"]: t for t in rep["tasks"]}
        hp, be = tasks["resnet50_rt"], tasks["resnet50_be"]
        g = rep["gpus"][0]
        print(json.dumps({
            "hint": label,
            "hp_requests": hp["requests"],
            "hp_infer_us_avg": hp["avgInferLatency(us)"],
            "hp_total_us_p50": hp["totalLatency(us)"]["p50"],
            "hp_total_us_p99": hp["totalLatency(us)"]["p99"],
            "hp_standalone_total_us": hp["standAloneTotalLatency(us)"],
            "hp_dispatch_delay_us_p99": g["hpDispatchDelay(us)"].get("p99"),
            "kernel_drain_us_p99": g["kernelDrain(us)"].get("p99"),
            "be_inf_per_s": be["throughput(inf/s)"],
            "be_resumes": g["beResumes"],
        }), flush=True)


if __name__ == "__main__":
    main()
