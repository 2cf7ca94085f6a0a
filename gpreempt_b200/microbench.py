"""Preemption microbenchmark (config "C2"): flag-to-drain latency and bit-exact resume of the
bf16 GEMM (M = N = K = 8192, tensor-bound) and the fp32 axpy (2^30 elements per vector,
HBM-bound) under uniformly random preemption triggers.

    python -m gpreempt_b200.microbench [--triggers 1000] [--gemm 8192] [--axpy 1073741824]
"""
from __future__ import annotations

import argparse
import json

from . import api


def run(triggers: int, gemm: int, axpy: int, transport: int = 1, device: int = 0) -> dict:
    api.init_cuda(device)
    out = {}
    for kind, size in (("gemm", gemm), ("axpy", axpy)):
        if size <= 0:
            continue
        r = api.preempt_microbench(kind, size, triggers, seed=5, transport=transport)
        r.pop("drain_us"), r.pop("seen_us")
        if kind == "gemm":
            r["tflops"] = 2.0 * size ** 3 / (r["kernel_ms"] * 1e-3) / 1e12
        else:
            r["gb_s"] = 12.0 * size / (r["kernel_ms"] * 1e-3) / 1e9
        out[kind] = r
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--triggers", type=int, default=1000)
    ap.add_argument("--gemm", type=int, default=8192)
    ap.add_argument("--axpy", type=int, default=1 << 30)
    ap.add_argument("--transport", type=int, default=1)
    a = ap.parse_args()
    print(json.dumps(run(a.triggers, a.gemm, a.axpy, a.transport)))
