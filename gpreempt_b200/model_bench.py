"""Stand-alone forward time of the built-in graphs: `python -m gpreempt_b200.model_bench`.

One JSON line per (model, batch, dtype): milliseconds per forward with the inputs resident on the
device, timed with CUDA events on the launching stream over `--iters` back-to-back executions
after `--warmup` untimed ones, the inference rate, and the arithmetic rate from the per-kernel
FLOP counts the model reports (`gpx_model_kernel_info`).  The default list is the set of models and
shapes the contention configurations use (latency-critical batch 1, best-effort batches).
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import api

DEFAULT = [
    # model, batch, dtype, seq_len
    ("resnet50", 1, "float32", 0), ("resnet50", 32, "float32", 0),
    ("resnet50", 1, "bfloat16", 0), ("resnet50", 32, "bfloat16", 0),
    ("bert_base", 1, "float16", 128), ("vgg16", 16, "float16", 0),
    ("mobilenet_v2", 1, "bfloat16", 0), ("densenet201", 64, "bfloat16", 0),
    ("bert_base", 32, "bfloat16", 512),
]


def parse_specs(text: str) -> list[tuple[str, int, str, int]]:
    """"model:batch:dtype[:seq_len]" entries separated by commas -> (model, batch, dtype, seq_len)."""
    out = []
    for item in text.split(","):
        f = item.strip().split(":")
        if len(f) < 3 or len(f) > 4:
            raise ValueError(f"'{item}': expected model:batch:dtype[:seq_len]")
        if f[2] not in ("float32", "bfloat16", "float16"):
            raise ValueError(f"'{item}': dtype must be float32, bfloat16 or float16")
        out.append((f[0], int(f[1]), f[2], int(f[3]) if len(f) > 3 else 0))
    return out


def synthetic_input(ex) -> np.ndarray | None:
    """Seeded input of the shape and type the model's `data` tensor has: N(0,1) images, or token
    ids uniform over the rows of the word-embedding table.  None for a workload without request
    data (miniweather: every execute advances the resident simulation)."""
    try:
        shape = ex.model.shape("data")
    except api.GpxError:
        return None
    info = ex.model.get_storage_info(ex.model.find_storage_idx("data"))
    if info["stype"] == "int64":
        vocab = ex.model.shape("embeddings.word_embeddings.weight")[0]
        return np.random.default_rng(6).integers(0, vocab, shape).astype(np.int64)
    return api.synth_normal(int(np.prod(shape)), 0, 0).reshape(shape)


def run(model: str, batch: int, dtype: str, seq_len: int, iters: int, warmup: int, graph: bool) -> dict:
    ex = api.BaseExecutor()
    ex.init(model, batch=batch, seed=1, seq_len=seq_len, dtype=dtype)
    data = synthetic_input(ex)
    if data is not None:
        ex.set_input("data", data)
    s = api.Stream(0)
    if graph:
        ex.capture_graph(s)
    for _ in range(warmup):
        ex.execute(s)
    s.sync()
    e0, e1 = api.Event(), api.Event()
    e0.record(s)
    for _ in range(iters):
        ex.execute(s)
    e1.record(s)
    s.sync()
    ms = e0.elapsed_ms(e1) / iters
    nk = ex.get_kernel_num()
    infos = [ex.model.get_kernel_info(i) for i in range(nk)]
    flops = sum(k["flops"] for k in infos)
    nbytes = sum(k["bytes"] for k in infos)
    err = ex.error()
    ex.clear()
    s.destroy()
    return {"model": model, "batch": batch, "dtype": dtype, "seq_len": seq_len, "kernels": nk,
            "cuda_graph": graph, "ms_per_forward": ms, "inf_per_s": batch / (ms * 1e-3),
            "gflop_per_forward": flops / 1e9, "tflops": flops / (ms * 1e-3) / 1e12,
            "layer_bytes_gb": nbytes / 1e9, "error": list(err)}


def per_kernel(model: str, batch: int, dtype: str, seq_len: int, reps: int) -> None:
    """Prints one line per kernel of the model: device time between CUDA events recorded around
    each launch on the launching stream (mean of `reps` passes), tiles, FLOP and byte rates."""
    ex = api.BLPExecutor()
    ex.init(model, batch=batch, seed=1, seq_len=seq_len, dtype=dtype)
    word = api.PreemptWord(1)
    ex.set_word(word)
    s = api.Stream(1)
    data = synthetic_input(ex)
    if data is not None:
        ex.set_input("data", data)
    nk = ex.get_kernel_num()
    infos = [ex.model.get_kernel_info(i) for i in range(nk)]
    for _ in range(3):
        ex.execute(s)
    s.sync()
    events = [api.Event() for _ in range(nk + 1)]
    ms = [0.0] * nk
    for _ in range(reps):
        ex.reset_cursors(s)
        events[0].record(s)
        for i in range(nk):
            ex.launch_kernel(i, s)
            events[i + 1].record(s)
        events[nk].sync()
        for i in range(nk):
            ms[i] += events[i].elapsed_ms(events[i + 1]) / reps
    total = sum(ms)
    print(f"# {model} batch {batch} {dtype}: {nk} kernels, {total:.3f} ms (sum of per-kernel times)")
    print(f"# {'kernel':44s} {'grid':>5s} {'thr':>4s} {'tiles':>7s} {'us':>9s} {'share':>6s} {'TFLOP/s':>8s} {'GB/s':>8s}")
    for i, k in enumerate(infos):
        lp = k["launch_params"]
        t = ms[i] * 1e-3
        print(f"{k['name']:46s} {lp[0]:5d} {lp[3]:4d} {k['total_tiles']:7d} {ms[i] * 1e3:9.1f} "
              f"{ms[i] / total:6.3f} {k['flops'] / t / 1e12:8.1f} {k['bytes'] / t / 1e9:8.0f}")
    ex.clear(), word.destroy(), s.destroy()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--graph", action="store_true", help="replay a captured CUDA graph instead of launching")
    ap.add_argument("--kernels", default="", help="model:batch:dtype[:seq_len] - print the per-kernel times instead")
    ap.add_argument("--only", default="", help="comma-separated model:batch:dtype[:seq_len] entries")
    args = ap.parse_args()
    api.init_cuda(args.device)
    if args.kernels:
        (model, batch, dtype, seq), = parse_specs(args.kernels)
        per_kernel(model, batch, dtype, seq, args.iters)
        return
    todo = parse_specs(args.only) if args.only else DEFAULT
    for model, batch, dtype, seq in todo:
        print(json.dumps(run(model, batch, dtype, seq, args.iters, args.warmup, args.graph)), flush=True)


if __name__ == "__main__":
    main()
