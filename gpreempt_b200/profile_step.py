"""Small, self-terminating workloads for `ncu` captures of the hot kernels.

    python -m gpreempt_b200.profile_step gemm  [--size 8192] [--iters 2]
    python -m gpreempt_b200.profile_step axpy  [--size 268435456] [--iters 2]
    python -m gpreempt_b200.profile_step model [--model resnet50] [--batch 32] [--dtype float32]
                                               [--seq-len 0] [--iters 2]
    python -m gpreempt_b200.profile_step model --model pagerank:/tmp/g/g.bel   (graph files: gpreempt_b200.graph_files)

Each run launches the kernels of interest `iters` times with preemption armed (the word stays
clear) and exits; inputs are larger than L2 so DRAM counters are meaningful, and at most a few
GB are held on the device.
"""
from __future__ import annotations

import argparse

from . import api


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "axpy", "model"])
    ap.add_argument("--size", type=int, default=0)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--seq-len", type=int, default=0)
    a = ap.parse_args()
    api.init_cuda(0)
    s = api.Stream(1)
    word = api.PreemptWord(1)
    if a.what == "gemm":
        n = a.size or 8192
        da, db = api.DeviceBuffer(n * n * 2), api.DeviceBuffer(n * n * 2)
        dc = api.DeviceBuffer(n * n * 2)
        api.fill_uniform(da, n * n, True, 3, 0, s)
        api.fill_uniform(db, n * n, True, 3, 1, s)
        ctx = api.GemmContext()
        blp = api.BlpContext(word, trace=False)
        for _ in range(a.iters):
            ctx.reset(), blp.reset()
            api.gemm_bf16(da, db, dc, n, n, n, ctx, blp, s)
            s.sync()
        assert ctx.status() == (0, 0)
    elif a.what == "axpy":
        n = a.size or (1 << 28)
        dx, dy = api.DeviceBuffer(n * 4), api.DeviceBuffer(n * 4)
        api.fill_uniform(dx, n, False, 4, 0, s)
        api.fill_uniform(dy, n, False, 4, 1, s)
        blp = api.BlpContext(word, trace=False)
        for _ in range(a.iters):
            blp.reset()
            api.axpy(1.0009765625, dx, dy, n, blp, s)
            s.sync()
    else:
        ex = api.BLPExecutor()
        graph = a.model.split(":")[0] in ("bfs", "sssp", "cc", "pagerank")
        ex.init(a.model, batch=a.batch, seed=None if graph else 1, dtype=a.dtype, seq_len=a.seq_len)
        ex.set_word(word)
        if a.model.startswith("miniweather") or graph:
            data = None  # no request data: every execute advances the resident simulation / reruns the algorithm
        elif a.model.startswith("bert"):
            import numpy as np

            vocab = 30522 if a.model == "bert_base" else 1000
            data = np.random.default_rng(6).integers(0, vocab, (a.batch, a.seq_len or 128)).astype(np.int64)
        else:
            data = api.synth_normal(a.batch * 3 * 224 * 224, 0).reshape(a.batch, 3, 224, 224)
        if data is not None:
            ex.set_input("data", data)
        for _ in range(a.iters):
            ex.execute(s)
            assert ex.getStopPoint(s) == -1
    print("done")


if __name__ == "__main__":
    main()
