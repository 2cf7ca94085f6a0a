"""Writes tests/golden/graph_reference.json from the reference's own graph-analytics kernels.

Run where a GPU is, after `make -C oracle ref` built oracle/_ref/libgraphcompute_ref.so from the
reference's unmodified src/workloads/graphcompute.cu:

    python tests/golden/make_graph_golden.py

Two seeded synthetic graphs (gpreempt_b200.graph_files.synthetic_banded) are written to a scratch
directory in the reference's file layout and run through GraphComputeRaw::{BFS,SSSP,CC,PageRank}.
For the small one the file keeps every label, distance, component id and rank; for the one of the
size of the reference's dataset it keeps digests (SHA-256 of the integer arrays, sums, extrema, the
values at 64 fixed vertices), so the CPU oracle can be checked where no GPU is.
"""
import hashlib
import json
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from gpreempt_b200 import graph_files  # noqa: E402
from oracle import graphs  # noqa: E402

OUT = os.path.join(ROOT, "tests", "golden", "graph_reference.json")
GRAPHS = {"small": dict(vertices=400, degree=10, band=25, seed=5, components=3),
          "crank": dict(vertices=52804, degree=201, band=1500, seed=1, components=1)}
ALGOS = ("bfs", "sssp", "cc", "pagerank")


def digest(algo, arr, full):
    picks = np.random.default_rng(99).integers(0, len(arr), 64)
    d = {"picks": picks.tolist(), "at_picks": [float(x) if algo == "pagerank" else int(x) for x in arr[picks]]}
    if algo == "pagerank":
        d.update(sum=float(arr.astype(np.float64).sum()), min=float(arr.min()), max=float(arr.max()))
    else:
        d.update(sha256=hashlib.sha256(arr.astype(np.uint64).tobytes()).hexdigest(),
                 sum=int(arr.astype(np.uint64).sum() % (1 << 62)), max=int(arr.max()))
    if full:
        d["values"] = [float(x) for x in arr] if algo == "pagerank" else [int(x) for x in arr]
    return d


def main():
    doc = {"source": "reference src/workloads/graphcompute.cu compiled unmodified (oracle/Makefile, target ref)",
           "graphs": {}}
    with tempfile.TemporaryDirectory() as tmp:
        for name, spec in GRAPHS.items():
            prefix = os.path.join(tmp, name, name + ".bel")
            info = graph_files.write_synthetic(prefix, **spec)
            entry = {"spec": spec, "edges": info["edges"], "results": {}, "reference_ms_per_run_on_this_gpu": {}}
            for algo in ALGOS:
                ref = graphs.Reference(algo, prefix)
                ref.compute(2)
                entry["results"][algo] = digest(algo, ref.result(), full=name == "small")
                entry["reference_ms_per_run_on_this_gpu"][algo] = ref.compute(10) / 10
                ref.close()
            doc["graphs"][name] = entry
    with open(OUT, "w") as f:
        json.dump(doc, f, indent=1)
    print("wrote", OUT)


if __name__ == "__main__":
    main()
