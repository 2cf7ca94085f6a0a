"""The multi-rank plumbing on CPU: two gloo ranks meet at the barrier, take the max of their
times and split clients round-robin (one scheduler replica per rank, no data-path collective)."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, %r)
    from gpreempt_b200 import dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    g = dist.init(world, rank)
    dist.barrier(g)
    worst = dist.max_over_ranks(g, 10.0 + rank)
    total = dist.sum_over_ranks(g, 1.0 + rank)
    mine = dist.shard(["c0", "c1", "c2", "c3", "c4"], world, rank)
    dist.barrier(g)
    dist.finish(g)
    print(json.dumps({"rank": rank, "worst": worst, "total": total, "mine": mine}))
""") % ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_ranks_barrier_max_and_shard():
    import json

    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-c", CHILD], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0, err
        outs.append(json.loads(out.strip().splitlines()[-1]))
    outs.sort(key=lambda o: o["rank"])
    assert [o["worst"] for o in outs] == [11.0, 11.0]
    assert [o["total"] for o in outs] == [3.0, 3.0]
    assert outs[0]["mine"] == ["c0", "c2", "c4"] and outs[1]["mine"] == ["c1", "c3"]


def test_single_process_needs_no_group():
    sys.path.insert(0, ROOT)
    from gpreempt_b200 import dist

    g = dist.init(1, 0)
    assert g is None
    dist.barrier(g)
    assert dist.max_over_ranks(g, 3.5) == 3.5
    assert dist.shard([1, 2, 3], 1, 0) == [1, 2, 3]
    dist.finish(g)
