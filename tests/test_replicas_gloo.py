"""CPU test of the N > 1 host logic with two gloo ranks: request sharding and whole-job aggregation
(max of the per-rank device times, sum of the per-rank token counts)."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, %r)
    import __graft_entry__ as entry
    import torch.distributed as dist
    pkg = entry.load_package()
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    mine = pkg.replicas.shard_requests(7, world, rank)
    t, c = pkg.replicas.aggregate(dist, [10.0 + rank, 5.0 - rank], [100.0 * (rank + 1), len(mine)])
    if rank == 0:
        print(json.dumps({"t": t.tolist(), "c": c.tolist(), "mine": mine, "tput": pkg.replicas.throughput(c[0], t[0])}))
    dist.barrier()
    dist.destroy_process_group()
""") % ROOT


def test_two_gloo_ranks_shard_and_aggregate(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29653", str(script)],
                         capture_output=True, text=True, env=env, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1]
    r = json.loads(line)
    assert r["t"] == [11.0, 5.0]            # max over ranks
    assert r["c"] == [300.0, 7.0]           # sums: tokens, and every request served exactly once
    assert r["mine"] == [0, 1, 2, 3]
    assert abs(r["tput"] - 300.0 / 11.0e-3) < 1e-6


def test_shard_requests_covers_everything_once():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    pkg = entry.load_package()
    for n in (1, 7, 32, 33):
        for world in (1, 2, 4, 8):
            got = sum((pkg.replicas.shard_requests(n, world, r) for r in range(world)), [])
            assert got == list(range(n))
