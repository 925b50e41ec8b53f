"""GPU tests of the tensor-parallel FFN pair (gate/up column-parallel, down row-parallel, one-shot all-reduce
fused into the down GEMM's epilogue).

On one GPU all ranks of a group live in one process and every push is queued before any reduce, so no kernel
ever waits for another: that checks the data path, the receive-area layout and the (rank, segment) summation
order bit for bit.  The cross-GPU run (one process per GPU, IPC-mapped receive areas) is the worker at the
bottom, started under torch.distributed.run when the machine has at least two GPUs.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
H, F, N_OUT, MAX_ROWS = 256, 1024, 256, 32
TOL = 5e-3      # max |gpu - oracle| / max |oracle|: the device's expf in SiLU may flip an int8 of the hidden row


def make_weights(orc, seed):
    rng = np.random.default_rng(seed)
    gate = orc.quantize_q8_0(rng.normal(0, 0.05, (F, H)).astype(np.float32))
    up = orc.quantize_q8_0(rng.normal(0, 0.05, (F, H)).astype(np.float32))
    down = orc.quantize_q8_0(rng.normal(0, 0.05, (N_OUT, F)).astype(np.float32))
    return gate, up, down


def oracle_rank_partials(orc, gu, dn, f, x):
    """Split partials [S][M][N_OUT] of one rank's down GEMM, from the CPU restatement."""
    q, d = orc.quantize_act(x)
    y = orc.gemm_engine(gu, 2 * f, H, q, d)
    g, u = y[:, :f], y[:, f:]
    h = (g / (np.float32(1) + np.exp(-g, dtype=np.float32)) * u).astype(np.float32)
    hq, hd = orc.quantize_act(h)
    return orc.gemm_engine(dn, N_OUT, f, hq, hd, want_partials=True)[1]


def ordered_sum(parts):
    """float32 sum of [R][S][M][N]: each rank's segments ascending, then the ranks ascending."""
    acc = None
    for rank_parts in parts:
        mine = rank_parts[0].copy()
        for p in rank_parts[1:]:
            mine = (mine + p).astype(np.float32)
        acc = mine if acc is None else (acc + mine).astype(np.float32)
    return acc


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("M", [1, 4, 17, 32])
def test_tp_ffn_ranks_in_one_process(qb, orc, ctx, world, M):
    gate, up, down = make_weights(orc, 7)
    f = F // world
    shards = [qb.tp.shard_blocks(gate, up, down, F, H, N_OUT, world, r) for r in range(world)]
    wts = [(qb.Weight.from_blocks(ctx, gu, 2 * f, H), qb.Weight.from_blocks(ctx, dn, N_OUT, f)) for gu, dn in shards]
    groups, areas = qb.tp.local_groups(ctx, world, MAX_ROWS, H, f, N_OUT)
    S = orc.ksplit_policy(N_OUT, f)
    region = S * MAX_ROWS * N_OUT
    rng = np.random.default_rng(100 + M)
    for step in range(3):                               # three steps: both parities, and a receive slot reused
        x = rng.normal(0, 1, (M, H)).astype(np.float32)
        xd = ctx.array(x)
        ys = [ctx.empty((M, N_OUT), np.float32) for _ in range(world)]
        for r in range(world):
            groups[r].push(wts[r][0], wts[r][1], xd, M)
        for r in range(world):
            groups[r].reduce(M, ys[r])
        ctx.sync()
        got = [y.download() for y in ys]
        for r in range(1, world):
            assert np.array_equal(got[0], got[r]), "ranks disagree"
        # the receive area of every rank holds what all ranks pushed (their split partials, or from 32 rows on
        # their sums over the segments); the rank-ordered sum of it IS the result
        Sp = S if M < 32 else 1
        for r in range(world):
            raw = areas[r].download()
            slot = raw[256:].view(np.float32)[(step & 1) * world * region:((step & 1) + 1) * world * region]
            parts = np.stack([slot[k * region:k * region + Sp * M * N_OUT].reshape(Sp, M, N_OUT) for k in range(world)])
            assert np.array_equal(ordered_sum(parts), got[r]), "reduce order"
        want_parts = np.stack([oracle_rank_partials(orc, shards[r][0], shards[r][1], f, x) for r in range(world)])
        want = ordered_sum(want_parts)
        err = np.abs(got[0] - want).max() / np.abs(want).max()
        assert err < TOL, (world, M, step, err)
    for g in groups:
        g.close()
    for w in wts:
        w[0].free(); w[1].free()


def test_tp_sharded_sum_equals_unsharded_ffn(qb, orc, ctx):
    """The 4-way sharded result equals the unsharded FFN up to the order of the fp32 additions."""
    gate, up, down = make_weights(orc, 9)
    M = 4
    x = np.random.default_rng(5).normal(0, 1, (M, H)).astype(np.float32)
    outs = []
    for world in (1, 4):
        f = F // world
        shards = [qb.tp.shard_blocks(gate, up, down, F, H, N_OUT, world, r) for r in range(world)]
        wts = [(qb.Weight.from_blocks(ctx, gu, 2 * f, H), qb.Weight.from_blocks(ctx, dn, N_OUT, f)) for gu, dn in shards]
        groups, _areas = qb.tp.local_groups(ctx, world, MAX_ROWS, H, f, N_OUT)
        xd, y = ctx.array(x), ctx.empty((M, N_OUT), np.float32)
        for r in range(world):
            groups[r].push(wts[r][0], wts[r][1], xd, M)
        groups[0].reduce(M, y)
        ctx.sync()
        outs.append(y.download())
        for g in groups:
            g.close()
    assert np.abs(outs[0] - outs[1]).max() / np.abs(outs[0]).max() < 1e-5


def test_tp_reduce_gives_up_when_a_peer_never_arrives(qb, orc, ctx):
    """Rank 1 never pushes: rank 0's reduce runs out its bounded wait, the next synchronize reports it and the
    context keeps working."""
    gate, up, down = make_weights(orc, 11)
    f = F // 2
    gu, dn = qb.tp.shard_blocks(gate, up, down, F, H, N_OUT, 2, 0)
    w_gu, w_dn = qb.Weight.from_blocks(ctx, gu, 2 * f, H), qb.Weight.from_blocks(ctx, dn, N_OUT, f)
    groups, _areas = qb.tp.local_groups(ctx, 2, MAX_ROWS, H, f, N_OUT)
    x = ctx.array(np.ones((2, H), np.float32))
    y = ctx.empty((2, N_OUT), np.float32)
    groups[0].push(w_gu, w_dn, x, 2)
    groups[0].reduce(2, y)
    with pytest.raises(qb.QbError, match="bounded wait"):
        ctx.sync()
    ctx.sync()                                          # the flag was cleared; the context is usable
    z = ctx.array(np.arange(8, dtype=np.float32))
    assert np.array_equal(z.download(), np.arange(8, dtype=np.float32))
    for g in groups:
        g.close()


WORKER = r"""
import json, os, sys
import numpy as np
sys.path.insert(0, %(root)r)
import __graft_entry__ as entry
import torch
import torch.distributed as dist
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("gloo")
pkg = entry.load_package()
O = entry.load_oracle()
ctx = pkg.Context(local)
H, F, N_OUT, MAX_ROWS = %(dims)s
rng = np.random.default_rng(7)
gate = O.quantize_q8_0(rng.normal(0, 0.05, (F, H)).astype(np.float32))
up = O.quantize_q8_0(rng.normal(0, 0.05, (F, H)).astype(np.float32))
down = O.quantize_q8_0(rng.normal(0, 0.05, (N_OUT, F)).astype(np.float32))
f = F // world
gu, dn = pkg.tp.shard_blocks(gate, up, down, F, H, N_OUT, world, rank)
w_gu, w_dn = pkg.Weight.from_blocks(ctx, gu, 2 * f, H), pkg.Weight.from_blocks(ctx, dn, N_OUT, f)
group, area, opened = pkg.tp.ipc_group(ctx, dist, MAX_ROWS, H, f, N_OUT)
ok, worst = True, 0.0
for step, M in enumerate([4, 1, 17, 4, 4, 32]):
    x = np.random.default_rng(100 + step).normal(0, 1, (M, H)).astype(np.float32)
    y = ctx.empty((M, N_OUT), np.float32)
    dist.barrier()                      # ranks enter a step together: the device-side wait is about a second
    group.ffn(w_gu, w_dn, ctx.array(x), M, y)
    ctx.sync()
    got = y.download()
    all_got = [None] * world
    dist.all_gather_object(all_got, got.tobytes())
    ok = ok and all(b == all_got[0] for b in all_got)
    if rank == 0:
        parts = []
        for r in range(world):
            g_r, d_r = pkg.tp.shard_blocks(gate, up, down, F, H, N_OUT, world, r)
            q, d = O.quantize_act(x)
            yy = O.gemm_engine(g_r, 2 * f, H, q, d)
            g, u = yy[:, :f], yy[:, f:]
            h = (g / (np.float32(1) + np.exp(-g, dtype=np.float32)) * u).astype(np.float32)
            hq, hd = O.quantize_act(h)
            parts.append(O.gemm_engine(d_r, N_OUT, f, hq, hd, want_partials=True)[1])
        acc = None
        for rp in parts:
            mine = rp[0].copy()
            for p in rp[1:]:
                mine = (mine + p).astype(np.float32)
            acc = mine if acc is None else (acc + mine).astype(np.float32)
        worst = max(worst, float(np.abs(got - acc).max() / np.abs(acc).max()))
dist.barrier()
if rank == 0:
    print(json.dumps({"ranks_identical": bool(ok), "worst_rel_err": worst, "world": world}))
group.close()
pkg.tp.ipc_release(ctx, opened)
dist.barrier()
dist.destroy_process_group()
"""


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_ffn_one_process_per_gpu(world, tmp_path):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER % dict(root=ROOT, dims=(H, F, N_OUT, MAX_ROWS)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % world,
                          "--master-addr", "127.0.0.1", "--master-port", "29671", str(script)],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    r = json.loads([ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1])
    assert r["ranks_identical"] and r["worst_rel_err"] < TOL, r


STEP_WORKER = r"""
import json, os, sys
import numpy as np
sys.path.insert(0, %(root)r)
import __graft_entry__ as entry
import torch
import torch.distributed as dist
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("gloo")
pkg = entry.load_package()
O = entry.load_oracle()
ctx = pkg.Context(local)
cfg = pkg.configs.tiny()
K, N_NEW = 3, 40
prompt = O.synth_prompt(pkg.configs.PROMPT_SEED + 31, cfg.vocab_size, 50)
model = pkg.Model.synth_tp(ctx, cfg, pkg.configs.MODEL_SEED, rank, world)
f = cfg.n_ff // world


def run(k):
    b = pkg.Batch(model, 1, 256, k)
    group, area, opened = pkg.tp.ipc_group(ctx, dist, b.max_rows, cfg.n_embd, f, cfg.n_embd)
    b.set_tp(group)
    ctx.sync(); dist.barrier()
    b.prefill(0, prompt)
    toks, logits = list(b.read_output()[0]), [b.last_logits(1)[0].copy()]
    while len(toks) < N_NEW:
        b.mtp_step() if k else b.greedy_step()
        toks += b.read_output()[0]
    st = b.stats()
    ctx.sync(); dist.barrier()
    b.close(); group.close(); pkg.tp.ipc_release(ctx, opened)
    return toks[:N_NEW], logits[0], st

greedy, lg, _ = run(0)
spec, _, st = run(K)
everyone = [None] * world
dist.all_gather_object(everyone, (greedy, spec, lg.tobytes()))
out = {"world": world, "lossless": spec == greedy, "ranks_identical": all(e == everyone[0] for e in everyone), "steps": st["steps"]}
if rank == 0:
    # the single-GPU model of the same seed: same function up to the order of the FFN's additions
    whole = pkg.Model(ctx, cfg, pkg.configs.MODEL_SEED)
    b = pkg.Batch(whole, 1, 256, 0)
    b.prefill(0, prompt)
    ref = b.last_logits(1)[0]
    out["prefill_logit_rel_err_vs_one_gpu"] = float(np.abs(lg - ref).max() / np.abs(ref).max())
    b.close(); whole.close()
    print(json.dumps(out))
model.close()
dist.barrier()
dist.destroy_process_group()
"""


@pytest.mark.parametrize("world", [2, 4])
def test_tp_step_is_lossless_one_process_per_gpu(world, tmp_path):
    """The FFN pairs of the whole step tensor-sharded over `world` GPUs (qb_model_create_synth_tp + qb_batch_set_tp):
    every rank emits the same tokens, the speculative stream equals the greedy stream of the same rank count exactly, and
    the prefill logits stay within the model's rounding noise of the single-GPU model."""
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    script = tmp_path / "tp_step_worker.py"
    script.write_text(STEP_WORKER % dict(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % world,
                          "--master-addr", "127.0.0.1", "--master-port", "29673", str(script)],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    r = json.loads([ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1])
    print(r)
    assert r["lossless"] and r["ranks_identical"] and r["steps"] > 0, r
    assert r["prefill_logit_rel_err_vs_one_gpu"] < 2.5e-2, r


def test_tp_step_path_on_one_gpu(qb, orc, ctx):
    """The tensor-parallel form of the step with a group of one rank (nothing waits): the speculative stream equals the
    greedy stream of the same form exactly, and its logits stay within the rounding noise of the ordinary form (the FFN
    output is added to the residual stream as one sum instead of segment by segment)."""
    cfg = qb.configs.tiny()
    prompt = orc.synth_prompt(qb.configs.PROMPT_SEED + 32, cfg.vocab_size, 40)
    model = qb.Model.synth_tp(ctx, cfg, qb.configs.MODEL_SEED, 0, 1)
    plain = qb.Model(ctx, cfg, qb.configs.MODEL_SEED)
    assert model.weight_bytes == plain.weight_bytes
    streams, logits = [], []
    for k in (0, 3):
        b = qb.Batch(model, 1, 256, k)
        groups, _areas = qb.tp.local_groups(ctx, 1, b.max_rows, cfg.n_embd, cfg.n_ff, cfg.n_embd)
        b.set_tp(groups[0])
        b.prefill(0, prompt)
        toks = list(b.read_output()[0])
        logits.append(b.last_logits(1)[0].copy())
        while len(toks) < 30:
            b.mtp_step() if k else b.greedy_step()
            toks += b.read_output()[0]
        streams.append(toks[:30])
        b.close()
        groups[0].close()
    assert streams[0] == streams[1]
    assert np.array_equal(logits[0], logits[1])
    b = qb.Batch(plain, 1, 256, 0)
    b.prefill(0, prompt)
    ref = b.last_logits(1)[0]
    assert float(np.abs(logits[0] - ref).max() / np.abs(ref).max()) < 2.5e-2
    b.close(); model.close(); plain.close()
