"""Benchmark of the MTP speculative-decode step (27B-class qwen35 shape, Q8_0, k=3).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--sub all|none]

One "step" is one speculative step of one request: 3 chained MTP-head drafts, the 4-row target verification forward
over all 64 layers, greedy acceptance and commit.  The headline workload is benchmark configuration 2 (batch 1, prompt
2048 seeded uniform token ids in paged fp16 KV, page 16) in its forced-acceptance form: seeded random weights give the
MTP head no natural acceptance, so the drafts that are verified follow a fixed schedule of accepted lengths with the
counts of a 70 % per-position acceptance (6 x 0, 4 x 1, 3 x 2, 7 x 3 accepted drafts in every block of 20 steps, the
same on every rank); the MTP-head drafts are still computed and timed every step.  Prints ONE JSON line on rank 0.

With one GPU the line also carries, under "sub", short driver-timed runs of the other configurations: 3 (prompt
32768), 4 (32 requests, prompts 512-8192, 128 verify rows) and 5 (the isolated verify-GEMM sweep).  With --gpus N > 1
(launched by torch.distributed.run) every rank runs an independent replica of the step -- the path has no exchange
step, so the only collectives are the barrier and the max/sum of the timings -- and "sub" carries the one sharded
case, the tensor-parallel FFN pair across the N ranks (all-reduce fused into the down GEMM against GEMMs + NCCL).

--impl reference times the CPU restatement of the reference's arithmetic (oracle/; the reference has no CPU
implementation of this path and its CUDA build is not a CPU baseline) on the host cores.

Other workloads, one GPU, for profiling (each prints its own lines):
    --workload gemm      configuration 5 in full: both kernels, every M, bit-identity between them
    --workload attn      paged gated attention alone at --ctx (comma list), cold L2
    --workload timeline  per-launch device timeline of the tensor-core GEMMs of one step
    --workload serve     the continuous-batching loops at the 27B shape, wall clock
    --workload tokenizer the byte-level BPE tokenizer on the host (no GPU): MB/s beside the reference's own, where built
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

K_DRAFT = 3
PROMPT_LEN = 2048
ACCEPT_RATE = 0.7
FORCE_SEED = 0xACCE97
NCU_TRAFFIC_RATIO = 94.79 / 94.70
EXPECTED_EMITTED = 1 + ACCEPT_RATE + ACCEPT_RATE ** 2 + ACCEPT_RATE ** 3   # tokens per step at 70 % per position
INT8_PEAK_TOPS = 4570.0      # tcgen05.mma.kind::i8 128x256x32 back to back from shared memory, one CTA per SM, measured on this pool
BLOCK = 20                   # steps per block of the acceptance schedule
BLOCK_COUNTS = (6, 4, 3, 7)  # accepted lengths 0..3 per block: 20 * (0.3, 0.21, 0.147, 0.343) rounded


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="step", choices=["step", "gemm", "attn", "timeline", "serve", "tokenizer"])
    ap.add_argument("--sub", default="all", choices=["all", "none"], help="the short runs of configurations 3, 4, 5 / the TP FFN pair")
    ap.add_argument("--layers", type=int, default=64, help="target layers (64 = the 27B-class shape)")
    ap.add_argument("--prompt", type=int, default=PROMPT_LEN)
    ap.add_argument("--seqs", type=int, default=1, help="concurrent requests per GPU of the headline run")
    ap.add_argument("--prompt-min", type=int, default=512, help="with --seqs > 1 prompt lengths are uniform in [prompt-min, prompt]")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--lean", action="store_true", help="profiling aid: headline timing only (no phase / trace / timeline / e2e passes)")
    # workload options
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shapes", default="17408x5120,5120x17408,5120x6144,34816x5120,151936x5120")
    ap.add_argument("--m", "--rows", dest="m", default="1,4,16,64,128,512")
    ap.add_argument("--impls", default="1,2")
    ap.add_argument("--ctx", default="2048,32768")
    ap.add_argument("--tp", action="store_true", help="--workload gemm: the tensor-parallel FFN pair over the ranks of this launch")
    ap.add_argument("--slots", type=int, default=8)
    ap.add_argument("--requests", type=int, default=24)
    return ap.parse_args()


# ---- clocks --------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons during the timed region."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        """Number of samples so far (brackets the timed region inside a longer sampling run)."""
        return len(self.lines)

    def stop(self, first=0, last=None):
        """Summary of the samples [first, last); of all samples (taken under load) when the region caught none."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        window = self.lines[first:last] if len(self.lines[first:last]) > 0 else self.lines
        for ln in window:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---- the acceptance schedule ----------------------------------------------------------------------
def accept_schedule(n_steps, warmup, k=K_DRAFT):
    """Accepted draft count of every step after the prompt: blocks of 20 steps, each holding the accepted lengths
    0..3 with the counts of a 70 % per-position acceptance in a seeded order; the first timed step (index `warmup`)
    starts a block, so a timed window of whole blocks emits exactly 51 tokens per 20 steps on every rank."""
    base = np.concatenate([np.full(c, a, np.int64) for a, c in enumerate(BLOCK_COUNTS)])
    base = np.minimum(base, k)
    rs = np.random.RandomState(FORCE_SEED)
    blocks = [rs.permutation(base) for _ in range((n_steps + warmup) // BLOCK + 3)]
    flat = np.concatenate(blocks)
    shift = (-warmup) % BLOCK
    return flat[shift:shift + n_steps]


def window_tokens(steps, warmup, k=K_DRAFT):
    """Tokens one request emits in the timed window of `steps` steps (the same figure in both arms of the benchmark)."""
    return int((accept_schedule(warmup + steps, warmup, k)[warmup:] + 1).sum())


def forced_table(stream, plen, sched, vocab, k=K_DRAFT):
    """forced[p] = the guess offered for the token at absolute position p: the true continuation for the drafts the
    schedule accepts, a different token for the first one it rejects (and everywhere else)."""
    forced = ((stream + 1) % vocab).astype(np.int32)
    pos = plen
    for a in sched:
        forced[pos + 1:pos + 1 + a] = stream[pos + 1:pos + 1 + a]
        pos += int(a) + 1
    return forced, pos


# ---- algorithmic bytes ------------------------------------------------------------------------------
def q8_bytes(rows, cols):
    return rows * cols / 32 * 34


def step_bytes(cfg, k, ctx_lens):
    """Algorithmic HBM bytes of one speculative step of the requests at the given context lengths: every weight the
    verify forward, the k drafts and the MTP prefix pass stream (each once per pass, whatever the row count), the K/V
    every attention layer reads (one pass for all rows of a request), the DeltaNet state read once and written per
    checkpoint."""
    H, F, V = cfg.n_embd, cfg.n_ff, cfg.vocab_size
    inner, kvd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    qkv = (2 * cfg.ssm_num_k_heads + cfg.ssm_num_v_heads) * cfg.ssm_head_dim
    vdim = cfg.ssm_num_v_heads * cfg.ssm_head_dim
    ffn = q8_bytes(2 * F, H) + q8_bytes(H, F)
    attn = q8_bytes(2 * inner + 2 * kvd, H) + q8_bytes(H, inner) + ffn
    dn = q8_bytes(qkv + vdim + 2 * cfg.ssm_num_v_heads, H) + q8_bytes(H, vdim) + ffn
    n_attn = sum(1 for i in range(cfg.n_layers) if cfg.full_attention_interval and (i + 1) % cfg.full_attention_interval == 0)
    n_dn = cfg.n_layers - n_attn
    head = q8_bytes(V, H)
    verify_w = n_attn * attn + n_dn * dn + head
    draft_w = attn + q8_bytes(H, 2 * H) + head
    prefix_w = q8_bytes(H, 2 * H) + q8_bytes(2 * kvd, H)
    kv = sum(ctx_lens) * kvd * 2 * 2 * (n_attn + k)
    state = len(ctx_lens) * n_dn * (k + 2) * cfg.ssm_num_v_heads * cfg.ssm_head_dim * cfg.ssm_head_dim * 4
    return {"verify_weights": verify_w, "draft_weights": k * draft_w, "mtp_prefix_weights": prefix_w, "kv": kv, "deltanet_state": state,
            "total": verify_w + k * draft_w + prefix_w + kv + state}


# ---- CPU baseline ----------------------------------------------------------------------------------
def cpu_step_sample(O, models, seqs):
    """One bounded CPU sample of the step on a 4-layer slice of the 27B shape; returns seconds scaled
    to the full 64-layer step: 3 drafts + head + 16 x (4-layer slice of the 4-row verify)."""
    A, Z = seqs
    toks = np.array([1, 2, 3, 4], np.int32)
    t0 = time.perf_counter(); A.forward_rows(toks); tA = time.perf_counter() - t0      # 4 layers + head
    t0 = time.perf_counter(); Z.forward_rows(toks); th = time.perf_counter() - t0      # head only
    t0 = time.perf_counter(); Z.mtp_step(K_DRAFT); tz = time.perf_counter() - t0       # 3 drafts + head
    return max(tz - th, 0.0) + 16.0 * max(tA - th, 0.0) + th


def cpu_setup(O, pkg):
    cfg = pkg.configs.qwen27b()
    ocfg = O.ModelConfig(**cfg.as_dict())
    mA = O.Model(ocfg, pkg.configs.MODEL_SEED, max_layers=4)
    mZ = O.Model(ocfg, pkg.configs.MODEL_SEED, max_layers=0)
    prompt = O.synth_prompt(pkg.configs.PROMPT_SEED + 2, cfg.vocab_size, 8)
    A, Z = O.Seq(mA, 4096), O.Seq(mZ, 4096)
    A.prefill(prompt, 8)
    Z.prefill(prompt, 8)
    return (mA, mZ), (A, Z)


CPU_SAMPLE_TEXT = ("EXTRAPOLATED: one step per sample on a 4-layer slice (3 DeltaNet + 1 attention) of the 27B shape with the full LM "
                   "head and MTP layer at context 8: 3 MTP drafts + 4-row verify; the slice's layer time is scaled x16 to 64 layers; "
                   "tokens per step = the acceptance schedule's, as in the GPU arm")


def all_host_threads():
    """The CPU legs use every core the process may run on: the launcher of multi-rank runs exports
    OMP_NUM_THREADS=1, which must not throttle the CPU baseline.  Call before the CPU library is loaded."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(n)


def run_reference(args, rank):
    if rank != 0:
        return
    all_host_threads()
    pkg, O = entry.load_package(), entry.load_oracle()
    models, seqs = cpu_setup(O, pkg)
    for _ in range(args.warmup):
        cpu_step_sample(O, models, seqs)
    t = [cpu_step_sample(O, models, seqs) for _ in range(args.steps)]
    sec = float(np.mean(t))
    tok_per_step = window_tokens(args.steps, args.warmup) / args.steps
    value = tok_per_step / sec
    line = {
        "impl": "reference", "metric": "accepted_tok_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic", "extrapolated": True, "tokens_per_step": tok_per_step,
        "config": workload_config(args),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": O.num_threads(), "kind": "port", "sample": CPU_SAMPLE_TEXT},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(args):
    return {"workload": "configuration 2: 27B-class qwen35 shape (%d layers, hidden 5120, 24q/4kv x 256, DeltaNet 16k/48v x 128, "
                        "FFN 17408, vocab 151936), Q8_0, MTP k=3, batch %d, prompt %d, forced drafts: accepted lengths in blocks of 20 steps "
                        "with the counts of a 70%% per-position acceptance (6/4/3/7 x 0/1/2/3), same schedule on every rank" % (args.layers, args.seqs, args.prompt),
            "draft_k": K_DRAFT, "prompt_len": args.prompt, "requests_per_gpu": args.seqs, "page_size": 16, "kv_dtype": "fp16", "accept_rate_target": ACCEPT_RATE,
            "l2": "weights streamed per step (28.7 GB) exceed the 126 MB L2, no flush needed",
            "replicas": args.gpus}


# ---- GPU arm ---------------------------------------------------------------------------------------
def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (earlier pool measurement)"


class SpecRun:
    """A batch of requests after prompt ingestion, its greedy continuation and the forced-draft table of a schedule."""

    def __init__(self, pkg, ctx, model, prompts, n_steps, warmup, k=K_DRAFT):
        self.pkg, self.ctx, self.model, self.k = pkg, ctx, model, k
        cfg = model.cfg
        self.ns, self.plen = len(prompts), [len(p) for p in prompts]
        self.sched = accept_schedule(n_steps, warmup, k)
        n_tok = int((self.sched + 1).sum()) + k + 4
        # room for every step at its upper bound: a device-resident loop does not read the step records, and the host's
        # position mirror then advances by k + 1 per step
        self.max_ctx = max(self.plen) + max(n_tok, (n_steps + 2) * (k + 1)) + 16
        self.stride = self.max_ctx + 8
        e0, e1 = ctx.event(), ctx.event()
        self.b = pkg.Batch(model, self.ns, self.max_ctx, k)
        ctx.sync(); ctx.record(e0)
        for s, p in enumerate(prompts):
            self.b.prefill(s, p)
        ctx.record(e1); ctx.sync()
        self.prefill_ms = ctx.elapsed_ms(e0, e1)
        first = [t[0] for t in self.b.read_output()]
        self.snap = self.b.snapshot()
        # the non-speculative greedy continuation on the same batch (also the losslessness reference), then back to the
        # state after the prompt
        greedy = [[t] for t in first]
        ctx.sync(); ctx.record(e0)
        for _ in range(n_tok - 1):
            self.b.greedy_step()
            for s, t in enumerate(self.b.read_output()):
                greedy[s] += t
        ctx.record(e1); ctx.sync()
        self.greedy_ms = ctx.elapsed_ms(e0, e1) / max(n_tok - 1, 1)
        self.b.restore(self.snap)
        self.stream = np.zeros((self.ns, self.stride), np.int32)          # stream[s][p] = token at absolute position p
        forced = np.zeros((self.ns, self.stride), np.int32)
        for s in range(self.ns):
            self.stream[s, :self.plen[s]] = prompts[s]
            self.stream[s, self.plen[s]:self.plen[s] + len(greedy[s])] = greedy[s]
            forced[s], _ = forced_table(self.stream[s], self.plen[s], self.sched, cfg.vocab_size, k)
        self.forced = forced
        self.sdev = ctx.array(forced)

    def device_step(self):
        b = self.b
        b.mtp_draft()
        b.mtp_force_drafts(self.sdev, self.stride)
        b.mtp_verify()
        b.mtp_accept_commit()

    def rewind(self):
        self.b.restore(self.snap)

    def timed(self, dist, warmup, steps):
        """Device-resident loop: `warmup` untimed steps, then `steps` steps back to back with no host read-back inside.
        Returns (ms, emitted tokens, accepted drafts, launches, emitted tokens per sequence)."""
        ctx, b = self.ctx, self.b
        e0, e1 = ctx.event(), ctx.event()
        for _ in range(warmup):
            self.device_step()
            b.read_output()
        pos0 = [b.position(s) for s in range(self.ns)]
        if dist is not None:
            dist.barrier()
        ctx.sync()
        s0, l0 = b.stats(), ctx.launches
        ctx.record(e0)
        for _ in range(steps):
            self.device_step()
        ctx.record(e1)
        ctx.sync()
        ms = ctx.elapsed_ms(e0, e1)
        s1, l1 = b.stats(), ctx.launches
        b.read_output()
        pos1 = [b.position(s) for s in range(self.ns)]
        return ms, s1["emitted"] - s0["emitted"], s1["accepted"] - s0["accepted"], l1 - l0, [p1 - p0 for p0, p1 in zip(pos0, pos1)]

    def close(self):
        self.b.free_snapshot(self.snap)
        self.b.close()


def seeded_prompts(pkg, cfg, rank_free_seed, lens):
    rs = np.random.RandomState(rank_free_seed & 0x7FFFFFFF)
    return [rs.randint(0, cfg.vocab_size, n).astype(np.int32) for n in lens]


def run_ours(args, rank, world, local_rank, dist):
    pkg = entry.load_package()
    want_cpu = rank == 0 and world == 1 and not args.no_cpu_baseline
    if want_cpu:
        all_host_threads()
    O = entry.load_oracle() if want_cpu else None
    ctx = pkg.Context(local_rank)
    cfg = pkg.configs.qwen27b(args.layers)
    K, W, k, ns = args.steps, args.warmup, K_DRAFT, args.seqs
    phase_steps, prof_steps = (0, 0) if args.lean else (min(K, 16), min(K, 8))
    total_steps = W + K + phase_steps + prof_steps + 2
    model = pkg.Model(ctx, cfg, pkg.configs.MODEL_SEED)
    # seeded prompts, the same on every rank: one request of --prompt tokens, or --seqs requests with lengths uniform in
    # [--prompt-min, --prompt]
    rs = np.random.RandomState((pkg.configs.PROMPT_SEED + 2) & 0x7FFFFFFF)
    plen = [args.prompt] if ns == 1 else [int(v) for v in rs.randint(args.prompt_min, args.prompt + 1, ns)]
    prompts = seeded_prompts(pkg, cfg, pkg.configs.PROMPT_SEED + 3, plen)

    sampler = ClockSampler(local_rank)
    sampler.start()
    run = SpecRun(pkg, ctx, model, prompts, total_steps, W)
    b, ev = run.b, [ctx.event() for _ in range(6)]

    # 1. device-resident timing: K steps back to back, no host read-back inside
    first_sample = sampler.mark()
    dev_ms, dev_emitted, dev_accepted, launches, _ = run.timed(dist, W, K)
    last_sample = sampler.mark()

    ph, prof, trace, tl = [0.0, 0.0, 0.0], None, [], None
    if not args.lean:
        # 2. phase split in the real stream: three events per step at the phase boundaries, nothing else in the stream
        for _ in range(phase_steps):
            ctx.record(ev[0]); b.mtp_draft(); b.mtp_force_drafts(run.sdev, run.stride)
            ctx.record(ev[1]); b.mtp_verify()
            ctx.record(ev[2]); b.mtp_accept_commit()
            ctx.record(ev[3]); ctx.sync()
            for i in range(3):
                ph[i] += ctx.elapsed_ms(ev[i], ev[i + 1]) / phase_steps
            b.read_output()
        # 3. per-launch timing of every Q8_0 GEMM (an event pair around each launch: serialises them, conservative)
        ctx.prof_enable(True)
        for _ in range(prof_steps):
            run.device_step()
            b.read_output()
        prof = ctx.prof_summary()
        ctx.prof_enable(False)
        # one traced step: per-kernel time shares measured live (event after every launch)
        ctx.trace_enable(True)
        run.device_step()
        trace = ctx.trace_summary()
        ctx.trace_enable(False)
        b.read_output()
        # one step with device-side stamps inside the tensor-core GEMM (no events in the stream: the in-stream truth)
        ctx.timeline_enable(512)
        run.device_step()
        tl = ctx.timeline_gemm_summary(*ctx.timeline_read(512))
        ctx.timeline_enable(0)
        b.read_output()

    # 4. end to end through the host-driven API from the state after the prompt (same warm-up, same forced guesses):
    #    drafts come from pinned host memory every step and the step record goes back to the host every step
    e2e_ms, n_e2e, lossless = float("nan"), 0, None
    if not args.lean:
        run.rewind()
        pos = list(run.plen)
        pinned = ctx.pinned((ns, k), np.int32)

        def host_step():
            b.mtp_draft()
            for s_ in range(ns):
                pinned[s_, :] = run.forced[s_, pos[s_] + 1:pos[s_] + 1 + k]
            b.mtp_set_drafts(pinned)
            b.mtp_verify()
            b.mtp_accept_commit()
            return b.read_output()

        e2e_tokens = [[] for _ in range(ns)]
        for _ in range(W):
            for s_, t in enumerate(host_step()):
                pos[s_] += len(t)
        start_pos = list(pos)
        if dist is not None:
            dist.barrier()
        ctx.sync()
        ctx.record(ev[4])
        t0 = time.perf_counter()
        for _ in range(K):
            for s_, t in enumerate(host_step()):
                e2e_tokens[s_] += t
                pos[s_] += len(t)
        ctx.record(ev[5])
        ctx.sync()
        e2e_wall = time.perf_counter() - t0
        e2e_ms = max(ctx.elapsed_ms(ev[4], ev[5]), e2e_wall * 1e3)
        lossless = all(e2e_tokens[s_] == list(run.stream[s_, start_pos[s_] + 1:pos[s_] + 1]) for s_ in range(ns))
        n_e2e = sum(len(t) for t in e2e_tokens)
    clocks = sampler.stop(first_sample, last_sample)

    # 5. aggregate over replicas: max time, summed tokens
    tmax, tsum = pkg.replicas.aggregate(dist, [dev_ms, e2e_ms if e2e_ms == e2e_ms else 0.0], [float(dev_emitted), float(n_e2e), float(launches)])
    agg = np.concatenate([tmax, tsum])

    greedy_ms, prefill_ms = run.greedy_ms, run.prefill_ms
    sub = {}
    if args.sub == "all" and not args.lean:
        run.close()
        run = None
        if world == 1:
            sub = sub_records(pkg, ctx, model, cfg)
        else:
            sub = {"tp_ffn": tp_ffn_record(pkg, ctx, dist, rank, world, local_rank),
                   "tp_step": tp_step_record(pkg, ctx, dist, rank, world, cfg, prompts[0])}
    if rank != 0:
        if run:
            run.close()
        model.close(); ctx.close()
        return
    peak, peak_src = peaks()
    sb = step_bytes(cfg, k, [p + W * EXPECTED_EMITTED for p in plen])
    ms_per_step = agg[0] / K
    line = {
        "metric": "accepted_tok_per_s", "value": agg[2] / (agg[0] * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": workload_config(args), "clocks": clocks,
        "tokens_per_step": dev_emitted / (K * ns), "value_at_expected_acceptance": ns * world * EXPECTED_EMITTED / (ms_per_step * 1e-3),
        "gpu_launches": int(agg[4]),
        "step": {"accepted_per_step": dev_accepted / (K * ns), "emitted_per_step": dev_emitted / (K * ns), "acceptance_rate": dev_accepted / (K * k * ns),
                 "greedy_ms_per_token": greedy_ms, "greedy_tok_per_s": ns * 1e3 / greedy_ms, "prefill_ms": prefill_ms,
                 "algorithmic_bytes": {n: round(v) for n, v in sb.items()},
                 "step_hbm_frac": (sb["total"] / 1e9) / (ms_per_step * 1e-3) / peak if world == 1 else None},
    }
    if not args.lean:
        achieved = prof["bytes"] / (prof["ms"] * 1e-3) / 1e9 if prof["ms"] > 0 else 0.0
        line["e2e"] = {"value": agg[3] / (agg[1] * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": ns * k * 4, "d2h_bytes_per_step": ns * (k + 3) * 4,
                       "ms_per_step": agg[1] / K, "lossless_vs_greedy": bool(lossless)}
        line["roofline"] = {
            "bound": "hbm", "kernel": "gemm_tc_kernel + gemm_dp4a_kernel (every Q8_0 projection of the step, the fused gate/up launch included)",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
            # DRAM bytes per launch: the ncu capture of this kernel on a 94.70 MB weight read 94.79 MB
            # (ratio 1.001, the weight is streamed once); scaled to this run's average launch
            "traffic": NCU_TRAFFIC_RATIO * prof["bytes"] / max(prof["launches"], 1),
            "launches": prof["launches"], "launches_per_step": prof["launches"] / max(prof_steps, 1),
            "avg_launch_us": prof["ms"] * 1e3 / max(prof["launches"], 1), "bytes_per_launch_avg": prof["bytes"] / max(prof["launches"], 1),
            # the tensor-core kernel timed by global-timer stamps inside it, with the dependent-launch overlap of
            # the real stream intact (event pairs serialise the launches and add their own ~2 us)
            "in_stream": {"launches": tl["launches"], "busy_us": tl["busy_us"], "gaps_between_us": tl["gap_us"],
                          "achieved": tl["bytes"] / max(tl["busy_us"], 1e-9) / 1e3, "unit": "GB/s",
                          "frac": tl["bytes"] / max(tl["busy_us"], 1e-9) / 1e3 / peak}}
        line["step"].update({"verify_us": ph[1] * 1e3, "draft_us": ph[0] * 1e3, "accept_commit_us": ph[2] * 1e3,
                             "phase_split": "CUDA events at the three phase boundaries only, %d steps of the real stream" % phase_steps})
        ttot = sum(t for _, _, t in trace) or 1.0
        line["step"]["kernel_shares"] = {n: {"launches": c, "us": round(t, 1), "share": round(t / ttot, 4)} for n, c, t in trace}
    if sub:
        line["sub"] = sub
    if O is not None:
        models, seqs = cpu_setup(O, pkg)
        cpu_step_sample(O, models, seqs)
        t = [cpu_step_sample(O, models, seqs) for _ in range(3)]
        sec = float(np.mean(t))
        line["cpu_baseline"] = {"value": (dev_emitted / (K * ns)) / sec, "unit": "tok/s", "cores": O.num_threads(), "kind": "port",
                                "sample": CPU_SAMPLE_TEXT, "ms_per_step": sec * 1e3}
    print(json.dumps(line))
    if run:
        run.close()
    model.close(); ctx.close()


# ---- short runs of the other configurations -----------------------------------------------------------
def spec_record(pkg, ctx, model, cfg, prompts, steps, warmup, label):
    peak, _ = peaks()
    run = SpecRun(pkg, ctx, model, prompts, warmup + steps + 1, warmup)
    ms, emitted, accepted, launches, per_seq = run.timed(None, warmup, steps)
    ns = len(prompts)
    # losslessness of the device-resident run: every sequence sits exactly where the schedule puts it, and one more
    # host-read step emits the greedy continuation
    sched_tok = int((run.sched[warmup:warmup + steps] + 1).sum())
    run.device_step()
    out = run.b.read_output()
    ok = all(n == sched_tok for n in per_seq)
    for s in range(ns):
        p = run.b.position(s)
        ok = ok and out[s] == list(run.stream[s, p - len(out[s]) + 1:p + 1])
    sb = step_bytes(cfg, K_DRAFT, [len(p) + (warmup + steps / 2) * EXPECTED_EMITTED for p in prompts])
    rec = {"workload": label, "requests": ns, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
           "tok_per_s": emitted / (ms * 1e-3), "tokens_per_step_per_request": emitted / (steps * ns), "lossless_vs_greedy": bool(ok),
           "greedy_ms_per_step": run.greedy_ms, "prefill_tok_per_s": sum(len(p) for p in prompts) / (run.prefill_ms * 1e-3),
           "algorithmic_bytes": {n: round(v) for n, v in sb.items()}, "step_hbm_frac": (sb["total"] / 1e9) / (ms / steps * 1e-3) / peak,
           "gpu_launches": launches}
    run.close()
    return rec


def gemm_time(pkg, ctx, w, M, impl, iters, S=0):
    L = pkg.lib()
    N, K = w.rows, w.cols
    S = S or L.qb_ksplit_policy(N, K)
    rng = np.random.default_rng(5)
    q, d = pkg.binding.quantize_act(ctx, rng.standard_normal((M, K)).astype(np.float32))
    part = ctx.empty((S, M, N), np.float32)
    e0, e1 = ctx.event(), ctx.event()
    times = []
    for it in range(iters + 2):
        ctx.flush_l2()
        ctx.record(e0)
        pkg.binding.check(L.qb_q8_gemm_partials(ctx.h, w.h, q.ptr, d.ptr, M, part.ptr, S, impl))
        ctx.record(e1)
        ctx.sync()
        if it >= 2:
            times.append(ctx.elapsed_ms(e0, e1))
    out = part.download()
    q.free(); d.free(); part.free()
    return float(np.median(times)) * 1e3, N * K / 32 * 34 + M * K * 1.125 + S * M * N * 4, out, S


def sub_records(pkg, ctx, model, cfg):
    sub = {}
    rs = np.random.RandomState((pkg.configs.PROMPT_SEED + 4) & 0x7FFFFFFF)
    try:
        sub["config3"] = spec_record(pkg, ctx, model, cfg, seeded_prompts(pkg, cfg, pkg.configs.PROMPT_SEED + 5, [32768]), 20, 2,
                                     "configuration 3: prompt 32768 in paged KV (page 16, fp16), k=3, batch 1")
    except Exception as e:      # a sub-record must not take the headline down
        sub["config3"] = {"error": str(e)}
    try:
        lens = [int(v) for v in rs.randint(512, 8192 + 1, 32)]
        sub["config4"] = spec_record(pkg, ctx, model, cfg, seeded_prompts(pkg, cfg, pkg.configs.PROMPT_SEED + 6, lens), 20, 2,
                                     "configuration 4: 32 concurrent requests, prompts uniform 512-8192, k=3, 128 verify rows per step")
    except Exception as e:
        sub["config4"] = {"error": str(e)}
    try:
        peak, _ = peaks()
        rows = []
        for N, K in ((17408, 5120), (5120, 17408)):
            w = pkg.Weight.synth(ctx, 0x5EED, 77, N, K, 0.02)
            for M in (4, 16, 64, 128, 512):
                us, nbytes, _, S = gemm_time(pkg, ctx, w, M, 2, 5)
                rows.append({"N": N, "K": K, "M": M, "ksplit": S, "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1),
                             "frac_hbm": round(nbytes / us / 1e3 / peak, 3), "TOPs": round(2.0 * M * N * K / us / 1e6, 2),
                             "frac_int8_peak": round(2.0 * M * N * K / us / 1e6 / INT8_PEAK_TOPS, 4)})
            w.free()
        sub["config5"] = {"workload": "configuration 5: isolated verify GEMM, tcgen05 kernel, cold L2 before every launch, CUDA events (launch overhead included)",
                          "int8_peak_TOPs": INT8_PEAK_TOPS, "rows": rows}
    except Exception as e:
        sub["config5"] = {"error": str(e)}
    return sub


def tp_ffn_record(pkg, ctx, dist, rank, world, local, Ms=(4, 16, 64, 128, 512), iters=6):
    """The FFN pair of the 27B shape with the FFN dimension split over the ranks of the launch: all-reduce fused into the
    down GEMM's epilogue (plain peer stores) against the same GEMMs followed by an NCCL all-reduce; max over ranks of the
    CUDA-event time, cold L2; the fused result must be bit-identical on every rank."""
    import torch
    H, F = 5120, 17408
    try:
        f = F // world
        w_gu = pkg.Weight.synth(ctx, 0x5EED, 500 + rank, 2 * f, H, 0.02)
        w_dn = pkg.Weight.synth(ctx, 0x5EED, 600 + rank, H, f, 0.02)
        group, area, opened = pkg.tp.ipc_group(ctx, dist, max(Ms), H, f, H)
        solo, solo_area = pkg.tp.local_groups(ctx, 1, max(Ms), H, f, H)
        ext = torch.cuda.ExternalStream(int(pkg.lib().qb_stream(ctx.h)))

        class Raw:                                  # a device buffer of the library as a torch tensor (no copy)
            def __init__(self, arr):
                self.__cuda_array_interface__ = {"shape": arr.shape, "typestr": "<f4", "data": (int(arr.ptr.value), False), "version": 2}

        def tmax(v):
            t = torch.tensor([v], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t[0])

        e0, e1 = ctx.event(), ctx.event()
        rng = np.random.default_rng(5)
        rows = []
        for M in Ms:
            x = ctx.array(rng.standard_normal((M, H)).astype(np.float32))
            y, yb = ctx.empty((M, H), np.float32), ctx.empty((M, H), np.float32)
            yt = torch.as_tensor(Raw(yb), device="cuda:%d" % local)
            fused, unfused = [], []
            for it in range(iters + 2):
                ctx.flush_l2(); ctx.sync(); dist.barrier()
                ctx.record(e0); group.ffn(w_gu, w_dn, x, M, y); ctx.record(e1); ctx.sync()
                if it >= 2:
                    fused.append(ctx.elapsed_ms(e0, e1))
            with torch.cuda.stream(ext):
                for it in range(iters + 2):
                    ctx.flush_l2(); ctx.sync(); dist.barrier()
                    ctx.record(e0); solo[0].ffn(w_gu, w_dn, x, M, yb); dist.all_reduce(yt); ctx.record(e1); ctx.sync()
                    torch.cuda.synchronize()
                    if it >= 2:
                        unfused.append(ctx.elapsed_ms(e0, e1))
            # every rank ends with the same bits: compare a checksum of the fused result across ranks
            got = y.download()
            cs = torch.tensor([float(np.frombuffer(got.tobytes(), np.uint32).astype(np.uint64).sum() % (1 << 52))], dtype=torch.float64, device="cuda")
            lo, hi = cs.clone(), cs.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            close = bool(np.allclose(got, yb.download(), rtol=2e-3, atol=2e-3))
            rows.append({"M": M, "fused_us": round(tmax(float(np.median(fused)) * 1e3), 2),
                         "gemms_plus_nccl_allreduce_us": round(tmax(float(np.median(unfused)) * 1e3), 2),
                         "ranks_bit_identical": bool(float(lo[0]) == float(hi[0])), "matches_unfused": close})
            for a in (x, y, yb):
                a.free()
        ctx.sync(); dist.barrier()
        group.close(); solo[0].close()
        pkg.tp.ipc_release(ctx, opened)
        w_gu.free(); w_dn.free()
        dist.barrier()
        return {"workload": "tensor-parallel FFN pair 5120 -> 17408 -> 5120 split over %d GPUs, one process per GPU, cold L2" % world,
                "world": world, "weight_MB_per_rank": round((2 * f * H + H * f) / 32 * 34 / 1e6, 1), "rows": rows}
    except Exception as e:
        return {"error": str(e)}


def tp_step_record(pkg, ctx, dist, rank, world, cfg, prompt, steps=20, warmup=2):
    """The latency configuration: ONE request served by all ranks of the launch, the FFN pairs of every layer sharded
    over them (all-reduce fused into the down GEMM, plain peer stores); attention, DeltaNet and the LM head replicated.
    Greedy continuation and the speculative run at the same rank count; max over ranks of the device time."""
    import torch
    try:
        model = pkg.Model.synth_tp(ctx, cfg, pkg.configs.MODEL_SEED, rank, world)
        f = cfg.n_ff // world
        sched = accept_schedule(warmup + steps + 1, warmup)
        n_tok = int((sched + 1).sum()) + K_DRAFT + 4
        max_ctx = len(prompt) + max(n_tok, (warmup + steps + 3) * (K_DRAFT + 1)) + 16
        b = pkg.Batch(model, 1, max_ctx, K_DRAFT)
        group, area, opened = pkg.tp.ipc_group(ctx, dist, b.max_rows, cfg.n_embd, f, cfg.n_embd)
        b.set_tp(group)
        e0, e1 = ctx.event(), ctx.event()
        ctx.sync(); dist.barrier()
        b.prefill(0, prompt)
        first = b.read_output()[0][0]
        snap = b.snapshot()
        greedy = [first]
        ctx.sync(); dist.barrier(); ctx.record(e0)
        for _ in range(n_tok - 1):
            b.greedy_step()
            greedy += b.read_output()[0]
        ctx.record(e1); ctx.sync()
        greedy_ms = ctx.elapsed_ms(e0, e1) / (n_tok - 1)
        b.restore(snap)
        stride = max_ctx + 8
        stream = np.zeros(stride, np.int32)
        stream[:len(prompt)] = prompt
        stream[len(prompt):len(prompt) + len(greedy)] = greedy
        forced, _ = forced_table(stream, len(prompt), sched, cfg.vocab_size)
        sdev = ctx.array(forced.reshape(1, -1))

        def step():
            b.mtp_draft(); b.mtp_force_drafts(sdev, stride); b.mtp_verify(); b.mtp_accept_commit()

        for _ in range(warmup):
            step(); b.read_output()
        p0 = b.position(0)
        ctx.sync(); dist.barrier(); ctx.record(e0)
        for _ in range(steps):
            step()
        ctx.record(e1); ctx.sync()
        ms = ctx.elapsed_ms(e0, e1)
        b.read_output()
        p1 = b.position(0)
        # phase split on a few more steps: events at the boundaries only
        ev = [ctx.event() for _ in range(4)]
        ctx.sync(); dist.barrier()
        ctx.record(ev[0]); b.mtp_draft(); b.mtp_force_drafts(sdev, stride)
        ctx.record(ev[1]); b.mtp_verify()
        ctx.record(ev[2]); b.mtp_accept_commit()
        ctx.record(ev[3]); ctx.sync()
        out = b.read_output()[0]
        p2 = b.position(0)
        lossless = (p1 - p0) == int((sched[warmup:warmup + steps] + 1).sum()) and out == list(stream[p2 - len(out) + 1:p2 + 1])
        t = torch.tensor([ms, greedy_ms, ctx.elapsed_ms(ev[0], ev[1]), ctx.elapsed_ms(ev[1], ev[2]), ctx.elapsed_ms(ev[2], ev[3]), 0.0 if lossless else 1.0],
                         dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ctx.sync(); dist.barrier()
        b.free_snapshot(snap); b.close(); group.close(); pkg.tp.ipc_release(ctx, opened); model.close()
        dist.barrier()
        ms, greedy_ms = float(t[0]), float(t[1])
        return {"workload": "configuration 2 as ONE request over %d GPUs: FFN pairs tensor-sharded, all-reduce fused into the down GEMM" % world,
                "world": world, "steps": steps, "ms_per_step": ms / steps, "tok_per_s": (p1 - p0) / (ms * 1e-3), "greedy_ms_per_token": greedy_ms,
                "draft_us": float(t[2]) * 1e3, "verify_us": float(t[3]) * 1e3, "accept_commit_us": float(t[4]) * 1e3,
                "lossless_vs_greedy_at_same_rank_count": bool(float(t[5]) == 0.0)}
    except Exception as e:
        return {"error": str(e)}


# ---- profiling workloads --------------------------------------------------------------------------------
def workload_gemm(args):
    if args.tp:
        rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        pkg = entry.load_package()
        ctx = pkg.Context(local)
        rec = tp_ffn_record(pkg, ctx, dist, rank, world, local, [int(v) for v in args.m.split(",") if int(v) > 1] or [4], args.iters)
        if rank == 0:
            print(json.dumps(rec), flush=True)
        ctx.close()
        dist.destroy_process_group()
        return
    pkg = entry.load_package()
    ctx = pkg.Context(0)
    peak, _ = peaks()
    for shape in args.shapes.split(","):
        N, K = [int(v) for v in shape.split("x")]
        w = pkg.Weight.synth(ctx, 0x5EED, 77, N, K, 0.02)
        for M in [int(v) for v in args.m.split(",")]:
            ref = None
            for impl in [int(v) for v in args.impls.split(",")]:
                if impl == 1 and M > 64:
                    continue          # the CUDA-core kernel is the small-batch kernel
                us, nbytes, out, S = gemm_time(pkg, ctx, w, M, impl, args.iters)
                same = None if ref is None else bool(np.array_equal(ref, out))
                ref = out if ref is None else ref
                print(json.dumps({"N": N, "K": K, "M": M, "ksplit": S, "impl": impl, "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1),
                                  "frac_hbm": round(nbytes / us / 1e3 / peak, 3), "TOPs": round(2.0 * M * N * K / us / 1e6, 2),
                                  "frac_int8_peak": round(2.0 * M * N * K / us / 1e6 / INT8_PEAK_TOPS, 4), "bit_identical_to_first_impl": same}), flush=True)
        w.free()
    ctx.close()


def workload_attn(args):
    """Paged gated attention alone (27B-class heads: 24 q / 4 kv x 256, page 16, 4 verify rows): split + merge, cold L2."""
    pkg = entry.load_package()
    ctx = pkg.Context(0)
    L = pkg.lib()
    peak, _ = peaks()
    n_heads, n_kv, hd, page, R = 24, 4, 256, 16, K_DRAFT + 1
    for ctxlen in [int(v) for v in args.ctx.split(",")]:
        max_pos = ctxlen + R
        pps = (max_pos + page) // page + 1
        pt = np.arange(pps, dtype=np.int32).reshape(1, pps)
        kvd = n_kv * hd
        rng = np.random.default_rng(1)
        kc = (rng.standard_normal((pps * page, kvd)) * 0.5).astype(np.float16)
        vc = (rng.standard_normal((pps * page, kvd)) * 0.5).astype(np.float16)
        stride = n_heads * 2 * hd + 2 * kvd
        qkv = rng.standard_normal((R, stride)).astype(np.float32)
        d_qkv, d_kc, d_vc, d_pt = ctx.array(qkv), ctx.array(kc.view(np.uint16)), ctx.array(vc.view(np.uint16)), ctx.array(pt)
        d_pos = ctx.array(np.array([ctxlen], np.int32))
        out = ctx.empty((R, n_heads * hd), np.float32)
        e0, e1 = ctx.event(), ctx.event()
        ts = []
        for it in range(args.iters):
            ctx.flush_l2()
            ctx.record(e0)
            pkg.binding.check(L.qb_attention_paged_gated(ctx.h, d_qkv.ptr, R, stride, n_heads, n_kv, hd, d_pos.ptr, 1,
                                                        d_pt.ptr, pps, page, d_kc.ptr, d_vc.ptr, max_pos, out.ptr))
            ctx.record(e1)
            ctx.sync()
            ts.append(ctx.elapsed_ms(e0, e1) * 1e3)
        kvbytes = ctxlen * kvd * 2 * 2
        us = float(np.median(ts[2:]))
        print(json.dumps({"ctx": ctxlen, "rows": R, "split_plus_merge_us": round(us, 1), "kv_MB": round(kvbytes / 1e6, 1),
                          "GBps": round(kvbytes / us / 1e3), "frac_hbm": round(kvbytes / us / 1e3 / peak, 3)}), flush=True)
        ctx.release_arrays()
    ctx.close()


def workload_timeline(args):
    """Per-CTA global-timer stamps inside every tensor-core GEMM of one step (no events in the stream)."""
    pkg = entry.load_package()
    ctx = pkg.Context(0)
    cfg = pkg.configs.qwen27b(args.layers)
    model = pkg.Model(ctx, cfg, pkg.configs.MODEL_SEED)
    prompt = np.random.RandomState(1).randint(0, cfg.vocab_size, args.prompt).astype(np.int32)
    b = pkg.Batch(model, 1, args.prompt + 256, K_DRAFT)
    b.prefill(0, prompt)
    b.read_output()
    for _ in range(3):
        b.mtp_step()
        b.read_output()
    ctx.timeline_enable(512)
    b.mtp_step()
    b.read_output()
    st, grids, nbytes = ctx.timeline_read(512)
    ctx.timeline_enable(0)
    print("idx  CTAs     MB | entry_first  dep_ok  exit_first  exit_last (us from first launch) |  dur_us  GB/s | gap_before_us")
    t00, prev_exit, busy, gaps = None, None, 0.0, 0.0
    for i in range(len(grids)):
        t = st[i, :int(grids[i])].astype(np.int64)
        e0, w0, x0, x1 = int(t[:, 0].min()), int(t[:, 1].min()), int(t[:, 2].min()), int(t[:, 2].max())
        t00 = e0 if t00 is None else t00
        dur = (x1 - w0) * 1e-3
        gap = (w0 - prev_exit) * 1e-3 if prev_exit is not None else 0.0
        busy += dur
        gaps += max(gap, 0.0)
        if i < 80:
            print("%3d  %4d  %5.1f | %9.1f %9.1f %9.1f %9.1f | %7.1f %5.0f | %7.1f" % (
                i, grids[i], nbytes[i] / 1e6, (e0 - t00) * 1e-3, (w0 - t00) * 1e-3, (x0 - t00) * 1e-3, (x1 - t00) * 1e-3, dur,
                nbytes[i] / dur / 1e3, gap))
        prev_exit = x1
    print("launches %d, bytes %.2f GB, inside the GEMMs %.1f us (%.0f GB/s), between them %.1f us" % (
        len(grids), nbytes.sum() / 1e9, busy, nbytes.sum() / busy / 1e3, gaps))
    b.close(); model.close(); ctx.close()


def workload_serve(args):
    """The continuous-batching loops at the 27B shape: requests arriving every 1-2 steps into --slots slots, wall clock
    with the prefills inside (natural acceptance of the random weights, about 0)."""
    pkg = entry.load_package()
    ctx = pkg.Context(0)
    cfg = pkg.configs.qwen27b(args.layers)
    model = pkg.Model(ctx, cfg, pkg.configs.MODEL_SEED)
    rs = np.random.RandomState(9)
    # the third run: one K/V page pool for all slots, 60 % of what private pages would hold; admission reserves pages
    for loop, pooled in (("run", False), ("run_compact", False), ("run_compact", True)):
        reqs = [pkg.serve.Request(i, rs.randint(0, cfg.vocab_size, int(rs.randint(256, 513))).tolist(), int(rs.randint(48, 97)), arrival_step=2 * i)
                for i in range(args.requests)]
        pages_private = args.slots * ((1024 + K_DRAFT + 1 + 15) // 16)
        b = pkg.Batch(model, args.slots, 1024, K_DRAFT, pool_pages=int(0.6 * pages_private) if pooled else 0)
        ctx.sync()
        t0 = time.perf_counter()
        done = getattr(pkg.serve, loop)(b, reqs)
        ctx.sync()
        dt = time.perf_counter() - t0
        print(json.dumps({"loop": loop, "kv_pages": int(0.6 * pages_private) if pooled else pages_private, "pooled": pooled, "slots": args.slots,
                          "requests": len(done), "emitted": sum(len(r.tokens) for r in done),
                          "wall_s": round(dt, 2), "tok_per_s": round(sum(len(r.tokens) for r in done) / dt, 1)}), flush=True)
        b.close()
    model.close(); ctx.close()


def workload_tokenizer(args):
    """Host only.  A seeded chat-shaped text (about 2 MB) through the product's tokenizer and, as the CPU baseline, through
    the reference's own (oracle/_ref/libqw3ref_tokenizer.so, where it has been built) on the same seeded vocabulary."""
    import ctypes
    import tempfile
    os.environ["LC_ALL"] = "C"
    pkg = entry.load_package()
    tokens, merges = pkg.synth_vocab.synth_bpe_vocab(0x70C)
    bos = tokens.index(b"<|endoftext|>")
    words = pkg.synth_vocab.synth_corpus(11, 40000)
    rs = np.random.RandomState(12)
    msgs, at = [], 0
    while at < len(words):
        n = int(rs.randint(20, 400))
        body = " ".join(words[at:at + n])
        msgs.append("<|im_start|>%s\n%s<|im_end|>\n" % ("user" if len(msgs) % 2 == 0 else "assistant", body))
        at += n
    text = ("".join(msgs) * 8).encode("utf-8")
    tok = pkg.binding.Tokenizer.from_tables(tokens, merges, bos, bos, False)

    def best(fn, reps=3):
        out, t = None, float("inf")
        for _ in range(reps):
            t0 = time.perf_counter()
            out = fn()
            t = min(t, time.perf_counter() - t0)
        return out, t

    ids, t_enc = best(lambda: tok.encode(text))
    dec, t_dec = best(lambda: tok.decode(ids))
    rec = {"workload": "tokenizer: seeded chat-shaped text, %d-entry byte-level BPE vocabulary, one host thread" % len(tokens), "text_MB": round(len(text) / 1e6, 2),
           "tokens": int(ids.size), "encode_MB_per_s": round(len(text) / 1e6 / t_enc, 2), "encode_tok_per_s": round(ids.size / t_enc),
           "decode_MB_per_s": round(len(text) / 1e6 / t_dec, 1), "round_trip_exact": dec == text, "cpu_baseline": None}
    ref = os.path.join(ROOT, "oracle", "_ref", "libqw3ref_tokenizer.so")
    if os.path.exists(ref):
        # the CPU baseline leg: the reference's tokenizer reads the same tables from a file (writer: test infrastructure)
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import gguf_synth as G
        L = ctypes.CDLL(ref)
        L.rt_open.restype = ctypes.c_void_p
        L.rt_open.argtypes = [ctypes.c_char_p]
        L.rt_encode.restype = ctypes.c_int64
        L.rt_encode.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64]
        with tempfile.TemporaryDirectory() as d:
            h = L.rt_open(G.write_tokenizer_gguf(os.path.join(d, "tok.gguf"), tokens, merges, bos, bos, False).encode())
            out = np.zeros(len(text) + 8, np.int32)
            n, t_ref = best(lambda: L.rt_encode(h, text, len(text), 0, out.ctypes.data, out.size), reps=2)
        rec["cpu_baseline"] = {"kind": "reference", "what": "qw3::QwenTokenizer::encode on the same text and vocabulary (it uses up to all host threads above 512 KiB)",
                               "encode_MB_per_s": round(len(text) / 1e6 / t_ref, 2), "same_ids": bool(n == ids.size and np.array_equal(out[:n], ids))}
    print(json.dumps(rec), flush=True)
    tok.close()


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload != "step":
        return {"gemm": workload_gemm, "attn": workload_attn, "timeline": workload_timeline, "serve": workload_serve,
                "tokenizer": workload_tokenizer}[args.workload](args)
    if args.impl == "reference":
        run_reference(args, rank)
        return
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")      # plumbing only (barriers, sums of the timings)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    try:
        run_ours(args, rank, world, local_rank, dist)
    finally:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
