"""Benchmark of the MTP speculative-decode step (27B-class qwen35 shape, Q8_0, k=3).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one speculative step of one request: 3 chained MTP-head drafts, the 4-row target
verification forward over all 64 layers, greedy acceptance and commit.  The workload is benchmark
configuration 2 (batch 1, prompt 2048 seeded uniform token ids in paged fp16 KV, page 16) in its
forced-acceptance form: the verified drafts equal the true greedy continuation at a seeded 70% rate,
because seeded random weights give the MTP head no natural acceptance.  The MTP-head drafts are still
computed (and timed) every step.  Prints ONE JSON line on rank 0.

--gpus N runs N independent replicas (one process per GPU, launched by torch.distributed.run); the
path has no exchange step, so there is no data-path collective: only the barrier and the max-over-
ranks of the device time go through torch.distributed.

--impl reference times the CPU restatement of the reference's arithmetic (oracle/, the reference has
no CPU implementation of this path and its CUDA build is not a CPU baseline) on the host cores.
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
EXPECTED_EMITTED = 1 + ACCEPT_RATE + ACCEPT_RATE ** 2 + ACCEPT_RATE ** 3   # tokens per step at 70%


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=64, help="target layers (64 = the 27B-class shape)")
    ap.add_argument("--prompt", type=int, default=PROMPT_LEN)
    ap.add_argument("--seqs", type=int, default=1, help="concurrent requests per GPU (32 = the continuous-batching configuration)")
    ap.add_argument("--prompt-min", type=int, default=512, help="with --seqs > 1 prompt lengths are uniform in [prompt-min, prompt]")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-greedy", action="store_true", help="profiling aid: no greedy reference run (forced drafts then never match)")
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

    def stop(self, first=0):
        """Summary of the samples from index `first` on; of all samples (taken under the warm-up load) when the
        timed region was too short to catch one."""
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
        window = self.lines[first:] if len(self.lines) > first else self.lines
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


CPU_SAMPLE_TEXT = ("one step per sample on a 4-layer slice (3 DeltaNet + 1 attention) of the 27B shape with the full LM head "
                   "and MTP layer, ctx 8: 3 MTP drafts + 4-row verify; layer time scaled x16 to 64 layers")


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
    value = EXPECTED_EMITTED / sec
    line = {
        "impl": "reference", "metric": "accepted_tok_per_s", "value": value, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": O.num_threads(), "kind": "port", "sample": CPU_SAMPLE_TEXT},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(args):
    return {"workload": "configuration 2: 27B-class qwen35 shape (%d layers, hidden 5120, 24q/4kv x 256, DeltaNet 16k/48v x 128, "
                        "FFN 17408, vocab 151936), Q8_0, MTP k=3, batch %d, prompt %d, forced drafts = greedy continuation at a "
                        "seeded 70%% rate" % (args.layers, args.seqs, args.prompt),
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


def run_ours(args, rank, world, local_rank, dist):
    pkg = entry.load_package()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        all_host_threads()
    O = entry.load_oracle() if (rank == 0 and world == 1 and not args.no_cpu_baseline) else None
    ctx = pkg.Context(local_rank)
    cfg = pkg.configs.qwen27b(args.layers)
    K, W, k, ns = args.steps, args.warmup, K_DRAFT, args.seqs
    prof_steps = min(K, 8)
    total_steps = 2 * W + 2 * K + prof_steps + 6
    n_greedy = 4 * total_steps + 8
    model = pkg.Model(ctx, cfg, pkg.configs.MODEL_SEED)
    # seeded prompts: uniform token ids; one request of --prompt tokens, or --seqs requests with lengths
    # uniform in [--prompt-min, --prompt] (the continuous-batching configuration)
    rs = np.random.RandomState((pkg.configs.PROMPT_SEED + 2 + rank) & 0x7FFFFFFF)
    plen = [args.prompt] if ns == 1 else [int(v) for v in rs.randint(args.prompt_min, args.prompt + 1, ns)]
    prompts = [rs.randint(0, cfg.vocab_size, n).astype(np.int32) for n in plen]
    max_ctx = max(plen) + n_greedy + 16
    stride = max_ctx + 8

    # 1. the non-speculative greedy continuation (also the losslessness reference of this run)
    ev = [ctx.event() for _ in range(8)]
    if args.skip_greedy:
        greedy, greedy_ms = [[0] * n_greedy for _ in range(ns)], float("nan")
    else:
        g = pkg.Batch(model, ns, max_ctx, 0)
        for s_ in range(ns):
            g.prefill(s_, prompts[s_])
        greedy = [list(t) for t in g.read_output()]
        ctx.sync()
        ctx.record(ev[0])
        for _ in range(n_greedy - 1):
            g.greedy_step()
            for s_, t in enumerate(g.read_output()):
                greedy[s_] += t
        ctx.record(ev[1])
        ctx.sync()
        greedy_ms = ctx.elapsed_ms(ev[0], ev[1]) / (n_greedy - 1)
        g.close()
    stream = np.zeros((ns, stride), np.int32)          # stream[s][p] = token at absolute position p
    for s_ in range(ns):
        stream[s_, :plen[s_]] = prompts[s_]
        stream[s_, plen[s_]:plen[s_] + len(greedy[s_])] = greedy[s_]
    # the forced guess for every position: the true continuation at a seeded 70 % rate, else a different token
    frs = np.random.RandomState(FORCE_SEED + rank)
    forced = np.where(frs.rand(ns, stride) < ACCEPT_RATE, stream, (stream + 1) % cfg.vocab_size).astype(np.int32)
    sdev = ctx.array(forced)

    # the clock sampler runs from the prompt ingestion on (nvidia-smi needs a moment to start); the samples of
    # the timed region are cut out below
    sampler = ClockSampler(local_rank)
    sampler.start()
    b = pkg.Batch(model, ns, max_ctx, k)
    for s_ in range(ns):
        b.prefill(s_, prompts[s_])
    b.read_output()

    def device_step():
        b.mtp_draft()
        b.mtp_force_drafts(sdev, stride)
        b.mtp_verify()
        b.mtp_accept_commit()

    # 2. device-resident timing: K steps back to back, no host read-back inside
    for _ in range(W):
        device_step()
        b.read_output()
    if dist is not None:
        dist.barrier()
    ctx.sync()
    s0, l0 = b.stats(), ctx.launches
    first_sample = sampler.mark()
    ctx.record(ev[0])
    for _ in range(K):
        device_step()
    ctx.record(ev[1])
    ctx.sync()
    clocks = sampler.stop(first_sample)
    dev_ms = ctx.elapsed_ms(ev[0], ev[1])
    s1, l1 = b.stats(), ctx.launches
    dev_emitted = s1["emitted"] - s0["emitted"]
    dev_accepted = s1["accepted"] - s0["accepted"]
    b.read_output()

    # 3. phase split + per-launch GEMM timing (separate pass, event records perturb the stream slightly)
    ctx.prof_enable(True)
    ph = [0.0, 0.0, 0.0]
    for _ in range(prof_steps):
        ctx.record(ev[2]); b.mtp_draft(); b.mtp_force_drafts(sdev, stride)
        ctx.record(ev[3]); b.mtp_verify()
        ctx.record(ev[4]); b.mtp_accept_commit()
        ctx.record(ev[5]); ctx.sync()
        for i in range(3):
            ph[i] += ctx.elapsed_ms(ev[2 + i], ev[3 + i]) / prof_steps
        b.read_output()
    prof = ctx.prof_summary()
    ctx.prof_enable(False)
    # one traced step: per-kernel time shares measured live (event after every launch)
    ctx.trace_enable(True)
    device_step()
    trace = ctx.trace_summary()
    ctx.trace_enable(False)
    b.read_output()
    # one step with device-side stamps inside the tensor-core GEMM (no events in the stream: the in-stream truth)
    ctx.timeline_enable(512)
    device_step()
    tl = ctx.timeline_gemm_summary(*ctx.timeline_read(512))
    ctx.timeline_enable(0)
    b.read_output()

    # 4. end to end through the host-driven API, on a fresh batch that replays the same trajectory (same
    #    prompt, same warm-up, same forced guesses): drafts come from pinned host memory every step and the
    #    step record goes back to the host every step
    b.close()
    b = pkg.Batch(model, ns, max_ctx, k)
    for s_ in range(ns):
        b.prefill(s_, prompts[s_])
    b.read_output()
    pos = [b.position(s_) for s_ in range(ns)]
    pinned = ctx.pinned((ns, k), np.int32)

    def host_step():
        b.mtp_draft()
        for s_ in range(ns):
            pinned[s_, :] = forced[s_, pos[s_] + 1:pos[s_] + 1 + k]
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
    ctx.record(ev[6])
    t0 = time.perf_counter()
    for _ in range(K):
        for s_, t in enumerate(host_step()):
            e2e_tokens[s_] += t
            pos[s_] += len(t)
    ctx.record(ev[7])
    ctx.sync()
    e2e_wall = time.perf_counter() - t0
    e2e_ms = max(ctx.elapsed_ms(ev[6], ev[7]), e2e_wall * 1e3)
    lossless = all(e2e_tokens[s_] == list(stream[s_, start_pos[s_] + 1:pos[s_] + 1]) for s_ in range(ns)) and not args.skip_greedy
    n_e2e = sum(len(t) for t in e2e_tokens)

    # 5. aggregate over replicas: max time, summed tokens
    tmax, tsum = pkg.replicas.aggregate(dist, [dev_ms, e2e_ms], [float(dev_emitted), float(n_e2e), float(l1 - l0)])
    agg = np.concatenate([tmax, tsum])
    if rank != 0:
        b.close(); model.close(); ctx.close()
        return
    peak, peak_src = peaks()
    achieved = prof["bytes"] / (prof["ms"] * 1e-3) / 1e9 if prof["ms"] > 0 else 0.0
    step_bytes = model.weight_bytes - cfg.vocab_size * cfg.n_embd / 32 * 34      # token_embd is gathered, not streamed
    line = {
        "metric": "accepted_tok_per_s", "value": agg[2] / (agg[0] * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": agg[0] / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": workload_config(args), "clocks": clocks,
        "e2e": {"value": agg[3] / (agg[1] * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": ns * k * 4, "d2h_bytes_per_step": ns * (k + 3) * 4,
                "ms_per_step": agg[1] / K, "lossless_vs_greedy": bool(lossless)},
        "gpu_launches": int(agg[4]), "gpu_launches_before_timed_region": int(l0),
        "roofline": {"bound": "hbm", "kernel": "gemm_tc_kernel + gemm_dp4a_kernel (all Q8_0 projections of the step)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                     # DRAM bytes per launch: the ncu capture of this kernel on a 94.70 MB weight read 94.79 MB
                     # (ratio 1.001, the weight is streamed once); scaled to this run's average launch
                     "traffic": NCU_TRAFFIC_RATIO * prof["bytes"] / max(prof["launches"], 1),
                     "launches": prof["launches"], "avg_launch_us": prof["ms"] * 1e3 / max(prof["launches"], 1),
                     "bytes_per_launch_avg": prof["bytes"] / max(prof["launches"], 1),
                     # the same kernel timed by global-timer stamps inside it, with the dependent-launch overlap of
                     # the real stream intact (event pairs serialise the launches and add their own ~2 us)
                     "in_stream": {"launches": tl["launches"], "busy_us": tl["busy_us"], "gaps_between_us": tl["gap_us"],
                                   "achieved": tl["bytes"] / max(tl["busy_us"], 1e-9) / 1e3, "unit": "GB/s",
                                   "frac": tl["bytes"] / max(tl["busy_us"], 1e-9) / 1e3 / peak}},
        "step": {"verify_us": ph[1] * 1e3, "draft_us": ph[0] * 1e3, "accept_commit_us": ph[2] * 1e3,
                 "accepted_per_step": dev_accepted / K, "emitted_per_step": dev_emitted / K, "acceptance_rate": dev_accepted / (K * k * ns),
                 "greedy_ms_per_token": greedy_ms, "greedy_tok_per_s": 1e3 / greedy_ms,
                 "weight_bytes_per_step": step_bytes,
                 "step_hbm_frac": (step_bytes / 1e9) / ((agg[0] / K) * 1e-3) / peak if world == 1 else None},
    }
    ttot = sum(t for _, _, t in trace) or 1.0
    line["step"]["kernel_shares"] = {n: {"launches": c, "us": round(t, 1), "share": round(t / ttot, 4)} for n, c, t in trace}
    if O is not None:
        models, seqs = cpu_setup(O, pkg)
        cpu_step_sample(O, models, seqs)
        t = [cpu_step_sample(O, models, seqs) for _ in range(3)]
        sec = float(np.mean(t))
        line["cpu_baseline"] = {"value": EXPECTED_EMITTED / sec, "unit": "tok/s", "cores": O.num_threads(), "kind": "port",
                                "sample": CPU_SAMPLE_TEXT, "ms_per_step": sec * 1e3}
    print(json.dumps(line))
    b.close(); model.close(); ctx.close()


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
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
