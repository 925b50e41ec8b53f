"""Throughput of the continuous-batching loop (serve.py) on one GPU: seeded synthetic requests of the 27B shape admitted
into `--slots` sequence slots as they arrive; wall clock over the whole run (prefills included), one JSON line.

    python kvmem-qw3_b200/serve_bench.py [--slots 8] [--requests 24] [--prompt 512] [--new 96] [--gap 2] [--chunk 0] [--fixed-slots] [--tiny]
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as entry  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--slots", type=int, default=8)
    ap.add_argument("--requests", type=int, default=24)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=96)
    ap.add_argument("--gap", type=int, default=2, help="a new request arrives every GAP decode steps")
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--fixed-slots", action="store_true", help="the loop that steps every slot (serve.run) instead of the compacting one")
    ap.add_argument("--chunk", type=int, default=0, help="compacting loop: prompt tokens ingested per iteration (0 = whole prompt)")
    args = ap.parse_args()
    pkg = entry.load_package()
    ctx = pkg.Context(0)
    cfg = pkg.configs.tiny() if args.tiny else pkg.configs.qwen27b()
    model = pkg.Model(ctx, cfg, pkg.configs.MODEL_SEED)
    import numpy as np
    rng = np.random.default_rng(11)
    reqs = []
    for i in range(args.requests):
        n = int(rng.integers(args.prompt // 2, args.prompt + 1))
        new = int(rng.integers(args.new // 2, args.new + 1))
        reqs.append(pkg.serve.Request(i, rng.integers(0, cfg.vocab_size, n).tolist(), new, arrival_step=i * args.gap))
    batch = pkg.Batch(model, args.slots, args.prompt + args.new + 4 * (args.k + 1) + 64, args.k)
    ctx.sync()
    t0 = time.perf_counter()
    if args.fixed_slots:
        done = pkg.serve.run(batch, reqs, speculative=args.k > 0)
    else:
        done = pkg.serve.run_compact(batch, reqs, speculative=args.k > 0, prefill_chunk=args.chunk)
    ctx.sync()
    wall = time.perf_counter() - t0
    st = batch.stats()
    emitted = sum(len(r.tokens) for r in done)
    prompt_tokens = sum(len(r.prompt) for r in done)
    print(json.dumps({"loop": "fixed slots" if args.fixed_slots else "compacting, chunk %d" % args.chunk, "slots": args.slots, "requests": len(done), "prompt_tokens": prompt_tokens, "emitted_tokens": emitted,
                      "wall_s": round(wall, 3), "emitted_tok_per_s": round(emitted / wall, 1),
                      "sequence_steps": st["steps"], "accepted_drafts": st["accepted"], "last_finish_step": max(r.finished_step for r in done),
                      "mean_queue_steps": round(float(np.mean([r.admitted_step - r.arrival_step for r in done])), 2),
                      "model": "tiny" if args.tiny else "27B-class qwen35 shape, Q8_0, k=%d" % args.k}))
    batch.close()
    model.close()
    ctx.close()


if __name__ == "__main__":
    main()
