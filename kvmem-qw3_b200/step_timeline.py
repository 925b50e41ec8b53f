"""Device timeline of one MTP step (27B-class shape, k=3, batch 1): where the stream's time goes.

Every tensor-core GEMM launch of the step records, per CTA, global-timer stamps at entry, when its dependency
on the preceding kernel is satisfied, and at exit (qb_debug_timeline_*).  No events are put in the stream, so the
programmatic-dependent-launch overlap of the real step is intact.  Prints one line per GEMM launch
(duration = earliest "dependency satisfied" to last exit; gap = previous GEMM's last exit to this launch's
"dependency satisfied", i.e. everything that ran in between) and the totals.

    python kvmem-qw3_b200/step_timeline.py [--layers 64] [--prompt 2048] [--rows 80]
"""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as entry  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=80, help="launches to print in full")
    args = ap.parse_args()
    pkg = entry.load_package()
    ctx = pkg.Context(0)
    cfg = pkg.configs.qwen27b(args.layers)
    model = pkg.Model(ctx, cfg, pkg.configs.MODEL_SEED)
    prompt = np.random.RandomState(1).randint(0, cfg.vocab_size, args.prompt).astype(np.int32)
    b = pkg.Batch(model, 1, args.prompt + 256, 3)
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
        if i < args.rows:
            print("%3d  %4d  %5.1f | %9.1f %9.1f %9.1f %9.1f | %7.1f %5.0f | %7.1f" % (
                i, grids[i], nbytes[i] / 1e6, (e0 - t00) * 1e-3, (w0 - t00) * 1e-3, (x0 - t00) * 1e-3, (x1 - t00) * 1e-3, dur,
                nbytes[i] / dur / 1e3, gap))
        prev_exit = x1
    print("launches %d, bytes %.2f GB, inside the GEMMs %.1f us (%.0f GB/s), between them %.1f us" % (
        len(grids), nbytes.sum() / 1e9, busy, nbytes.sum() / busy / 1e3, gaps))
    b.close(); model.close(); ctx.close()


if __name__ == "__main__":
    main()
