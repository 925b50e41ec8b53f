"""Isolated verify-GEMM sweep (BASELINE configuration 5 on one GPU).

Q8_0 weights 5120x17408 and 17408x5120 (seeded), activations N(0,1) quantised per 32-block to int8,
M in {1, 4, 16, 64, 128, 512}; both kernels (1 = CUDA-core dp4a streaming, 2 = tcgen05 INT8).  Each
timed launch starts with a cold L2 (a 256 MB buffer is rewritten before it); times are CUDA events on
the launching stream.  Prints one JSON line per (shape, M, kernel).

    python kvmem-qw3_b200/gemm_sweep.py [--iters 10] [--shapes 17408x5120,5120x17408] [--m 1,4,16]
"""
import argparse
import ctypes as C
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as entry  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shapes", default="17408x5120,5120x17408,5120x6144,34816x5120,151936x5120")
    ap.add_argument("--m", default="1,4,16,64,128,512")
    ap.add_argument("--impls", default="1,2")
    ap.add_argument("--ksplit", type=int, default=0)
    ap.add_argument("--no-flush", action="store_true")
    args = ap.parse_args()
    pkg = entry.load_package()
    L = pkg.lib()
    ctx = pkg.Context(0)
    peak = 6548.5
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = float(json.load(open(p))["hbm_gbs"])
    rng = np.random.default_rng(5)
    e0, e1 = ctx.event(), ctx.event()
    for shape in args.shapes.split(","):
        N, K = [int(v) for v in shape.split("x")]
        w = pkg.Weight.synth(ctx, 0x5EED, 77, N, K, 0.02)
        S = args.ksplit or L.qb_ksplit_policy(N, K)
        for M in [int(v) for v in args.m.split(",")]:
            x = rng.standard_normal((M, K)).astype(np.float32)
            q, d = pkg.binding.quantize_act(ctx, x)
            part = ctx.empty((S, M, N), np.float32)
            ref = None
            for impl in [int(v) for v in args.impls.split(",")]:
                if impl == 1 and M > 64:
                    continue          # the CUDA-core kernel is the small-batch kernel
                times = []
                for it in range(args.iters + 2):
                    if not args.no_flush:
                        ctx.flush_l2()
                    ctx.record(e0)
                    pkg.binding.check(L.qb_q8_gemm_partials(ctx.h, w.h, q.ptr, d.ptr, M, part.ptr, S, impl))
                    ctx.record(e1)
                    ctx.sync()
                    if it >= 2:
                        times.append(ctx.elapsed_ms(e0, e1))
                out = part.download()
                same = None
                if ref is None:
                    ref = out
                else:
                    same = bool(np.array_equal(ref, out))
                us = float(np.median(times)) * 1e3
                nbytes = N * K / 32 * 34 + M * K * 1.125 + S * M * N * 4
                print(json.dumps({"N": N, "K": K, "M": M, "ksplit": S, "impl": impl, "us": round(us, 2),
                                  "GBps": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / peak, 3),
                                  "TOPs": round(2.0 * M * N * K / us / 1e6, 2), "bit_identical_to_first_impl": same}), flush=True)
            q.free(); d.free(); part.free()
        w.free()
    ctx.close()


if __name__ == "__main__":
    main()
