"""Isolated verify-GEMM sweep (benchmark configuration 5 on one GPU).

Q8_0 weights 5120x17408 and 17408x5120 (seeded), activations N(0,1) quantised per 32-block to int8,
M in {1, 4, 16, 64, 128, 512}; both kernels (1 = CUDA-core dp4a streaming, 2 = tcgen05 INT8).  Each
timed launch starts with a cold L2 (a 256 MB buffer is rewritten before it); times are CUDA events on
the launching stream.  Prints one JSON line per (shape, M, kernel).

    python kvmem-qw3_b200/gemm_sweep.py [--iters 10] [--shapes 17408x5120,5120x17408] [--m 1,4,16]

--tp times the tensor-parallel FFN pair (5120 -> 17408 gate/up, SwiGLU, 17408 -> 5120 down, all-reduce fused
into the down GEMM's epilogue) with the FFN dimension split over the ranks of the launch:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 --master-port 29700 \
        kvmem-qw3_b200/gemm_sweep.py --tp [--rows 4,16,64,128,512]

One JSON line per M on rank 0: the time is the max over ranks of the CUDA-event time of one FFN (cold L2).
With --nccl-baseline every M is also timed in the unfused form: the same two GEMMs on the rank's shard, its own
sum over the K segments, then torch.distributed.all_reduce (NCCL) of the [M, 5120] result on the same stream.
"""
import argparse
import ctypes as C
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as entry  # noqa: E402


def tp_sweep(args):
    """FFN pair of the 27B shape with the FFN dimension split over WORLD_SIZE GPUs (one process each)."""
    H, F = 5120, 17408
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    pkg = entry.load_package()
    ctx = pkg.Context(local)
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("gloo")      # plumbing only: handle exchange, barriers, max of the times
    Ms = [int(v) for v in args.m.split(",") if int(v) > 1] or [4]
    f = F // world
    w_gu = pkg.Weight.synth(ctx, 0x5EED, 500 + rank, 2 * f, H, 0.02)
    w_dn = pkg.Weight.synth(ctx, 0x5EED, 600 + rank, H, f, 0.02)
    if dist is not None:
        group, area, opened = pkg.tp.ipc_group(ctx, dist, max(Ms), H, f, H)
    else:
        groups, area = pkg.tp.local_groups(ctx, 1, max(Ms), H, f, H)
        group, opened = groups[0], []
    rng = np.random.default_rng(5)
    e0, e1 = ctx.event(), ctx.event()
    nccl = None
    if args.nccl_baseline and dist is not None:
        import torch
        nccl = dist.new_group(backend="nccl")
        ext = torch.cuda.ExternalStream(int(pkg.lib().qb_stream(ctx.h)))
        solo_groups, solo_area = pkg.tp.local_groups(ctx, 1, max(Ms), H, f, H)      # the rank's shard alone: GEMMs + own sum

        class Raw:                                  # a device buffer of the library as a torch tensor (no copy)
            def __init__(self, arr):
                self.__cuda_array_interface__ = {"shape": arr.shape, "typestr": "<f4", "data": (int(arr.ptr.value), False), "version": 2}
    for M in Ms:
        x = ctx.array(rng.standard_normal((M, H)).astype(np.float32))
        y = ctx.empty((M, H), np.float32)
        base_us = None
        if nccl is not None:
            import torch
            yb = ctx.empty((M, H), np.float32)
            yt = torch.as_tensor(Raw(yb), device="cuda:%d" % local)
            bt = []
            with torch.cuda.stream(ext):
                for it in range(args.iters + 3):
                    if not args.no_flush:
                        ctx.flush_l2()
                    ctx.sync()
                    dist.barrier()
                    ctx.record(e0)
                    solo_groups[0].ffn(w_gu, w_dn, x, M, yb)
                    dist.all_reduce(yt, group=nccl)
                    ctx.record(e1)
                    ctx.sync()
                    torch.cuda.synchronize()
                    if it >= 3:
                        bt.append(ctx.elapsed_ms(e0, e1))
            t = torch.tensor([float(np.median(bt)) * 1e3], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            base_us = float(t[0])
        times = []
        for it in range(args.iters + 3):
            if not args.no_flush:
                ctx.flush_l2()
            ctx.sync()
            if dist is not None:
                dist.barrier()
            ctx.record(e0)
            group.ffn(w_gu, w_dn, x, M, y)
            ctx.record(e1)
            ctx.sync()
            if it >= 3:
                times.append(ctx.elapsed_ms(e0, e1))
        us = float(np.median(times)) * 1e3
        if dist is not None:
            import torch
            t = torch.tensor([us], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t[0])
        if rank == 0:
            wbytes = (2 * f * H + H * f) / 32 * 34
            print(json.dumps({"tp": world, "M": M, "ffn_us": round(us, 2), "weight_MB_per_rank": round(wbytes / 1e6, 1),
                              "GBps_per_rank": round(wbytes / us / 1e3, 1), "allreduce_bytes": M * H * 4,
                              "unfused_gemms_plus_nccl_allreduce_us": None if base_us is None else round(base_us, 2),
                              "TOPs_total": round(2.0 * M * 3 * F * H / us / 1e6, 2)}), flush=True)
    ctx.sync()
    if dist is not None:
        dist.barrier()                  # nobody unmaps a receive area a peer may still write
    group.close()
    if nccl is not None:
        solo_groups[0].close()
    pkg.tp.ipc_release(ctx, opened)
    w_gu.free(); w_dn.free()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shapes", default="17408x5120,5120x17408,5120x6144,34816x5120,151936x5120")
    ap.add_argument("--m", "--rows", dest="m", default="1,4,16,64,128,512")
    ap.add_argument("--impls", default="1,2")
    ap.add_argument("--ksplit", type=int, default=0)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--tp", action="store_true", help="tensor-parallel FFN pair over the ranks of this launch")
    ap.add_argument("--nccl-baseline", action="store_true", help="with --tp: also time the unfused form (GEMMs, then an NCCL all-reduce)")
    args = ap.parse_args()
    if args.tp:
        return tp_sweep(args)
    pkg = entry.load_package()
    L = pkg.lib()
    ctx = pkg.Context(0)
    peak = 6548.5
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = float(json.load(open(p))["hbm_gbs"])
    rng = np.random.default_rng(5)
    e0, e1 = ctx.event(), ctx.event()
    int8_peak = ctx.int8_mma_peak()
    print(json.dumps({"int8_mma_peak_TOPs": round(int8_peak, 1), "how": "tcgen05.mma.kind::i8 128x256x32 back to back, operands in shared memory, one CTA per SM"}), flush=True)
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
                                  "TOPs": round(2.0 * M * N * K / us / 1e6, 2), "frac_int8_peak": round(2.0 * M * N * K / us / 1e6 / int8_peak, 4),
                                  "bit_identical_to_first_impl": same}), flush=True)
            q.free(); d.free(); part.free()
        w.free()
    ctx.close()


if __name__ == "__main__":
    main()
