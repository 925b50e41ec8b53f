"""The reference's own CUDA GEMM kernels (compiled for sm_100a into oracle/_ref) timed beside the product kernel on
the verify shapes: same weights, same activations, cold L2 before every launch, CUDA events.  The numbers are
printed (run with -s to see them); the assertion is only that the product kernel is not slower than the reference
kernel on any shape of the step."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K", [(17408, 5120), (5120, 17408)])
def test_reference_gemm_kernels_timed_beside_ours(qb, orc, ctx, ref, N, K):
    if ref is None or not hasattr(ref, "ref_time_gemm"):
        pytest.skip("oracle/_ref not built")
    L = qb.lib()
    w = qb.Weight.synth(ctx, 0x5EED, 77, N, K, 0.02)
    blocks = w.download()
    wref = ctx.array(orc.repack_split_plane(blocks, N, K))
    flush = ctx.empty((256 << 20,), np.uint8)
    rng = np.random.default_rng(3)
    e0, e1 = ctx.event(), ctx.event()
    lines = []
    for M in (1, 4, 16, 64):
        x = rng.standard_normal((M, K)).astype(np.float32)
        xdev = ctx.array(x)
        out = ctx.empty((M, N), np.float32)
        times = {}
        # reference: mul_mat_vec for the small batches (its verify path up to 8 rows), MMQ kernels otherwise
        if M <= 8:
            y81 = ctx.empty(M * (K // 32) * 36, np.uint8)
            assert ref.ref_quantize_q8_1(xdev.ptr, y81.ptr, C.c_uint32(M), C.c_uint32(K)) == 0
            kinds = [(0, "mmvq", y81)]
        else:
            kinds = []
        ymq = ctx.empty((K // 128) * M * 144, np.uint8)
        assert ref.ref_quantize_mmq_q8_1(xdev.ptr, ymq.ptr, C.c_uint32(M), C.c_uint32(K)) == 0
        kinds += [(1, "mmq", ymq), (2, "mmq_medium", ymq)]
        for kind, name, y in kinds:
            us = C.c_float()
            rc = ref.ref_time_gemm(kind, wref.ptr, y.ptr, out.ptr, C.c_uint32(N), C.c_uint32(K), C.c_uint32(M), 8, flush.ptr,
                                   C.c_size_t(flush.nbytes), C.byref(us))
            if rc == 0:
                times[name] = us.value
        # ours: the GEMM launch alone on pre-quantised activations (engine split policy)
        q, d = qb.binding.quantize_act(ctx, x)
        S = L.qb_ksplit_policy(N, K)
        part = ctx.empty((S, M, N), np.float32)
        ts = []
        for it in range(10):
            ctx.flush_l2()
            ctx.record(e0)
            qb.binding.check(L.qb_q8_gemm_partials(ctx.h, w.h, q.ptr, d.ptr, M, part.ptr, S, 0))
            ctx.record(e1)
            ctx.sync()
            if it >= 2:
                ts.append(ctx.elapsed_ms(e0, e1) * 1e3)
        ours = float(np.median(ts))
        best_ref = min(times.values())
        lines.append("N=%d K=%d M=%d: ours %.1f us; reference %s" % (N, K, M, ours, ", ".join("%s %.1f us" % kv for kv in times.items())))
        assert ours <= best_ref * 1.05, lines[-1]
    print("\n" + "\n".join(lines))
    w.free()
