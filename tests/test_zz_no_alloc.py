"""The matmul entry point for hosts that must not allocate device memory.

qb_q8_0_matmul_noalloc keeps its work area in an array built into the library instead of a buffer grown
with cudaMalloc (for servers whose own arena owns the device, or loops that cannot take the device-wide
synchronisation of an allocation).  It must give the bits of qb_q8_0_matmul, also when the shared work area
still holds the previous call's data, and must refuse shapes that do not fit.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(qb, ctx, fn_name, w, x, ksplit):
    M, K = x.shape
    N = w.rows
    xd = ctx.array(x)
    yd = ctx.empty((M, N), np.float32)
    yd.zero()
    L = qb.lib()
    if fn_name == "noalloc":
        qb.binding.check(L.qb_q8_0_matmul_noalloc(ctx.h, w.h, xd.ptr, M, K, yd.ptr, N, ksplit))
    else:
        qb.binding.check(L.qb_q8_0_matmul(ctx.h, w.h, xd.ptr, M, K, yd.ptr, N, ksplit, 1))
    return yd.download()


def test_noalloc_matmul_matches_matmul_on_two_calls_in_a_row(qb, orc, ctx):
    rng = np.random.default_rng(99)
    # call 1: split-K shape (partials live in the work area); call 2: a different, smaller shape whose
    # operands land on top of call 1's leftovers, with a single segment written straight to the output
    cases = [(640, 2048, 4, 3), (384, 512, 7, 1)]
    for (N, K, M, ksplit) in cases:
        blocks = orc.quantize_q8_0((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
        w = qb.Weight.from_blocks(ctx, blocks, N, K)
        x = rng.standard_normal((M, K)).astype(np.float32)
        got = _run(qb, ctx, "noalloc", w, x, ksplit)
        want = _run(qb, ctx, "alloc", w, x, ksplit)
        assert np.array_equal(got, want)                                  # bit-exact: integer dots, same fp32 order
        assert np.array_equal(got, orc.matmul_engine(blocks, N, K, x, ksplit=ksplit))
        w.free()


def test_noalloc_matmul_refuses_what_does_not_fit(qb, orc, ctx):
    rng = np.random.default_rng(98)
    N, K, M = 4096, 4096, 600          # 600 x 4096 int8 + 8 x 600 x 4096 partial floats > 8 MiB
    blocks = orc.quantize_q8_0((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    w = qb.Weight.from_blocks(ctx, blocks, N, K)
    xd = ctx.array(np.zeros((M, K), np.float32))
    yd = ctx.empty((M, N), np.float32)
    status = qb.lib().qb_q8_0_matmul_noalloc(ctx.h, w.h, xd.ptr, M, K, yd.ptr, N, 8)
    assert status == 4                                                    # QB_ERR_CAPACITY
    assert b"work area" in qb.lib().qb_last_error()
    w.free()


def test_noalloc_matmul_leaves_device_memory_alone(qb, orc, ctx):
    """The point of the entry point: between two readings of the device's free memory it allocates nothing, whatever
    the shapes it is given (the ordinary entry point may grow the context's work area meanwhile, so it is not called)."""
    rng = np.random.default_rng(97)
    shapes = [(640, 2048, 4, 3), (1024, 4096, 16, 0), (384, 512, 7, 1)]
    prepared = []
    for (N, K, M, ksplit) in shapes:
        blocks = orc.quantize_q8_0((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
        w = qb.Weight.from_blocks(ctx, blocks, N, K)
        prepared.append((w, ctx.array(rng.standard_normal((M, K)).astype(np.float32)), ctx.empty((M, N), np.float32), M, K, N, ksplit))
    L = qb.lib()
    w0, x0, y0, M0, K0, N0, k0 = prepared[0]
    qb.binding.check(L.qb_q8_0_matmul_noalloc(ctx.h, w0.h, x0.ptr, M0, K0, y0.ptr, N0, k0))      # first call on the device: address look-up
    ctx.sync()
    free_before, _ = ctx.mem_info()
    for _ in range(3):
        for (w, x, y, M, K, N, ksplit) in prepared:
            qb.binding.check(L.qb_q8_0_matmul_noalloc(ctx.h, w.h, x.ptr, M, K, y.ptr, N, ksplit))
    ctx.sync()
    free_after, _ = ctx.mem_info()
    assert free_after == free_before
    for p in prepared:
        p[0].free()
