"""GPU parity tests of the Q8_0 weight path, the activation quantisers and the Q8 GEMM, all
through the C ABI, against the CPU oracle and (when built) the reference's own CUDA kernels."""
import ctypes as C

import numpy as np
import pytest

from conftest import std_mt19937_uniform
from test_oracle_cpu import MMQ_PARITY_SHAPES

pytestmark = pytest.mark.gpu


def _w(orc, rng, N, K, scale=0.02):
    return orc.quantize_q8_0((rng.standard_normal((N, K)) * scale).astype(np.float32))


def test_weight_upload_download_roundtrip(qb, orc, ctx):
    rng = np.random.default_rng(10)
    for (N, K) in [(128, 128), (200, 256), (48, 512), (1000, 384)]:   # ragged row counts too
        blocks = _w(orc, rng, N, K)
        w = qb.Weight.from_blocks(ctx, blocks, N, K)
        assert np.array_equal(w.download(), blocks)
        w.free()


def test_synth_weight_matches_host_recipe(qb, orc, ctx):
    for (tid, N, K) in [(33, 256, 256), (7, 130, 512)]:
        w = qb.Weight.synth(ctx, 0x5EED, tid, N, K, 0.02)
        assert np.array_equal(w.download(), orc.synth_q8_0(0x5EED, tid, N, K, 0.02))
        w.free()


def test_get_rows(qb, orc, ctx):
    rng = np.random.default_rng(11)
    N, K = 300, 256
    blocks = _w(orc, rng, N, K)
    w = qb.Weight.from_blocks(ctx, blocks, N, K)
    ids = np.array([0, 299, 17, 17, 128], np.int32)
    out = ctx.empty((len(ids), K), np.float32)
    qb.binding.check(qb.lib().qb_q8_0_get_rows(ctx.h, w.h, ctx.array(ids).ptr, len(ids), out.ptr, K))
    assert np.array_equal(out.download(), orc.get_rows(blocks, N, K, ids))


@pytest.mark.parametrize("M,K", [(1, 128), (4, 5120), (7, 256), (33, 1024)])
def test_activation_quantisers_bit_exact(qb, orc, ctx, M, K):
    rng = np.random.default_rng(12 + M)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.01, 30.0, (M, 1))).astype(np.float32)
    x[0, :32] = 0.0
    q, d = qb.binding.quantize_act(ctx, x)
    oq, od = orc.quantize_act(x)
    assert np.array_equal(q.download(), oq)
    assert np.array_equal(d.download()[:, :M], od)
    xd = ctx.array(x)
    o81 = ctx.empty(M * (K // 32) * 36, np.uint8)
    qb.binding.check(qb.lib().qb_quantize_q8_1(ctx.h, xd.ptr, M, K, K, o81.ptr))
    g, w = o81.download().reshape(-1, 36), orc.quantize_q8_1(x).reshape(-1, 36)
    assert np.array_equal(g[:, :2], w[:, :2]) and np.array_equal(g[:, 4:], w[:, 4:])
    # the block sum is a float reduction: same value up to fp16 rounding of a differently ordered sum
    gs, ws = g[:, 2:4].copy().view(np.float16).astype(np.float32), w[:, 2:4].copy().view(np.float16).astype(np.float32)
    assert np.allclose(gs, ws, rtol=2e-3, atol=2e-2)
    if K % 128 == 0:
        omq = ctx.empty((K // 128) * M * 144, np.uint8)
        qb.binding.check(qb.lib().qb_quantize_q8_1_mmq(ctx.h, xd.ptr, M, K, K, omq.ptr))
        assert np.array_equal(omq.download(), orc.quantize_q8_1_mmq(x))


def test_block_dots_exact(qb, orc, ctx):
    rng = np.random.default_rng(13)
    N, K, M = 192, 512, 5
    blocks = _w(orc, rng, N, K)
    w = qb.Weight.from_blocks(ctx, blocks, N, K)
    q = rng.integers(-127, 128, (M, K)).astype(np.int8)
    out = ctx.empty((M, N, K // 32), np.int32)
    qb.binding.check(qb.lib().qb_q8_block_dots(ctx.h, w.h, ctx.array(q).ptr, M, out.ptr))
    assert np.array_equal(out.download(), orc.block_dots(blocks, N, K, q))


GEMM_CASES = [(128, 128, 1, 0), (256, 512, 4, 0), (200, 256, 3, 2), (768, 256, 8, 0), (130, 1024, 5, 3),
              (512, 2048, 16, 1), (1024, 640, 2, 5), (384, 384, 9, 0), (5120, 6144, 4, 0), (2048, 5120, 1, 0)]


@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("N,K,M,ksplit", GEMM_CASES)
def test_gemm_bit_exact_vs_oracle(qb, orc, ctx, N, K, M, ksplit, impl):
    """Integer dots exact, fp32 accumulation in the engine order: every output bit-identical."""
    rng = np.random.default_rng(N + K + M)
    blocks = _w(orc, rng, N, K)
    w = qb.Weight.from_blocks(ctx, blocks, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    try:
        y = qb.binding.matmul(ctx, w, x, ksplit=ksplit, impl=impl)
    except qb.QbError as e:
        if impl == 2 and "does not support" in str(e) or "not built" in str(e):
            pytest.skip("tensor-core kernel not available for this shape")
        raise
    want = orc.matmul_engine(blocks, N, K, x, ksplit=ksplit)
    assert np.array_equal(y, want), float(np.abs(y - want).max())
    w.free()


@pytest.mark.parametrize("N,K,M,ksplit", [(256, 512, 16, 0), (384, 1024, 33, 2), (128, 2048, 64, 1), (640, 512, 128, 0),
                                          (256, 640, 130, 3), (130, 256, 300, 0), (5120, 5120, 12, 0)])
def test_gemm_tensor_core_bit_exact_large_m(qb, orc, ctx, N, K, M, ksplit):
    """tcgen05 kernel over every activation-tile width (16/32/64/128) and several tiles."""
    rng = np.random.default_rng(N * 3 + K + M)
    blocks = _w(orc, rng, N, K)
    w = qb.Weight.from_blocks(ctx, blocks, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    y = qb.binding.matmul(ctx, w, x, ksplit=ksplit, impl=2)
    want = orc.matmul_engine(blocks, N, K, x, ksplit=ksplit)
    assert np.array_equal(y, want), float(np.abs(y - want).max())
    ctx.sync()    # also reads the kernel's bounded-wait error flag
    w.free()


def test_gemm_partials_layout(qb, orc, ctx):
    rng = np.random.default_rng(14)
    N, K, M, S = 256, 1024, 3, 4
    blocks = _w(orc, rng, N, K)
    w = qb.Weight.from_blocks(ctx, blocks, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    q, d = qb.binding.quantize_act(ctx, x)
    part = ctx.empty((S, M, N), np.float32)
    qb.binding.check(qb.lib().qb_q8_gemm_partials(ctx.h, w.h, q.ptr, d.ptr, M, part.ptr, S, 1))
    oq, od = orc.quantize_act(x)
    _, want = orc.gemm_engine(blocks, N, K, oq, od, ksplit=S, want_partials=True)
    assert np.array_equal(part.download(), want)


def test_row_result_independent_of_batch(qb, orc, ctx):
    """A row's output must not depend on how many rows share the launch (greedy M=1 vs verify M=k+1)."""
    rng = np.random.default_rng(15)
    N, K = 640, 1024
    w = qb.Weight.from_blocks(ctx, _w(orc, rng, N, K), N, K)
    x = rng.standard_normal((16, K)).astype(np.float32)
    y16 = qb.binding.matmul(ctx, w, x, impl=1)
    for M in (1, 2, 4, 5, 8):
        assert np.array_equal(qb.binding.matmul(ctx, w, x[:M], impl=1), y16[:M])


def test_mmq_parity_procedure_gpu(qb, orc, ctx):
    """tests/mmq_parity.cu on the product kernel: all 16 shapes, reference tolerance."""
    rs = np.random.RandomState(0x5EED)
    for (M, N, K) in MMQ_PARITY_SHAPES:
        W = std_mt19937_uniform(rs, M * K, -0.5, 0.5).reshape(M, K)
        X = std_mt19937_uniform(rs, N * K, -1.0, 1.0).reshape(N, K)
        if N > 256:
            X = X[:256]        # the CUDA-core kernel is a small-batch kernel; rows are independent
        blocks = orc.quantize_q8_0(W)
        w = qb.Weight.from_blocks(ctx, blocks, M, K)
        got = qb.binding.matmul(ctx, w, X)
        Wd = orc.dequant_q8_0(blocks, M, K)
        q, d = orc.quantize_act(X)
        Xd = (q.astype(np.float32).reshape(len(X), K // 32, 32) * d.T[..., None]).reshape(len(X), K)
        ref = Xd.astype(np.float64) @ Wd.T.astype(np.float64)
        diff = np.abs(got - ref)
        bad = (diff > 5e-3) & (diff > 1e-3 * np.maximum(np.abs(ref), 1e-6))
        assert not bad.any(), (M, N, K, float(diff.max()))
        w.free()


# ---- the reference's own kernels as comparator --------------------------------------------------

def _dev(ctx, arr):
    return ctx.array(arr)


@pytest.mark.parametrize("N,K,M", [(256, 512, 1), (384, 2048, 4), (128, 5120, 3), (512, 1024, 8)])
def test_oracle_matches_reference_mmvq_kernel(qb, orc, ctx, ref, N, K, M):
    """Pins the oracle's restatement of quantize_q8_1 + mul_mat_vec_q8_0 (src/mmvq_q8.cu) on the
    reference kernels compiled for sm_100a."""
    if ref is None:
        pytest.skip("oracle/_ref not built")
    rng = np.random.default_rng(16 + M)
    blocks = _w(orc, rng, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    wdev = _dev(ctx, orc.repack_split_plane(blocks, N, K))
    xdev = _dev(ctx, x)
    y81 = ctx.empty(M * (K // 32) * 36, np.uint8)
    out = ctx.empty((M, N), np.float32)
    assert ref.ref_quantize_q8_1(xdev.ptr, y81.ptr, C.c_uint32(M), C.c_uint32(K)) == 0
    g, w = y81.download().reshape(-1, 36), orc.quantize_q8_1(x).reshape(-1, 36)
    assert np.array_equal(g[:, :2], w[:, :2]) and np.array_equal(g[:, 4:], w[:, 4:])
    assert ref.ref_mmvq_q8_0(wdev.ptr, y81.ptr, out.ptr, C.c_uint32(N), C.c_uint32(K), C.c_uint32(M)) == 0
    got = out.download()
    want = orc.matmul_mmvq(blocks, N, K, x)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-6), float(np.abs(got - want).max())
    # and the product kernel agrees with the reference kernel within the reference's cross-kernel bound
    # (tests/vmed_bench.cu:92-117, max rel 2e-2 of the output scale)
    mine = qb.binding.matmul(ctx, qb.Weight.from_blocks(ctx, blocks, N, K), x)
    assert np.abs(mine - got).max() <= 2e-2 * np.abs(got).max()


@pytest.mark.parametrize("N,K,M", [(256, 512, 16), (128, 2048, 64), (384, 1024, 128), (256, 256, 12)])
def test_oracle_matches_reference_mmq_kernel(qb, orc, ctx, ref, N, K, M):
    """Pins quantize_mmq_q8_1 and the MMQ accumulation order (src/mmq_q8.cu) on the reference kernels:
    bit-exact, since the integer dots are exact and the fp32 order is sequential in K."""
    if ref is None:
        pytest.skip("oracle/_ref not built")
    rng = np.random.default_rng(17 + M)
    blocks = _w(orc, rng, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    wdev = _dev(ctx, orc.repack_split_plane(blocks, N, K))
    xdev = _dev(ctx, x)
    ymq = ctx.empty((K // 128) * M * 144, np.uint8)
    assert ref.ref_quantize_mmq_q8_1(xdev.ptr, ymq.ptr, C.c_uint32(M), C.c_uint32(K)) == 0
    assert np.array_equal(ymq.download(), orc.quantize_q8_1_mmq(x))
    want = orc.matmul_mmq(blocks, N, K, x)
    for fn in (ref.ref_mmq_q8_0, ref.ref_mmq_q8_0_medium):
        out = ctx.empty((M, N), np.float32)
        out.zero()
        rc = fn(wdev.ptr, ymq.ptr, out.ptr, C.c_uint32(N), C.c_uint32(K), C.c_uint32(M))
        if rc == -1:
            continue   # launcher declined the shape
        assert rc == 0
        got = out.download()
        assert np.array_equal(got, want), float(np.abs(got - want).max())
    # the engine order with a single segment is the same order: product kernel == reference kernel
    mine = qb.binding.matmul(ctx, qb.Weight.from_blocks(ctx, blocks, N, K), x, ksplit=1)
    assert np.array_equal(mine, want)
