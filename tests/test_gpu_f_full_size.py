"""Size-independent properties at the full sizes of the 27B-class shape (where the CPU oracle would take minutes):
the two GEMM kernels agree bit for bit, a row's result does not depend on the batch it is in, a K-segment split
leaves partials that add up to the one-segment result within fp32 reassociation, and the attention / DeltaNet
kernels give a sequence the same bits alone and inside a batch."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _partials(qb, ctx, w, x, S, impl):
    L = qb.lib()
    M = x.shape[0]
    q, d = qb.binding.quantize_act(ctx, x)
    part = ctx.empty((S, M, w.rows), np.float32)
    qb.binding.check(L.qb_q8_gemm_partials(ctx.h, w.h, q.ptr, d.ptr, M, part.ptr, S, impl))
    return part.download()


@pytest.mark.parametrize("N,K", [(17408, 5120), (5120, 17408)])
def test_full_size_gemm_kernels_agree_and_rows_are_batch_invariant(qb, ctx, N, K):
    L = qb.lib()
    w = qb.Weight.synth(ctx, 0x5EED, 91, N, K, 0.02)
    S = L.qb_ksplit_policy(N, K)
    x = np.random.default_rng(8).standard_normal((128, K)).astype(np.float32)
    tc4 = _partials(qb, ctx, w, x[:4], S, 2)
    assert np.array_equal(tc4, _partials(qb, ctx, w, x[:4], S, 1)), "tensor-core and CUDA-core kernels differ"
    tc1 = _partials(qb, ctx, w, x[:1], S, 2)
    assert np.array_equal(tc1[:, 0], tc4[:, 0]), "row 0 alone differs from row 0 of a 4-row launch"
    tc128 = _partials(qb, ctx, w, x, S, 2)                       # the 128-row tile, 16 epilogue warps
    assert np.array_equal(tc128[:, :4], tc4), "rows of a 128-row launch differ from the 4-row launch"
    tc33 = _partials(qb, ctx, w, x[:33], S, 2)                    # 64-row tile with a ragged edge
    assert np.array_equal(tc33, tc128[:, :33])
    # the split partials add up to the single-segment product (fp32 reassociation only)
    one = _partials(qb, ctx, w, x[:4], 1, 2)[0]
    tot = tc4.sum(axis=0, dtype=np.float64)
    assert np.abs(tot - one).max() <= 1e-4 * np.abs(one).max()
    w.free()


def test_full_size_lm_head_argmax_agrees_between_kernels(qb, ctx):
    """151936 x 5120 LM head: the M = 1 CUDA-core matvec and the tensor-core kernel give identical logits."""
    N, K = 151936, 5120
    w = qb.Weight.synth(ctx, 0x5EED, 92, N, K, 0.02)
    x = np.random.default_rng(9).standard_normal((1, K)).astype(np.float32)
    a = _partials(qb, ctx, w, x, 1, 1)[0, 0]
    b = _partials(qb, ctx, w, x, 1, 2)[0, 0]
    assert np.array_equal(a, b)
    assert int(np.argmax(a)) == int(np.argmax(b))
    w.free()


def test_full_size_deltanet_sequence_alone_equals_sequence_in_batch(qb, ctx):
    """48 v / 16 k heads x 128: sequence 1 of a 3-sequence launch (64-column form) == the same sequence launched
    alone (32-column form), bit for bit, checkpoints included."""
    nk, nv, hd, R, n_slots = 16, 48, 128, 4, 4
    rng = np.random.default_rng(10)
    Cq = (2 * nk + nv) * hd
    stride = Cq + nv * hd + 2 * nv
    L = qb.lib()

    def run(n_seqs, proj, state, conv, slot):
        d = {k: ctx.array(v) for k, v in dict(proj=proj, state=state, conv=conv, slot=slot).items()}
        core = ctx.empty((n_seqs * R, nv * hd), np.float32)
        qb.binding.check(L.qb_deltanet_rows(ctx.h, d["proj"].ptr, n_seqs, R, stride, cw.ptr, sa.ptr, dt.ptr, nw.ptr, nk, nv, hd,
                                            C.c_float(1e-6), d["state"].ptr, d["conv"].ptr, n_slots, d["slot"].ptr, 1, core.ptr))
        return core.download(), d["state"].download(), d["conv"].download()

    cw = ctx.array(rng.uniform(-0.5, 0.5, (Cq, 4)).astype(np.float32))
    sa = ctx.array((-np.exp(rng.uniform(0, np.log(16), nv))).astype(np.float32))
    dt = ctx.array(rng.uniform(-4, -1, nv).astype(np.float32))
    nw = ctx.array(np.ones(hd, np.float32))
    proj = rng.standard_normal((3 * R, stride)).astype(np.float32)
    state = (rng.standard_normal((3, n_slots, nv, hd, hd)) * 0.05).astype(np.float32)
    conv = rng.standard_normal((3, n_slots, Cq, 3)).astype(np.float32)
    slot = np.array([0, 2, 1], np.int32)
    core3, st3, cv3 = run(3, proj, state, conv, slot)
    core1, st1, cv1 = run(1, proj[R:2 * R], state[1:2], conv[1:2], slot[1:2])
    assert np.array_equal(core3[R:2 * R], core1)
    assert np.array_equal(st3[1], st1[0]) and np.array_equal(cv3[1], cv1[0])
