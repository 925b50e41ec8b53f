"""GPU tests of the fused [gate; up] projection + SwiGLU + int8 quantisation: the one-launch form (GEMM epilogue)
and the two-launch form give the same bits, and both match the CPU oracle's arithmetic."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(qb, ctx, w, x, F, mode):
    L = qb.lib()
    M, K = x.shape
    ld = (M + 3) & ~3
    hq = ctx.empty((M, F), np.int8)
    hd = ctx.empty((F // 32, ld), np.float32)
    hd.zero()
    qb.binding.check(L.qb_q8_0_matmul_silu_mul_q8(ctx.h, w, ctx.array(x).ptr, M, K, hq.ptr, hd.ptr, mode))
    ctx.sync()
    return hq.download(), hd.download()[:, :M]


@pytest.mark.parametrize("M", [1, 4, 13, 16])
def test_fused_gate_up_swiglu_one_launch_equals_two_launches_and_oracle(qb, orc, ctx, M):
    # 2F = 19456 rows = 152 tiles: one K segment under the split policy, so the one-launch form is available
    F, K = 9728, 1280
    assert orc.ksplit_policy(2 * F, K) == 1
    rng = np.random.default_rng(21)
    wg = rng.normal(0, 0.05, (F, K)).astype(np.float32)
    wu = rng.normal(0, 0.05, (F, K)).astype(np.float32)
    gate, up = orc.quantize_q8_0(wg), orc.quantize_q8_0(wu)
    w = qb.binding.vp()
    qb.binding.check(qb.lib().qb_weight_q8_0_gate_up(ctx.h, gate.ctypes.data_as(qb.binding.vp), up.ctypes.data_as(qb.binding.vp), F, K,
                                                    C.byref(w)))
    x = rng.standard_normal((M, K)).astype(np.float32)
    q1, d1 = _run(qb, ctx, w, x, F, 2)          # one launch
    q2, d2 = _run(qb, ctx, w, x, F, 1)          # GEMM, then the SwiGLU kernel
    assert np.array_equal(q1, q2) and np.array_equal(d1, d2)
    # oracle: engine-order products of the two tensors, silu(g) * u, the activation quantiser
    oq, od = orc.quantize_act(x)
    g = orc.gemm_engine(gate, F, K, oq, od, ksplit=1)
    u = orc.gemm_engine(up, F, K, oq, od, ksplit=1)
    h = (g / (np.float32(1) + np.exp(-g, dtype=np.float32)) * u).astype(np.float32)
    wq, wd = orc.quantize_act(h)
    # the device's expf may differ from numpy's in the last bit: allow one quantisation step on rare elements
    assert np.abs(q1.astype(np.int32) - wq.astype(np.int32)).max() <= 1
    assert (q1 != wq).mean() < 1e-3
    assert np.allclose(d1, wd, rtol=1e-5, atol=0)
    qb.lib().qb_weight_free(ctx.h, w)


def test_two_launch_form_with_split_partials(qb, orc, ctx):
    """A narrow FFN (several K segments under the policy): products stay split partials, the SwiGLU kernel adds them."""
    F, K, M = 512, 256, 5
    assert orc.ksplit_policy(2 * F, K) > 1
    rng = np.random.default_rng(22)
    gate = orc.quantize_q8_0(rng.normal(0, 0.05, (F, K)).astype(np.float32))
    up = orc.quantize_q8_0(rng.normal(0, 0.05, (F, K)).astype(np.float32))
    w = qb.binding.vp()
    qb.binding.check(qb.lib().qb_weight_q8_0_gate_up(ctx.h, gate.ctypes.data_as(qb.binding.vp), up.ctypes.data_as(qb.binding.vp), F, K,
                                                    C.byref(w)))
    x = rng.standard_normal((M, K)).astype(np.float32)
    q1, d1 = _run(qb, ctx, w, x, F, 0)
    oq, od = orc.quantize_act(x)
    S = orc.ksplit_policy(2 * F, K)
    g = orc.gemm_engine(gate, F, K, oq, od, ksplit=S)
    u = orc.gemm_engine(up, F, K, oq, od, ksplit=S)
    h = (g / (np.float32(1) + np.exp(-g, dtype=np.float32)) * u).astype(np.float32)
    wq, wd = orc.quantize_act(h)
    assert np.abs(q1.astype(np.int32) - wq.astype(np.int32)).max() <= 1 and (q1 != wq).mean() < 1e-3
    assert np.allclose(d1, wd, rtol=1e-5, atol=0)
    with pytest.raises(qb.QbError):
        _run(qb, ctx, w, x, F, 2)               # the one-launch form is not available for this shape
    qb.lib().qb_weight_free(ctx.h, w)
