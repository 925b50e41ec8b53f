"""Pins the operators of the step on the reference's own CUDA DeviceBackend (CudaDeviceBackend, src/kernels_cuda.cu:9564,
built without FlashInfer from the reference sources into oracle/_ref/libqw3ref_backend.so; `make -C oracle ref-backend`):
the reference's tensors, weights, stream and kernel dispatch on one side, this project's C ABI and the CPU oracle on the
other, same inputs.  Every test skips when the library has not been built.

Tolerances: the reference's RoPE uses __powf / __sincosf (src/kernels_cuda.cu:4711-4714), ours a host-made inverse-frequency
table and sincosf, so rotated values differ by up to ~1e-3 at positions in the thousands; everything else agrees to a few
float32 ulps per accumulated term."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def rb():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_backend
    if not ref_backend.available():
        pytest.skip("oracle/_ref/libqw3ref_backend.so not built (make -C oracle ref-backend)")
    b = ref_backend.RefBackend(linear=1)
    yield b
    b.close()


@pytest.fixture(autouse=True)
def _free_ref_tensors(request):
    yield
    if "rb" in request.fixturenames:
        request.getfixturevalue("rb").release()


def err(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max())


def test_reference_backend_is_the_cuda_backend(rb):
    assert "cuda" in rb.name().lower()


@pytest.mark.parametrize("M", [1, 4])
def test_rms_norm_batch(qb, orc, ctx, rb, M):
    rng = np.random.default_rng(300 + M)
    n = 5120
    x = (rng.standard_normal((M, n)) * 3).astype(np.float32)
    w = rng.uniform(0.5, 1.5, n).astype(np.float32)
    t_out = rb.empty(M * n)
    rb.call("rms_norm_batch", t_out, rb.tensor(x), rb.weight_f32(w), M, n, 1e-6)
    ref = rb.download(t_out, (M, n))
    want = orc.rms_norm(x, w, 1e-6)
    assert np.allclose(want, ref, rtol=1e-5, atol=1e-6), err(want, ref)
    out = ctx.empty((M, n), np.float32)
    qb.binding.check(qb.lib().qb_rms_norm(ctx.h, ctx.array(x).ptr, ctx.array(w).ptr, M, n, n, 1e-6, out.ptr))
    got = out.download()
    assert np.allclose(got, ref, rtol=1e-5, atol=1e-6), err(got, ref)


@pytest.mark.parametrize("n_heads,n_kv,hd,base,R", [(24, 4, 256, 700, 4), (16, 2, 128, 300, 3), (24, 4, 256, 2500, 1)])
def test_qk_norm_rope_append_and_gated_attention_chain(qb, orc, ctx, rb, n_heads, n_kv, hd, base, R):
    """rmsnorm_per_head_batch + rope_partial_batch + kv_append_batch (the reference's q/k preparation, three ops on
    separate q, k, v tensors) against the fused qb_qk_norm_rope_append, then attention_decode_batch_gated of the
    reference backend against qb_attention_paged_gated and the oracle on identical q and fp16 caches."""
    rng = np.random.default_rng(400 + base)
    T = base + R
    page = 16
    pps = (T + page) // page + 1
    pt = np.arange(pps, dtype=np.int32).reshape(1, pps)
    kvd = n_kv * hd
    qd = n_heads * 2 * hd
    stride = qd + 2 * kvd
    rope_dim = hd // 4
    theta, eps = 1e7, 1e-6
    qw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    kw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    qkv = rng.standard_normal((T, stride)).astype(np.float32)

    # the reference's three ops, all T rows as one batch from position 0, into its own fp16 caches
    t_q, t_k, t_v = rb.tensor(qkv[:, :qd]), rb.tensor(qkv[:, qd:qd + kvd]), rb.tensor(qkv[:, qd + kvd:])
    w_q, w_k = rb.weight_f32(qw), rb.weight_f32(kw)
    rb.call("rmsnorm_per_head_batch", t_q, w_q, T, qd, n_heads, 2 * hd, hd, eps)
    rb.call("rmsnorm_per_head_batch", t_k, w_k, T, kvd, n_kv, hd, hd, eps)
    rb.call("rope_partial_batch", t_q, T, qd, n_heads, 2 * hd, rope_dim, 0, theta)
    rb.call("rope_partial_batch", t_k, T, kvd, n_kv, hd, rope_dim, 0, theta)
    t_kc, t_vc = rb.empty(pps * page * kvd, kind=1), rb.empty(pps * page * kvd, kind=1)
    assert rb.L.rb_tensor_elem_size(t_kc) == 2
    rb.call("kv_append_batch", t_kc, t_k, 0, kvd, T)
    rb.call("kv_append_batch", t_vc, t_v, 0, kvd, T)
    ref_q = rb.download(t_q, (T, qd))
    ref_kc = rb.download(t_kc, (pps * page, kvd), np.uint16).view(np.float16).astype(np.float32)
    ref_vc = rb.download(t_vc, (pps * page, kvd), np.uint16)

    # ours: the fused kernel over the same rows
    d_qkv = ctx.array(qkv)
    d_kc, d_vc = ctx.array(np.zeros((pps * page, kvd), np.uint16)), ctx.array(np.zeros((pps * page, kvd), np.uint16))
    d_pt, d_pos = ctx.array(pt), ctx.array(np.array([0], np.int32))
    invf = orc.inv_freq(rope_dim, theta)
    L = qb.lib()
    qb.binding.check(L.qb_qk_norm_rope_append(ctx.h, d_qkv.ptr, T, stride, ctx.array(qw).ptr, ctx.array(kw).ptr, ctx.array(invf).ptr,
                                              n_heads, n_kv, hd, rope_dim, eps, d_pos.ptr, 1, d_pt.ptr, pps, page, d_kc.ptr, d_vc.ptr))
    ctx.sync()
    got_rows = d_qkv.download()
    got_kc_bits, got_vc_bits = d_kc.download(), d_vc.download()
    got_kc = got_kc_bits.view(np.float16).astype(np.float32)
    # the reference's angle is off by up to ~1.2e-6 * position radians (fp32 exponent of __powf, the fp32 range
    # reduction of __sincosf); a rotated pair moves by its length times that
    scale_q = float(np.abs(ref_q).max())
    bound = (5e-5 + 1.2e-6 * T) * scale_q * 1.5
    assert err(got_rows[:, :qd], ref_q) < bound, (err(got_rows[:, :qd], ref_q), bound)
    assert err(got_kc[:T], ref_kc[:T]) < bound + 4e-3, (err(got_kc[:T], ref_kc[:T]), bound)      # + one fp16 step
    assert np.array_equal(got_vc_bits[:T], ref_vc[:T])           # V is a pure fp32 -> fp16 conversion: same bits
    # the oracle's restatement of the same three ops
    o_rows = qkv.copy()
    okc, ovc = np.zeros((pps * page, kvd), np.uint16), np.zeros((pps * page, kvd), np.uint16)
    orc.qk_norm_rope_append(o_rows, qw, kw, invf, n_heads, n_kv, hd, rope_dim, eps, np.zeros(T, np.int32),
                            np.arange(T, dtype=np.int32), pt, page, okc, ovc)
    assert err(o_rows[:, :qd], ref_q) < bound, (err(o_rows[:, :qd], ref_q), bound)
    assert np.array_equal(ovc[:T], ref_vc[:T])
    # rows near position 0, where the fast sincos is as good as the precise one: a tight bound on norm + rotation
    assert np.allclose(o_rows[:8, :qd], ref_q[:8], rtol=2e-5, atol=2e-5), err(o_rows[:8, :qd], ref_q[:8])
    assert np.allclose(got_rows[:8, :qd], ref_q[:8], rtol=2e-5, atol=2e-5), err(got_rows[:8, :qd], ref_q[:8])

    # attention of the last R rows on identical inputs: our q and our caches go into reference tensors
    q_last = np.ascontiguousarray(got_rows[base:, :qd])
    t_q2 = rb.tensor(q_last)
    t_kc2, t_vc2 = rb.tensor(got_kc_bits, kind=1), rb.tensor(got_vc_bits, kind=1)
    t_out = rb.empty(R * n_heads * hd)
    rb.call("attention_decode_batch_gated", t_out, t_q2, 2 * hd, t_kc2, t_vc2, n_heads, n_kv, hd, base, R, qd, n_heads * hd,
            float(1.0 / np.sqrt(hd)))
    ref_out = rb.download(t_out, (R, n_heads * hd))
    rows_last = ctx.array(np.ascontiguousarray(got_rows[base:]))
    d_pos2 = ctx.array(np.array([base], np.int32))
    out = ctx.empty((R, n_heads * hd), np.float32)
    qb.binding.check(L.qb_attention_paged_gated(ctx.h, rows_last.ptr, R, stride, n_heads, n_kv, hd, d_pos2.ptr, 1, d_pt.ptr, pps, page,
                                                d_kc.ptr, d_vc.ptr, T, out.ptr))
    ctx.sync()
    got = out.download()
    # fp16 q and p on our side, fp32 on the reference's
    assert np.allclose(got, ref_out, rtol=2e-3, atol=1e-3), err(got, ref_out)
    want = orc.attention_paged_gated(got_rows[base:], n_heads, n_kv, hd, np.zeros(R, np.int32),
                                     (base + np.arange(R)).astype(np.int32), pt, page, got_kc_bits, got_vc_bits)
    assert np.allclose(want, ref_out, rtol=1e-4, atol=2e-5), err(want, ref_out)


# head size 128 only: the reference normalises q and k with l2_norm_128_batch_kernel (src/kernels_cuda.cu:4122)
@pytest.mark.parametrize("nk,nv,hd,T,ckpt", [(16, 48, 128, 4, True), (16, 48, 128, 1, True), (16, 48, 128, 37, False),
                                             (4, 8, 128, 3, True)])
def test_recurrent_batch_layer_core(qb, orc, ctx, rb, nk, nv, hd, T, ckpt):
    """recurrent_batch (src/kernels_cuda.cu:15053: conv1d + SiLU, L2 norm of q and k, gated delta rule, RMSNorm * SiLU(z),
    with the per-row state checkpoints the MTP verifier rolls back to) against qb_deltanet_rows and the oracle."""
    rng = np.random.default_rng(500 + T)
    C_ = (2 * nk + nv) * hd
    vdim = nv * hd
    stride = C_ + vdim + 2 * nv
    proj = rng.standard_normal((T, stride)).astype(np.float32)
    conv_w = rng.uniform(-0.5, 0.5, (C_, 4)).astype(np.float32)
    ssm_a = (-np.exp(rng.uniform(0, np.log(16), nv))).astype(np.float32)
    dt = rng.uniform(-4, -1, nv).astype(np.float32)
    nw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    state0 = (rng.standard_normal((nv, hd, hd)) * 0.05).astype(np.float32)
    conv0 = rng.standard_normal((C_, 3)).astype(np.float32)
    n_slots = T if ckpt else 1

    t_core, t_state, t_conv = rb.empty(T * vdim), rb.tensor(state0), rb.tensor(conv0)
    t_cout = rb.empty(T * C_)
    t_proj, t_gate = rb.tensor(proj[:, :C_]), rb.tensor(proj[:, C_:C_ + vdim])
    t_alpha, t_beta = rb.tensor(proj[:, C_ + vdim:C_ + vdim + nv]), rb.tensor(proj[:, C_ + vdim + nv:])
    t_sck = rb.empty(T * state0.size) if ckpt else None
    t_cck = rb.empty(T * conv0.size) if ckpt else None
    rb.call("recurrent_batch", t_core, t_state, t_conv, t_cout, t_proj, t_gate, t_alpha, t_beta, rb.weight_f32(conv_w),
            rb.weight_f32(ssm_a), rb.weight_f32(dt), rb.weight_f32(nw), T, nk, nv, hd, hd, 4, C_, C_, vdim, nv, nv, vdim, 1e-6,
            t_sck, t_cck, T if ckpt else 0)
    ref_core = rb.download(t_core, (T, vdim))
    ref_state, ref_conv = rb.download(t_state, state0.shape), rb.download(t_conv, conv0.shape)

    st = np.zeros((n_slots,) + state0.shape, np.float32); st[0] = state0
    cv = np.zeros((n_slots,) + conv0.shape, np.float32); cv[0] = conv0
    want = orc.deltanet_rows(proj, conv_w, ssm_a, dt, nw, nk, nv, hd, 1e-6, st, cv, 0, ckpt)
    last = T - 1 if ckpt else 0
    assert np.allclose(want, ref_core, rtol=2e-3, atol=2e-4), err(want, ref_core)
    assert np.allclose(st[last], ref_state, rtol=1e-3, atol=1e-4), err(st[last], ref_state)
    assert np.array_equal(cv[last], ref_conv)
    if ckpt:
        ref_sck, ref_cck = rb.download(t_sck, (T,) + state0.shape), rb.download(t_cck, (T,) + conv0.shape)
        assert np.allclose(st, ref_sck, rtol=1e-3, atol=1e-4), err(st, ref_sck)
        assert np.array_equal(cv, ref_cck)

    g_st = np.zeros((1, n_slots) + state0.shape, np.float32); g_st[0, 0] = state0
    g_cv = np.zeros((1, n_slots) + conv0.shape, np.float32); g_cv[0, 0] = conv0
    d_state, d_conv = ctx.array(g_st), ctx.array(g_cv)
    core = ctx.empty((T, vdim), np.float32)
    qb.binding.check(qb.lib().qb_deltanet_rows(ctx.h, ctx.array(proj).ptr, 1, T, stride, ctx.array(conv_w).ptr, ctx.array(ssm_a).ptr,
                                               ctx.array(dt).ptr, ctx.array(nw).ptr, nk, nv, hd, 1e-6, d_state.ptr, d_conv.ptr,
                                               n_slots, ctx.array(np.zeros(1, np.int32)).ptr, 1 if ckpt else 0, core.ptr))
    ctx.sync()
    got, got_st, got_cv = core.download(), d_state.download()[0], d_conv.download()[0]
    assert np.allclose(got, ref_core, rtol=2e-3, atol=2e-4), err(got, ref_core)
    assert np.allclose(got_st[last], ref_state, rtol=1e-3, atol=1e-4), err(got_st[last], ref_state)
    assert np.array_equal(got_cv[last], ref_conv)
    if ckpt:
        assert np.allclose(got_st, ref_sck, rtol=1e-3, atol=1e-4), err(got_st, ref_sck)
        assert np.array_equal(got_cv, ref_cck)


def test_argmax_batch_with_ties(qb, orc, ctx, rb):
    rng = np.random.default_rng(600)
    M, n = 4, 151936
    x = rng.standard_normal((M, n)).astype(np.float32)
    x[0, 77] = x[0, 150000] = 9.0          # a tie: lowest index wins
    x[1, n - 1] = 11.0                     # last column
    x[2, 0] = 12.0                         # first column
    x[3, 4096] = x[3, 4097] = x[3, 90000] = 8.5
    tok, val = np.zeros(M, np.int32), np.zeros(M, np.float32)
    rb.call("argmax_batch", rb.tensor(x), M, n, tok.ctypes.data, val.ctypes.data)
    want = orc.argmax_rows(x)
    assert np.array_equal(tok, want), (tok, want)
    assert np.array_equal(val, x[np.arange(M), want])
    out = ctx.empty((M,), np.int32)
    qb.binding.check(qb.lib().qb_argmax_rows(ctx.h, ctx.array(x).ptr, M, n, n, out.ptr))
    assert np.array_equal(out.download(), tok)


def test_q8_0_get_rows_batch(qb, orc, ctx, rb):
    rng = np.random.default_rng(700)
    rows, cols = 4096, 5120
    blocks = orc.quantize_q8_0(rng.normal(0, 0.02, (rows, cols)).astype(np.float32))
    ids = np.array([0, 4095, 17, 17, 2048], np.int32)
    t_out = rb.empty(len(ids) * cols)
    ids64 = ids.astype(np.uint64)
    rb.call("q8_0_get_rows_batch", t_out, rb.weight_q8_0(blocks, rows, cols), ids64.ctypes.data, len(ids))
    ref = rb.download(t_out, (len(ids), cols))
    assert np.array_equal(orc.get_rows(blocks, rows, cols, ids), ref)
    w = qb.Weight.from_blocks(ctx, blocks, rows, cols)
    out = ctx.empty((len(ids), cols), np.float32)
    qb.binding.check(qb.lib().qb_q8_0_get_rows(ctx.h, w.h, ctx.array(ids).ptr, len(ids), out.ptr, cols))
    assert np.array_equal(out.download(), ref)
    w.free()


@pytest.mark.parametrize("M", [1, 4, 16])
def test_q8_0_matmul_through_the_backend_dispatch(qb, orc, ctx, rb, M):
    """q8_0_matmul as the reference backend dispatches it for this row count (its own activation quantisation and kernel
    choice).  For 1 and 4 rows it runs the matvec kernel, which the oracle restates bit for bit (matmul_mmvq); that kernel
    quantises activations as round(x / d), the MMQ family (and our engine, at every row count) as round(x * (127 / amax)),
    so a few int8 values differ by one step and the products by ~1e-4 of the output scale."""
    rng = np.random.default_rng(800 + M)
    N, K = 1024, 5120
    blocks = orc.quantize_q8_0(rng.normal(0, 0.02, (N, K)).astype(np.float32))
    x = rng.standard_normal((M, K)).astype(np.float32)
    t_out = rb.empty(M * N)
    rb.call("q8_0_matmul", t_out, rb.weight_q8_0(blocks, N, K), rb.tensor(x), M, K, N)
    ref = rb.download(t_out, (M, N))
    scale = float(np.abs(ref).max())
    exact = [bool(np.array_equal(f(blocks, N, K, x), ref)) for f in (orc.matmul_mmvq, orc.matmul_mmq)]
    want = orc.matmul_engine(blocks, N, K, x)
    if M <= 4:
        assert exact[0], "the oracle's matvec restatement is not the kernel the backend ran"
    if not any(exact):
        assert err(want, ref) < 2e-5 * scale, (err(want, ref), scale)
    w = qb.Weight.from_blocks(ctx, blocks, N, K)
    y = ctx.empty((M, N), np.float32)
    qb.binding.check(qb.lib().qb_q8_0_matmul(ctx.h, w.h, ctx.array(x).ptr, M, K, y.ptr, N, 0, 0))
    got = y.download()
    assert np.array_equal(got, want)
    assert err(got, ref) < (1e-3 if M <= 4 else 2e-5) * scale, (err(got, ref), scale, exact)
    w.free()


@pytest.mark.parametrize("M", [1, 4])
def test_ffn_input_silu_mul(qb, orc, ctx, rb, M):
    """h = silu(W_gate x) * (W_up x) as the reference backend computes it for Q8_0 weights (q8_0_matvec_silu_mul for one
    row; two q8_0_matmul + silu_mul_n for verifier rows: its batched fused form takes FP8 pairs only) against ours, which
    leaves h quantised for the down projection: compared after dequantisation, to half a quantisation step of each
    32-block plus the activation-rounding difference described in the test above."""
    rng = np.random.default_rng(900 + M)
    F, K = 2048, 5120
    gate = orc.quantize_q8_0(rng.normal(0, 0.02, (F, K)).astype(np.float32))
    up = orc.quantize_q8_0(rng.normal(0, 0.02, (F, K)).astype(np.float32))
    x = rng.standard_normal((M, K)).astype(np.float32)
    t_out, t_x = rb.empty(M * F), rb.tensor(x)
    w_g, w_u = rb.weight_q8_0(gate, F, K), rb.weight_q8_0(up, F, K)
    if M == 1:
        rb.call("q8_0_matvec_silu_mul", t_out, w_g, w_u, t_x)
    else:
        t_g, t_u = rb.empty(M * F), rb.empty(M * F)
        rb.call("q8_0_matmul", t_g, w_g, t_x, M, K, F)
        rb.call("q8_0_matmul", t_u, w_u, t_x, M, K, F)
        rb.call("silu_mul_n", t_out, t_g, t_u, M * F)
    ref = rb.download(t_out, (M, F))
    big = float(np.abs(ref).max())
    g, u = orc.matmul_mmvq(gate, F, K, x), orc.matmul_mmvq(up, F, K, x)
    want = (g / (np.float32(1) + np.exp(-g, dtype=np.float32)) * u).astype(np.float32)
    assert np.allclose(want, ref, rtol=1e-5, atol=1e-6 * big), err(want, ref)
    h = C.c_void_p()
    vp = qb.binding.vp
    qb.binding.check(qb.lib().qb_weight_q8_0_gate_up(ctx.h, gate.ctypes.data_as(vp), up.ctypes.data_as(vp), F, K, C.byref(h)))
    ld = (M + 3) // 4 * 4
    hq, hd_ = ctx.empty((M, F), np.int8), ctx.empty((F // 32, ld), np.float32)
    qb.binding.check(qb.lib().qb_q8_0_matmul_silu_mul_q8(ctx.h, h, ctx.array(x).ptr, M, K, hq.ptr, hd_.ptr, 0))
    ctx.sync()
    q, d = hq.download().astype(np.float32), hd_.download()
    deq = (q.reshape(M, F // 32, 32) * d.T[:M, :, None]).reshape(M, F)
    step = np.repeat(d.T[:M], 32, axis=1)
    assert np.all(np.abs(deq - ref) <= 0.5 * step * 1.001 + 2e-3 * big), err(deq, ref)
    qb.lib().qb_weight_free(ctx.h, h)
