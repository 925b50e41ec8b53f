"""GPU parity tests of the attention, DeltaNet, norm and argmax kernels through the C ABI."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_rms_norm(qb, orc, ctx):
    rng = np.random.default_rng(20)
    x = rng.standard_normal((5, 5120)).astype(np.float32) * 3
    w = rng.uniform(0.5, 1.5, 5120).astype(np.float32)
    out = ctx.empty(x.shape, np.float32)
    qb.binding.check(qb.lib().qb_rms_norm(ctx.h, ctx.array(x).ptr, ctx.array(w).ptr, 5, 5120, 5120, 1e-6, out.ptr))
    got, want = out.download(), orc.rms_norm(x, w, 1e-6)
    assert np.allclose(got, want, rtol=5e-6, atol=1e-6), float(np.abs(got - want).max())


def test_argmax_rows_ties_and_edges(qb, orc, ctx):
    rng = np.random.default_rng(21)
    x = rng.standard_normal((6, 151936)).astype(np.float32)
    x[1, [5, 150000]] = 9.0          # tie: lowest index wins
    x[2, 151935] = 10.0              # last element
    x[3, :] = -2.0                   # all equal
    x[4, 0] = 11.0
    out = ctx.empty(6, np.int32)
    qb.binding.check(qb.lib().qb_argmax_rows(ctx.h, ctx.array(x).ptr, 6, 151936, 151936, out.ptr))
    assert out.download().tolist() == orc.argmax_rows(x).tolist()


def _attn_case(qb, orc, ctx, n_heads, n_kv, hd, rope_dim, page_size, seq_base, R, order, seed):
    rng = np.random.default_rng(seed)
    n_seqs = len(seq_base)
    max_pos = max(seq_base) + R
    pps = (max_pos + page_size) // page_size + 1
    total_pages = n_seqs * pps
    perm = np.arange(total_pages, dtype=np.int32)
    if order == "reverse":
        perm = perm[::-1].copy()
    elif order == "shuffle":
        rng.shuffle(perm)
    pt = perm.reshape(n_seqs, pps)
    kvd = n_kv * hd
    stride = n_heads * 2 * hd + 2 * kvd
    kc = np.zeros((total_pages * page_size, kvd), np.uint16)
    vc = np.zeros_like(kc)
    invf = orc.inv_freq(rope_dim, 1e7)
    qw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    kw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    # history: fill every sequence's past positions through the oracle's append
    for s in range(n_seqs):
        if seq_base[s] == 0:
            continue
        hist = rng.standard_normal((seq_base[s], stride)).astype(np.float32)
        orc.qk_norm_rope_append(hist, qw, kw, invf, n_heads, n_kv, hd, rope_dim, 1e-6, np.full(seq_base[s], s, np.int32),
                                np.arange(seq_base[s], dtype=np.int32), pt, page_size, kc, vc)
    rows = n_seqs * R
    qkv = rng.standard_normal((rows, stride)).astype(np.float32)
    row_seq = np.repeat(np.arange(n_seqs, dtype=np.int32), R)
    row_pos = (np.repeat(np.array(seq_base, np.int32), R) + np.tile(np.arange(R, dtype=np.int32), n_seqs)).astype(np.int32)
    # GPU
    d_qkv, d_kc, d_vc, d_pt = ctx.array(qkv), ctx.array(kc), ctx.array(vc), ctx.array(pt)
    d_pos = ctx.array(np.array(seq_base, np.int32))
    L = qb.lib()
    qb.binding.check(L.qb_qk_norm_rope_append(ctx.h, d_qkv.ptr, rows, stride, ctx.array(qw).ptr, ctx.array(kw).ptr,
                                              ctx.array(invf).ptr, n_heads, n_kv, hd, rope_dim, 1e-6, d_pos.ptr, n_seqs,
                                              d_pt.ptr, pps, page_size, d_kc.ptr, d_vc.ptr))
    out = ctx.empty((rows, n_heads * hd), np.float32)
    qb.binding.check(L.qb_attention_paged_gated(ctx.h, d_qkv.ptr, rows, stride, n_heads, n_kv, hd, d_pos.ptr, n_seqs,
                                                d_pt.ptr, pps, page_size, d_kc.ptr, d_vc.ptr, max_pos, out.ptr))
    got = out.download()
    # oracle
    o_qkv = qkv.copy()
    orc.qk_norm_rope_append(o_qkv, qw, kw, invf, n_heads, n_kv, hd, rope_dim, 1e-6, row_seq, row_pos, pt, page_size, kc, vc)
    want = orc.attention_paged_gated(o_qkv, n_heads, n_kv, hd, row_seq, row_pos, pt, page_size, kc, vc)
    # q after norm+rope, and the cache rows written by this call
    assert np.allclose(d_qkv.download()[:, :n_heads * 2 * hd], o_qkv[:, :n_heads * 2 * hd], rtol=2e-5, atol=2e-5)
    gk, gv = d_kc.download(), d_vc.download()
    assert np.allclose(gk.view(np.float16).astype(np.float32), kc.view(np.float16).astype(np.float32), rtol=2e-3, atol=1e-3)
    assert np.array_equal(gv, vc)      # K within an fp16 ulp or two (device rsqrt / sincos), V exact
    # the kernel multiplies fp16 operands (q and the probabilities are rounded to fp16, as on the reference's
    # FlashInfer path, whose OUTPUT is fp16 as well: ulp 1e-3 for values in [1, 2)) with fp32 accumulation; the
    # oracle keeps q and p in fp32
    assert np.allclose(got, want, rtol=2e-3, atol=1e-3), float(np.abs(got - want).max())
    return got


@pytest.mark.parametrize("order", ["identity", "reverse", "shuffle"])
def test_attention_verify_rows_27b_heads(qb, orc, ctx, order):
    """4 verify rows, 24 q / 4 kv heads x 256, page 16; context crosses split (256) and tile (64) edges."""
    got = _attn_case(qb, orc, ctx, 24, 4, 256, 64, 16, [0, 61, 255, 700], 4, order, seed=30)
    assert np.isfinite(got).all()


def test_attention_page_order_invariance(qb, orc, ctx):
    """Identical output bits under identity / reverse / shuffled page tables
    (the reference's paged_kv_regression idea)."""
    a = _attn_case(qb, orc, ctx, 4, 2, 64, 16, 16, [300, 5], 2, "identity", seed=31)
    b = _attn_case(qb, orc, ctx, 4, 2, 64, 16, 16, [300, 5], 2, "reverse", seed=31)
    assert np.array_equal(a, b)


def test_attention_single_row_and_tiny_heads(qb, orc, ctx):
    _attn_case(qb, orc, ctx, 4, 2, 64, 16, 16, [0], 1, "identity", seed=32)        # first token, one key
    _attn_case(qb, orc, ctx, 4, 2, 64, 16, 32, [129, 1000], 1, "shuffle", seed=33)  # page size 32
    _attn_case(qb, orc, ctx, 16, 2, 128, 32, 16, [257], 5, "identity", seed=34)     # GQA 8, 5 rows (k=4)


@pytest.mark.parametrize("n_heads,n_kv,hd,base,R", [(24, 4, 256, 700, 45), (4, 2, 64, 130, 70), (16, 2, 128, 0, 33)])
def test_attention_prompt_chunk_shape_has_the_bits_of_the_verify_shape(qb, orc, ctx, monkeypatch, n_heads, n_kv, hd, base, R):
    """A prompt chunk (many rows of one sequence) runs the 64-query shape of the attention kernel, decode and verify
    rows the 32-query shape; a row must get the same bits from either, or a request's tokens would depend on how its
    prompt was cut into chunks.  The chunk's rows are recomputed four at a time and compared bit for bit; the chunk
    itself is checked against the oracle by _attn_case."""
    _attn_case(qb, orc, ctx, n_heads, n_kv, hd, 16 if hd == 64 else 64, 16, [base], R, "shuffle", seed=70 + R)
    monkeypatch.setenv("QW3B200_ATTN_TC", "0")       # the four-row calls below on the mma.sync shape, not on the tcgen05 kernel
    rng = np.random.default_rng(90 + R)
    page_size, rope_dim = 16, 16 if hd == 64 else 64
    max_pos = base + R
    pps = (max_pos + page_size) // page_size + 1
    pt = rng.permutation(pps).astype(np.int32).reshape(1, pps)
    kvd = n_kv * hd
    stride = n_heads * 2 * hd + 2 * kvd
    kc = np.zeros((pps * page_size, kvd), np.uint16)
    vc = np.zeros_like(kc)
    invf = orc.inv_freq(rope_dim, 1e7)
    qw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    kw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    if base:
        hist = rng.standard_normal((base, stride)).astype(np.float32)
        orc.qk_norm_rope_append(hist, qw, kw, invf, n_heads, n_kv, hd, rope_dim, 1e-6, np.zeros(base, np.int32),
                                np.arange(base, dtype=np.int32), pt, page_size, kc, vc)
    qkv = rng.standard_normal((R, stride)).astype(np.float32)
    d_qkv, d_kc, d_vc, d_pt = ctx.array(qkv), ctx.array(kc), ctx.array(vc), ctx.array(pt)
    L = qb.lib()
    qb.binding.check(L.qb_qk_norm_rope_append(ctx.h, d_qkv.ptr, R, stride, ctx.array(qw).ptr, ctx.array(kw).ptr, ctx.array(invf).ptr,
                                              n_heads, n_kv, hd, rope_dim, 1e-6, ctx.array(np.array([base], np.int32)).ptr, 1,
                                              d_pt.ptr, pps, page_size, d_kc.ptr, d_vc.ptr))
    wide = ctx.empty((R, n_heads * hd), np.float32)
    qb.binding.check(L.qb_attention_paged_gated(ctx.h, d_qkv.ptr, R, stride, n_heads, n_kv, hd, ctx.array(np.array([base], np.int32)).ptr, 1,
                                                d_pt.ptr, pps, page_size, d_kc.ptr, d_vc.ptr, max_pos, wide.ptr))
    want = wide.download()
    normed = d_qkv.download()
    for r0 in range(0, R, 4):
        n = min(4, R - r0)
        part = ctx.array(np.ascontiguousarray(normed[r0:r0 + n]))
        out = ctx.empty((n, n_heads * hd), np.float32)
        qb.binding.check(L.qb_attention_paged_gated(ctx.h, part.ptr, n, stride, n_heads, n_kv, hd, ctx.array(np.array([base + r0], np.int32)).ptr, 1,
                                                    d_pt.ptr, pps, page_size, d_kc.ptr, d_vc.ptr, max_pos, out.ptr))
        assert np.array_equal(out.download(), want[r0:r0 + n]), r0


@pytest.mark.parametrize("n_heads,n_kv,hd,bases,R", [(24, 4, 256, [0, 61, 255, 700, 3000], 4), (16, 2, 128, [257, 1, 1023], 5),
                                                    (24, 4, 256, [9000], 1), (8, 4, 128, [130, 511], 8)])
def test_attention_tensor_memory_kernel_vs_mma_sync_kernel(qb, orc, ctx, monkeypatch, n_heads, n_kv, hd, bases, R):
    """Decode / verify rows run the tcgen05 kernel (keys as the MMA's M, S and O in tensor memory, TMA-fed); the same
    call on the mma.sync kernel (QW3B200_ATTN_TC=0) must agree within the fp16 rounding of the probabilities, and both are
    checked against the oracle by _attn_case (contexts that end inside a tile, inside a split, and span many splits)."""
    got_tc = _attn_case(qb, orc, ctx, n_heads, n_kv, hd, 64, 16, bases, R, "shuffle", seed=120 + R)
    monkeypatch.setenv("QW3B200_ATTN_TC", "0")
    got_mma = _attn_case(qb, orc, ctx, n_heads, n_kv, hd, 64, 16, bases, R, "shuffle", seed=120 + R)
    assert np.allclose(got_tc, got_mma, rtol=2e-3, atol=1e-3), float(np.abs(got_tc - got_mma).max())


def _dn_inputs(rng, nk, nv, hd, n_seqs, R, n_slots):
    C_ = (2 * nk + nv) * hd
    stride = C_ + nv * hd + 2 * nv + 3    # a padded row stride
    proj = rng.standard_normal((n_seqs * R, stride)).astype(np.float32)
    conv_w = rng.uniform(-0.5, 0.5, (C_, 4)).astype(np.float32)
    ssm_a = (-np.exp(rng.uniform(0, np.log(16), nv))).astype(np.float32)
    dt = rng.uniform(-4, -1, nv).astype(np.float32)
    nw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    state = (rng.standard_normal((n_seqs, n_slots, nv, hd, hd)) * 0.05).astype(np.float32)
    conv = rng.standard_normal((n_seqs, n_slots, C_, 3)).astype(np.float32)
    return proj, conv_w, ssm_a, dt, nw, state, conv


@pytest.mark.parametrize("nk,nv,hd,n_seqs,R,write_all", [(16, 48, 128, 1, 4, True), (2, 4, 64, 3, 2, True),
                                                         (16, 48, 128, 2, 1, False), (2, 4, 64, 1, 37, False)])
def test_deltanet_rows_vs_oracle(qb, orc, ctx, nk, nv, hd, n_seqs, R, write_all):
    rng = np.random.default_rng(40 + R)
    n_slots = max(R, 4) if write_all else 4
    proj, conv_w, ssm_a, dt, nw, state, conv = _dn_inputs(rng, nk, nv, hd, n_seqs, R, n_slots)
    slot_in = rng.integers(0, n_slots, n_seqs).astype(np.int32)
    d_state, d_conv = ctx.array(state), ctx.array(conv)
    core = ctx.empty((n_seqs * R, nv * hd), np.float32)
    qb.binding.check(qb.lib().qb_deltanet_rows(ctx.h, ctx.array(proj).ptr, n_seqs, R, proj.shape[1], ctx.array(conv_w).ptr,
                                               ctx.array(ssm_a).ptr, ctx.array(dt).ptr, ctx.array(nw).ptr, nk, nv, hd, 1e-6,
                                               d_state.ptr, d_conv.ptr, n_slots, ctx.array(slot_in).ptr, 1 if write_all else 0,
                                               core.ptr))
    got_core, got_state, got_conv = core.download(), d_state.download(), d_conv.download()
    for s in range(n_seqs):
        st, cv = state[s].copy(), conv[s].copy()
        want = orc.deltanet_rows(proj[s * R:(s + 1) * R], conv_w, ssm_a, dt, nw, nk, nv, hd, 1e-6, st, cv, int(slot_in[s]), write_all)
        assert np.allclose(got_core[s * R:(s + 1) * R], want, rtol=2e-3, atol=2e-4)
        assert np.allclose(got_state[s], st, rtol=1e-3, atol=1e-4)
        assert np.allclose(got_conv[s], cv, rtol=0, atol=0)      # the conv window is a pure shift of inputs


def test_reference_gated_delta_net_kernel_matches_oracle_rule(qb, orc, ctx, ref):
    """Pins the oracle's delta rule on the reference's gated_delta_net.cu (compiled for sm_100a):
    same inputs (already convolved / normalised q,k,v), same state and checkpoints."""
    if ref is None:
        pytest.skip("oracle/_ref not built")
    rng = np.random.default_rng(50)
    nk, nv, hd, T = 16, 48, 128, 4
    C_ = (2 * nk + nv) * hd
    # feed the oracle inputs for which conv+silu+l2norm are easy to undo: use its own intermediate by
    # running the product kernel's fp32 path is not possible, so compare rule-only: craft conv weights
    # that pass the current sample through (w = [0,0,0,1]) and compare against silu/l2norm done in numpy.
    proj = rng.standard_normal((T, C_ + nv * hd + 2 * nv)).astype(np.float32)
    conv_w = np.zeros((C_, 4), np.float32); conv_w[:, 3] = 1.0
    ssm_a = (-np.exp(rng.uniform(0, np.log(16), nv))).astype(np.float32)
    dt = rng.uniform(-4, -1, nv).astype(np.float32)
    nw = np.ones(hd, np.float32)
    state0 = (rng.standard_normal((T, nv, hd, hd)) * 0.05).astype(np.float32)
    conv0 = np.zeros((T, C_, 3), np.float32)
    # oracle: full layer with checkpoints, but we only compare state (norm-gate does not touch it)
    st, cv = state0.copy(), conv0.copy()
    orc.deltanet_rows(proj, conv_w, ssm_a, dt, nw, nk, nv, hd, 1e-6, st, cv, 0, True)
    # reference kernel on numpy-prepared q,k,v
    x = proj[:, :C_].astype(np.float64)
    x = (x / (1.0 + np.exp(-x))).astype(np.float32)
    qk = x[:, :2 * nk * hd].reshape(T, 2 * nk, hd)
    qk = qk / np.sqrt((qk.astype(np.float64) ** 2).sum(-1, keepdims=True) + 1e-6).astype(np.float32)
    x[:, :2 * nk * hd] = qk.reshape(T, -1)
    alpha = proj[:, C_ + nv * hd:C_ + nv * hd + nv].copy()
    beta = proj[:, C_ + nv * hd + nv:C_ + nv * hd + 2 * nv].copy()
    d_state = ctx.array(state0[0])
    d_ck = ctx.empty((T, nv, hd, hd), np.float32)
    d_core = ctx.empty((T, nv * hd), np.float32)
    rc = ref.ref_gated_delta_net(ctx.array(alpha).ptr, ctx.array(beta).ptr, ctx.array(dt).ptr, ctx.array(ssm_a).ptr,
                                 ctx.array(x).ptr, C.c_uint32(0), C.c_uint32(nk * hd), C.c_uint32(2 * nk * hd), d_state.ptr,
                                 d_core.ptr, C.c_uint32(T), C.c_uint32(nk), C.c_uint32(nv), C.c_uint32(hd), C.c_uint32(C_),
                                 C.c_uint32(nv), C.c_uint32(nv * hd), d_ck.ptr, C.c_uint32(T))
    assert rc == 0
    ck = d_ck.download()
    for t in range(T):
        assert np.allclose(ck[t], st[t], rtol=1e-3, atol=1e-5), t
    assert np.allclose(d_state.download(), st[T - 1], rtol=1e-3, atol=1e-5)
