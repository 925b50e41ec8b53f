"""The product behind the reference's own operator interface: B200DeviceBackend (kvmem-qw3_b200/shim/b200_device_backend.cpp,
a qw3::DeviceBackend subclass over the C ABI, compiled against include/qw3/device_backend.hpp) and the reference's CUDA
DeviceBackend are driven through the SAME virtual calls by the same C driver (oracle/ref_backend_shim.cpp) on the same
inputs; results are compared with each other and with the oracle.  Skipped when the libraries have not been built
(`make -C oracle ref-backend b200-backend REF=<reference tree>`)."""
import os
import sys

import numpy as np
import pytest

from conftest import ROOT

sys.path.insert(0, os.path.join(ROOT, "oracle"))
import ref_backend as RB  # noqa: E402

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (os.path.exists(RB.PATH) and os.path.exists(RB.B200_PATH)), reason="oracle/_ref backends not built")]


@pytest.fixture(scope="module")
def backends():
    ref, mine = RB.RefBackend(1, RB.PATH), RB.RefBackend(1, RB.B200_PATH)
    assert mine.name() == "b200"
    yield ref, mine
    ref.close(); mine.close()


@pytest.fixture(autouse=True)
def _release(backends):
    yield
    for b in backends:
        b.release()


def scale_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.mark.parametrize("M", [1, 4, 16])
def test_q8_0_matmul_and_matvec_family(orc, backends, M):
    N, K = 1024, 2048
    rng = np.random.default_rng(M)
    blocks = orc.quantize_q8_0((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((M, K)).astype(np.float32)
    outs = []
    for be in backends:
        w, tx, ty = be.weight_q8_0(blocks, N, K), be.tensor(x), be.empty(M * N)
        be.call("q8_0_matmul", ty, w, tx, M, K, N)
        outs.append(be.download(ty, (M, N)))
    ref, got = outs
    # the reference's own bound between its matvec and MMQ kernels (tests/vmed_bench.cu:92-117): 2e-2 of the output scale
    assert scale_err(got, ref) < 2e-2
    assert np.array_equal(got, orc.matmul_engine(blocks, N, K, x))          # the product's arithmetic, bit for bit
    if M == 1:
        res = []
        for be in backends:
            w, tx = be.weight_q8_0(blocks, N, K), be.tensor(x[0])
            ty, acc = be.empty(N), be.tensor(np.full(N, 0.5, np.float32))
            be.call("q8_0_matvec", ty, w, tx)
            be.call("q8_0_matvec_add", acc, w, tx)
            res.append((be.download(ty, (N,)), be.download(acc, (N,))))
        assert scale_err(res[1][0], res[0][0]) < 2e-2 and scale_err(res[1][1], res[0][1]) < 2e-2
        assert np.array_equal(res[1][1], np.float32(0.5) + res[1][0])


def test_norms_elementwise_get_rows_argmax(orc, backends):
    rng = np.random.default_rng(7)
    M, n = 5, 5120
    x = rng.standard_normal((M, n)).astype(np.float32)
    g = rng.uniform(0.5, 1.5, n).astype(np.float32)
    a, b = rng.standard_normal(3000).astype(np.float32), rng.standard_normal(3000).astype(np.float32)
    V = 9000
    logits = rng.standard_normal((3, V)).astype(np.float32)
    logits[1, 77] = logits[1, 4000] = 9.0                                   # a tie: the lowest index wins
    blocks = orc.quantize_q8_0((rng.standard_normal((64, 256)) * 0.02).astype(np.float32))
    rows = np.array([5, 63, 0, 5], np.uint64)
    left, right = rng.standard_normal((3, 40)).astype(np.float32), rng.standard_normal((3, 48)).astype(np.float32)
    first, hb = rng.standard_normal(32).astype(np.float32), rng.standard_normal((2, 32)).astype(np.float32)
    res = []
    for be in backends:
        tn = be.empty(M * n)
        be.call("rms_norm_batch", tn, be.tensor(x), be.weight_f32(g), M, n, 1e-6)
        ts, ta = be.empty(3000), be.empty(3000)
        be.call("silu_mul_n", ts, be.tensor(a), be.tensor(b), 3000)
        be.call("add_n", ta, be.tensor(a), be.tensor(b), 3000)
        tok, val = np.zeros(3, np.int32), np.zeros(3, np.float32)
        be.call("argmax_batch", be.tensor(logits), 3, V, tok.ctypes.data, val.ctypes.data)
        t1, v1 = RB.C.c_int32(), RB.C.c_float()
        be.call("argmax_to_buffer_roundtrip", be.tensor(logits[2]), 4, 2, RB.C.byref(t1), RB.C.byref(v1))
        tg = be.empty(4 * 256)
        be.call("q8_0_get_rows_batch", tg, be.weight_q8_0(blocks, 64, 256), rows.ctypes.data, 4)
        tc = be.empty(3 * 70)
        be.call("pack_mtp_concat", tc, be.tensor(left), be.tensor(right), 3, 40, 48, 70, 32)
        tp = be.empty(3 * 32)
        be.call("pack_mtp_prefix_hinputs", tp, be.tensor(first), be.tensor(hb), 3, 32)
        res.append(dict(norm=be.download(tn, (M, n)), silu=be.download(ts, (3000,)), add=be.download(ta, (3000,)), tok=tok.copy(), val=val.copy(),
                        t1=(t1.value, v1.value), rows=be.download(tg, (4, 256)), cat=be.download(tc, (3, 70))[:, :64], pre=be.download(tp, (3, 32)),
                        cat_want=np.concatenate([left[:, :32], right[:, :32]], 1), pre_want=np.concatenate([first[None], hb], 0)))
    ref, got = res
    assert np.allclose(got["norm"], ref["norm"], rtol=1e-5, atol=1e-6)
    assert np.allclose(got["silu"], ref["silu"], rtol=1e-6, atol=1e-7) and np.array_equal(got["add"], ref["add"])
    assert got["tok"].tolist() == ref["tok"].tolist() == [int(np.argmax(logits[0])), 77, int(np.argmax(logits[2]))]
    assert np.array_equal(got["val"], ref["val"])
    assert got["t1"] == ref["t1"] == (int(np.argmax(logits[2])), float(logits[2].max()))
    assert np.array_equal(got["rows"], ref["rows"])
    for r in res:
        assert np.array_equal(r["cat"], r["cat_want"]) and np.array_equal(r["pre"], r["pre_want"])


@pytest.mark.parametrize("n_heads,n_kv,hd,base,R", [(24, 4, 256, 700, 4), (16, 2, 128, 300, 3)])
def test_attention_chain_through_the_interface(orc, backends, n_heads, n_kv, hd, base, R):
    """rmsnorm_per_head_batch -> rope_partial_batch -> kv_append_batch -> attention_decode_batch_gated on both backends
    (dense fp16 cache), then the paged calls (kv_append_batch_paged_device, attention_decode_batch_paged_gated_device,
    which the reference only has behind FlashInfer) on the product's backend with a shuffled page list: the paged result
    must equal its own dense result bit for bit."""
    rng = np.random.default_rng(base)
    T, kvd, qd = base + R, n_kv * hd, n_heads * 2 * hd
    rope_dim, theta, eps = hd // 4, 1e7, 1e-6
    qw, kw = rng.uniform(0.5, 1.5, hd).astype(np.float32), rng.uniform(0.5, 1.5, hd).astype(np.float32)
    q = rng.standard_normal((T, qd)).astype(np.float32)
    k = rng.standard_normal((T, kvd)).astype(np.float32)
    v = rng.standard_normal((T, kvd)).astype(np.float32)
    outs, caches = [], []
    for be in backends:
        tq, tk, tv = be.tensor(q), be.tensor(k), be.tensor(v)
        be.call("rmsnorm_per_head_batch", tq, be.weight_f32(qw), T, qd, n_heads, 2 * hd, hd, eps)
        be.call("rmsnorm_per_head_batch", tk, be.weight_f32(kw), T, kvd, n_kv, hd, hd, eps)
        be.call("rope_partial_batch", tq, T, qd, n_heads, 2 * hd, rope_dim, 0, theta)
        be.call("rope_partial_batch", tk, T, kvd, n_kv, hd, rope_dim, 0, theta)
        kc, vc = be.empty((T + 16) * kvd, kind=1), be.empty((T + 16) * kvd, kind=1)
        be.call("kv_append_batch", kc, tk, 0, kvd, T)
        be.call("kv_append_batch", vc, tv, 0, kvd, T)
        caches.append((be.download(tq, (T, qd)), be.download(kc, (T + 16, kvd), np.uint16), be.download(vc, (T + 16, kvd), np.uint16)))
    (rq, rkc, rvc), (gq, gkc, gvc) = caches
    assert np.array_equal(gvc[:T], rvc[:T])                                   # V: a conversion only
    ang = base * 1.2e-6 + 2e-5                                                # drift of the reference's fast-math RoPE per position
    assert scale_err(gq, rq) < 8 * ang + 1e-5
    # attention of the last R rows on identical inputs (the product's q and caches go into both backends)
    for be in backends:
        tq = be.tensor(np.ascontiguousarray(gq[base:]))
        kc, vc = be.tensor(gkc, kind=1), be.tensor(gvc, kind=1)
        to = be.empty(R * n_heads * hd)
        be.call("attention_decode_batch_gated", to, tq, 2 * hd, kc, vc, n_heads, n_kv, hd, base, R, qd, n_heads * hd, float(1.0 / np.sqrt(hd)))
        outs.append(be.download(to, (R, n_heads * hd)))
    ref, got = outs
    assert np.allclose(got, ref, rtol=2e-3, atol=1e-3), scale_err(got, ref)     # fp16 q and p on the product's side
    # paged form on the product's backend
    mine = backends[1]
    page = 16
    n_pages = (T + page - 1) // page + 1
    perm = np.random.default_rng(1).permutation(n_pages).astype(np.int32)
    tk2, tv2 = mine.tensor(np.ascontiguousarray(gkc[:T].view(np.float16).astype(np.float32))), mine.tensor(np.ascontiguousarray(gvc[:T].view(np.float16).astype(np.float32)))
    kc, vc = mine.empty(n_pages * page * kvd, kind=1), mine.empty(n_pages * page * kvd, kind=1)
    tp = mine.tensor(perm, kind=2)
    mine.call("kv_append_batch_paged_device", kc, tk2, 0, kvd, T, tp, n_pages, page)
    mine.call("kv_append_batch_paged_device", vc, tv2, 0, kvd, T, tp, n_pages, page)
    to = mine.empty(R * n_heads * hd)
    mine.call("attention_decode_batch_paged_gated_device", to, mine.tensor(np.ascontiguousarray(gq[base:])), 2 * hd, kc, vc, tp, n_pages, page,
              n_heads, n_kv, hd, base, R, qd, n_heads * hd, float(1.0 / np.sqrt(hd)))
    assert np.array_equal(mine.download(to, (R, n_heads * hd)), got)


@pytest.mark.parametrize("rows", [1, 4])
def test_recurrent_batch_with_checkpoints(orc, backends, rows):
    nk, nv, hd = 16, 48, 128
    C, vdim = (2 * nk + nv) * hd, nv * hd
    rng = np.random.default_rng(50 + rows)
    proj = (rng.standard_normal((rows, C)) * 0.5).astype(np.float32)
    z = rng.standard_normal((rows, vdim)).astype(np.float32)
    alpha, beta = rng.standard_normal((rows, nv)).astype(np.float32), rng.standard_normal((rows, nv)).astype(np.float32)
    conv_w = ((rng.random((C, 4)) * 2 - 1) * 0.5).astype(np.float32)
    ssm_a = (-np.exp(rng.random(nv) * np.log(16.0))).astype(np.float32)
    dt = (-4 + 3 * rng.random(nv)).astype(np.float32)
    norm = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    state0 = (rng.standard_normal((nv, hd, hd)) * 0.1).astype(np.float32)
    conv0 = (rng.standard_normal((C, 3)) * 0.5).astype(np.float32)
    res = []
    for be in backends:
        t_state, t_conv = be.tensor(state0), be.tensor(conv0)
        t_core, t_cout = be.empty(rows * vdim), be.empty(rows * C)
        ck_s, ck_c = be.empty(rows * nv * hd * hd), be.empty(rows * C * 3)
        be.call("recurrent_batch", t_core, t_state, t_conv, t_cout, be.tensor(proj), be.tensor(z), be.tensor(alpha), be.tensor(beta),
                be.weight_f32(conv_w), be.weight_f32(ssm_a), be.weight_f32(dt), be.weight_f32(norm), rows, nk, nv, hd, hd, 4, C, C, vdim, nv, nv, vdim,
                1e-6, ck_s, ck_c, rows)
        res.append((be.download(t_core, (rows, vdim)), be.download(t_state, (nv, hd, hd)), be.download(t_conv, (C, 3)),
                    be.download(ck_s, (rows, nv, hd, hd)), be.download(ck_c, (rows, C, 3))))
    ref, got = res
    assert np.allclose(got[0], ref[0], rtol=2e-3, atol=2e-4), scale_err(got[0], ref[0])
    assert np.allclose(got[1], ref[1], rtol=1e-3, atol=1e-5) and np.array_equal(got[2], ref[2])
    assert np.allclose(got[3], ref[3], rtol=1e-3, atol=1e-5) and np.array_equal(got[4], ref[4])
    assert np.array_equal(got[3][rows - 1], got[1]) and np.array_equal(got[4][rows - 1], got[2])


def test_fused_norm_fanout_and_ffn_input(orc, backends):
    H, F, M = 1024, 2048, 4
    rng = np.random.default_rng(3)
    x = rng.standard_normal((M, H)).astype(np.float32)
    g = rng.uniform(0.5, 1.5, H).astype(np.float32)
    w0 = orc.quantize_q8_0((rng.standard_normal((F, H)) * 0.02).astype(np.float32))
    w1 = orc.quantize_q8_0((rng.standard_normal((F, H)) * 0.02).astype(np.float32))
    res = []
    for be in backends:
        tn, o0, o1 = be.empty(M * H), be.empty(M * F), be.empty(M * F)
        W0, W1 = be.weight_q8_0(w0, F, H), be.weight_q8_0(w1, F, H)
        try:
            be.call("rms_norm_q8_0_matmul_fanout2", tn, o0, o1, W0, W1, F, F, be.tensor(x), be.weight_f32(g), M, H, 1e-6)
            fan = (be.download(o0, (M, F)), be.download(o1, (M, F)))
        except RB.RefError:
            fan = None                       # the executor takes its unfused fallback when a backend declines
        th = be.empty(M * F)
        try:
            be.call("q8_0_matmul_silu_mul", th, W0, W1, be.tensor(x), M, H, F)
        except RB.RefError:                  # the reference declines the batched form for Q8_0: its executor's unfused fallback
            tg, tu = be.empty(M * F), be.empty(M * F)
            be.call("q8_0_matmul", tg, W0, be.tensor(x), M, H, F)
            be.call("q8_0_matmul", tu, W1, be.tensor(x), M, H, F)
            be.call("silu_mul_n", th, tg, tu, M * F)
        res.append((fan, be.download(th, (M, F))))
    ref, got = res
    assert got[0] is not None
    if ref[0] is not None:
        assert scale_err(got[0][0], ref[0][0]) < 2e-2 and scale_err(got[0][1], ref[0][1]) < 2e-2
    assert scale_err(got[1], ref[1]) < 2e-2
