"""Pins the paged gated attention on the reference's own native decode attention kernel
(launch_fattn_vec_decode_f16, src/fattn_vec_decode.cu:514-537, compiled for sm_100a into oracle/_ref): same q
(after the product's q/k norm + RoPE), same fp16 K/V cache (identity page table, so the paged cache IS the dense
[position][kv head][head_dim] cache the reference kernel reads), rows at consecutive positions.  The reference
kernel leaves the sigmoid gate to a second op (apply_attn_gate, src/kernels_cuda.cu:9448-9465): applied here in
numpy."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_heads,n_kv,hd,base,R", [(24, 4, 256, 700, 4), (24, 4, 256, 63, 1), (16, 2, 128, 300, 3), (24, 4, 256, 2500, 4)])
def test_paged_attention_matches_reference_native_decode_kernel(qb, orc, ctx, ref_attn, n_heads, n_kv, hd, base, R):
    if ref_attn is None:
        pytest.skip("oracle/_ref/libqw3ref_attn.so not built (make -C oracle ref-attn)")
    rng = np.random.default_rng(50 + base)
    page = 16
    max_pos = base + R
    pps = (max_pos + page) // page + 1
    pt = np.arange(pps, dtype=np.int32).reshape(1, pps)            # identity: slot = position
    kvd = n_kv * hd
    stride = n_heads * 2 * hd + 2 * kvd
    rope_dim = hd // 4
    invf = orc.inv_freq(rope_dim, 1e7)
    qw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    kw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    kc = np.zeros((pps * page, kvd), np.uint16)
    vc = np.zeros_like(kc)
    hist = rng.standard_normal((base, stride)).astype(np.float32)
    orc.qk_norm_rope_append(hist, qw, kw, invf, n_heads, n_kv, hd, rope_dim, 1e-6, np.zeros(base, np.int32),
                            np.arange(base, dtype=np.int32), pt, page, kc, vc)
    qkv = rng.standard_normal((R, stride)).astype(np.float32)
    d_qkv, d_kc, d_vc, d_pt = ctx.array(qkv), ctx.array(kc), ctx.array(vc), ctx.array(pt)
    d_pos = ctx.array(np.array([base], np.int32))
    L = qb.lib()
    qb.binding.check(L.qb_qk_norm_rope_append(ctx.h, d_qkv.ptr, R, stride, ctx.array(qw).ptr, ctx.array(kw).ptr, ctx.array(invf).ptr,
                                              n_heads, n_kv, hd, rope_dim, 1e-6, d_pos.ptr, 1, d_pt.ptr, pps, page, d_kc.ptr, d_vc.ptr))
    out = ctx.empty((R, n_heads * hd), np.float32)
    qb.binding.check(L.qb_attention_paged_gated(ctx.h, d_qkv.ptr, R, stride, n_heads, n_kv, hd, d_pos.ptr, 1, d_pt.ptr, pps, page,
                                                d_kc.ptr, d_vc.ptr, max_pos, out.ptr))
    ctx.sync()
    got = out.download()
    # the reference kernel on the same device buffers: row b attends keys [0, base + 1 + b)
    ref_out = ctx.empty((R, n_heads * hd), np.float32)
    rc = ref_attn.ref_fattn_vec_decode_f16(ref_out.ptr, d_qkv.ptr, C.c_uint32(2 * hd), d_kc.ptr, d_vc.ptr, C.c_uint32(n_heads),
                                           C.c_uint32(n_kv), C.c_uint32(hd), C.c_uint32(base + 1), C.c_uint32(R), C.c_uint32(stride),
                                           C.c_uint32(n_heads * hd), C.c_float(1.0 / np.sqrt(hd)))
    if rc == -1:
        pytest.skip("the reference launcher declines this head size")
    assert rc == 0
    q_after = d_qkv.download()[:, :n_heads * 2 * hd].reshape(R, n_heads, 2, hd)
    gate = q_after[:, :, 1, :].reshape(R, n_heads * hd)
    want = ref_out.download() * (1.0 / (1.0 + np.exp(-gate)))
    # fp16 operands on our side (q, p), fp32 q on the reference's: the bound of the oracle comparison
    assert np.allclose(got, want, rtol=2e-3, atol=1e-3), float(np.abs(got - want).max())
    # and the CPU oracle's restatement of the same math (fp32 q and p, fp16 K/V) is pinned on the reference kernel
    o_qkv = d_qkv.download()
    okc, ovc = d_kc.download(), d_vc.download()
    row_seq = np.zeros(R, np.int32)
    row_pos = (base + np.arange(R)).astype(np.int32)
    ours_cpu = orc.attention_paged_gated(o_qkv, n_heads, n_kv, hd, row_seq, row_pos, pt, page, okc, ovc)
    assert np.allclose(ours_cpu, want, rtol=1e-4, atol=2e-5), float(np.abs(ours_cpu - want).max())
