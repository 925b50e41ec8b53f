"""Paged gated attention alone at a given context (27B-class heads: 24 q / 4 kv x 256, page 16, 4 verify rows):
split + merge timed with CUDA events, cold L2 before every call.

    ATT_CTX=2048,32768 ATT_R=4 python kvmem-qw3_b200/attn_probe.py
"""
import os, sys
import numpy as np
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as entry
pkg = entry.load_package()
ctx = pkg.Context(0)
L = pkg.lib()
n_heads, n_kv, hd, page = 24, 4, 256, 16
R = int(os.environ.get("ATT_R", "4"))
for ctxlen in [int(v) for v in os.environ.get("ATT_CTX", "2048,32768").split(",")]:
    max_pos = ctxlen + R
    pps = (max_pos + page) // page + 1
    pt = np.arange(pps, dtype=np.int32).reshape(1, pps)
    kvd = n_kv * hd
    rng = np.random.default_rng(1)
    kc = (rng.standard_normal((pps * page, kvd)) * 0.5).astype(np.float16)
    vc = (rng.standard_normal((pps * page, kvd)) * 0.5).astype(np.float16)
    stride = n_heads * 2 * hd + 2 * kvd
    qkv = rng.standard_normal((R, stride)).astype(np.float32)
    d_qkv, d_kc, d_vc, d_pt = ctx.array(qkv), ctx.array(kc.view(np.uint16)), ctx.array(vc.view(np.uint16)), ctx.array(pt)
    d_pos = ctx.array(np.array([ctxlen], np.int32))
    out = ctx.empty((R, n_heads * hd), np.float32)
    e0, e1 = ctx.event(), ctx.event()
    ts = []
    for it in range(8):
        ctx.flush_l2()
        ctx.record(e0)
        pkg.binding.check(L.qb_attention_paged_gated(ctx.h, d_qkv.ptr, R, stride, n_heads, n_kv, hd, d_pos.ptr, 1,
                                                    d_pt.ptr, pps, page, d_kc.ptr, d_vc.ptr, max_pos, out.ptr))
        ctx.record(e1)
        ctx.sync()
        ts.append(ctx.elapsed_ms(e0, e1) * 1e3)
    kvbytes = ctxlen * kvd * 2 * 2
    us = float(np.median(ts[2:]))
    print("ctx %d R %d: split+merge %.1f us, KV %.1f MB -> %.0f GB/s" % (ctxlen, R, us, kvbytes / 1e6, kvbytes / us / 1e3), flush=True)
    ctx.release_arrays()
