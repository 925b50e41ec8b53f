"""CPU tests: the oracle against the reference's known answers, its own golden fixtures and itself."""
import os

import numpy as np
import pytest

from conftest import std_mt19937_uniform, tiny_ocfg

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_f16_roundtrip_matches_numpy(orc):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(20000) * 10.0 ** rng.integers(-8, 5, 20000)).astype(np.float32)
    w = np.zeros((len(x) // 32, 32), np.float32)
    w[:, 0] = x[: len(x) // 32]
    # scale of each block is amax/127 stored as fp16: compare with numpy's round-to-nearest-even
    blocks = orc.quantize_q8_0(w).reshape(-1, 34)
    d_bits = blocks[:, :2].copy().view(np.uint16)[:, 0]
    want = (np.abs(w[:, 0]) / np.float32(127.0)).astype(np.float16).view(np.uint16)
    assert np.array_equal(d_bits, want)


def test_q8_0_quantiser_matches_reference_host_recipe(orc):
    """tests/mmq_parity.cu:54-80: d = amax/127, q = clamp(lrint(x / d))."""
    rng = np.random.default_rng(2)
    w = rng.uniform(-0.5, 0.5, (8, 256)).astype(np.float32)
    blocks = orc.quantize_q8_0(w).reshape(-1, 34)
    q = blocks[:, 2:].view(np.int8).reshape(8, 256)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32).reshape(8, 8)
    wb = w.reshape(8, 8, 32)
    dd = (np.abs(wb).max(-1) / np.float32(127.0)).astype(np.float32)
    want_q = np.clip(np.rint(wb * (np.float32(1.0) / dd)[..., None]), -127, 127).astype(np.int8).reshape(8, 256)
    assert np.array_equal(q, want_q)
    assert np.array_equal(d, dd.astype(np.float16).astype(np.float32))
    deq = orc.dequant_q8_0(blocks.reshape(-1), 8, 256)
    assert np.allclose(deq, w, atol=float(dd.max()) * 0.6)   # half a step + the fp16 rounding of d


def test_split_plane_repack(orc):
    """src/cuda_helpers.cuh:16-39: per row all fp16 scales, then all quants."""
    rng = np.random.default_rng(3)
    blocks = orc.quantize_q8_0(rng.standard_normal((4, 128)).astype(np.float32))
    sp = orc.repack_split_plane(blocks, 4, 128).reshape(4, 4 * 34)
    b = blocks.reshape(4, 4, 34)
    for r in range(4):
        assert np.array_equal(sp[r, :8], b[r, :, :2].reshape(-1))
        assert np.array_equal(sp[r, 8:], b[r, :, 2:].reshape(-1))


def test_activation_quantisers(orc):
    """src/mmvq_q8.cu:98-111 (q8_1) and :694-721 (q8_1_mmq)."""
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, 256)).astype(np.float32)
    x[1, 32:64] = 0.0   # an all-zero block
    q, d = orc.quantize_act(x)
    xb = x.reshape(3, 8, 32)
    amax = np.abs(xb).max(-1)
    with np.errstate(divide="ignore", invalid="ignore"):
        d_inv = np.where(amax == 0, np.float32(0), np.float32(127.0) / amax).astype(np.float32)
        want_d = np.where(amax == 0, np.float32(0), np.float32(1.0) / d_inv).astype(np.float32)
    want_q = np.rint(xb * d_inv[..., None]).astype(np.int8).reshape(3, 256)
    assert np.array_equal(q, want_q)
    assert np.array_equal(d.T, want_d)
    mmq = orc.quantize_q8_1_mmq(x).reshape(2, 3, 144)
    for sb in range(2):
        for m in range(3):
            assert np.array_equal(mmq[sb, m, :16].copy().view(np.float32), want_d[m, sb * 4:sb * 4 + 4])
            assert np.array_equal(mmq[sb, m, 16:].view(np.int8), want_q[m, sb * 128:(sb + 1) * 128])
    q81 = orc.quantize_q8_1(x).reshape(3, 8, 36)
    d81 = (amax / np.float32(127.0)).astype(np.float32)
    assert np.array_equal(q81[:, :, :2].copy().view(np.float16)[..., 0], d81.astype(np.float16))
    with np.errstate(divide="ignore", invalid="ignore"):
        want81 = np.where(amax[..., None] == 0, 0, np.rint(xb / d81[..., None])).astype(np.int8)
    assert np.array_equal(q81[:, :, 4:].view(np.int8), want81)


def test_closed_forms_of_reference_backend_test(orc):
    """tests/mixed_linear_parity.cu:204-281: scale 0.5, quants 1, x constant -> y = cols*0.5*x."""
    g = np.load(os.path.join(GOLD, "closed_forms.npz"))
    rows, cols = int(g["rows"]), int(g["cols"])
    blocks = np.zeros((rows * (cols // 32), 34), np.uint8)
    blocks[:, 0:2] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    blocks[:, 2:] = 1
    x = np.repeat(g["x_first_col"][:, None], cols, 1)
    for fn in (orc.matmul_engine, orc.matmul_mmq):
        y = fn(blocks.reshape(-1), rows, cols, x)
        assert np.allclose(y, g["expected"][:, None], rtol=0.01, atol=0.25)   # the reference's tolerance
        assert np.allclose(y, g["expected"][:, None], rtol=1e-6)              # and in fact exact to fp32
    y = orc.matmul_mmvq(blocks.reshape(-1), rows, cols, x[:4])
    assert np.allclose(y, g["expected"][:4, None], rtol=2e-3)                 # fp16 activation scale
    assert np.array_equal(orc.matmul_engine(blocks.reshape(-1), rows, cols, x)[:, 0], g["oracle_y_col0"])


MMQ_PARITY_SHAPES = [(128, 128, 256), (128, 128, 1024), (128, 128, 2048), (256, 128, 2048), (128, 256, 2048),
                     (256, 256, 1024), (384, 256, 2048), (2048, 2048, 2048), (2304, 2048, 2304), (640, 2048, 2304),
                     (2048, 2048, 2304), (2304, 2271, 2304), (2048, 2271, 2304), (2304, 223, 2304), (2048, 223, 2304),
                     (640, 223, 2304)]


def test_mmq_parity_procedure(orc):
    """The reference's GEMM parity test (tests/mmq_parity.cu:137-254) run on the oracle: inputs from
    std::mt19937(0x5eed), W~U(-.5,.5), X~U(-1,1); compare with an fp32 product of the dequantised
    operands the kernel sees; tolerance 5e-3 abs or 1e-3 rel.  The small and the tail shapes run here,
    the 2048-row ones on the GPU."""
    rs = np.random.RandomState(0x5EED)
    for (M, N, K) in MMQ_PARITY_SHAPES:
        W = std_mt19937_uniform(rs, M * K, -0.5, 0.5).reshape(M, K)
        X = std_mt19937_uniform(rs, N * K, -1.0, 1.0).reshape(N, K)
        if M * N * K > 400e6:
            continue
        blocks = orc.quantize_q8_0(W)
        Wd = orc.dequant_q8_0(blocks, M, K)
        q, d = orc.quantize_act(X)
        Xd = q.astype(np.float32).reshape(N, K // 32, 32) * d.T[..., None]
        ref = Xd.reshape(N, K).astype(np.float64) @ Wd.T.astype(np.float64)
        for fn in (orc.matmul_mmq, orc.matmul_engine):
            got = fn(blocks, M, K, X)
            diff = np.abs(got - ref)
            bad = (diff > 5e-3) & (diff > 1e-3 * np.maximum(np.abs(ref), 1e-6))
            assert not bad.any(), (M, N, K, float(diff.max()))


def test_block_dots_and_orders_agree(orc):
    rng = np.random.default_rng(5)
    N, K, M = 160, 512, 5
    blocks = orc.quantize_q8_0((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((M, K)).astype(np.float32)
    q, d = orc.quantize_act(x)
    dots = orc.block_dots(blocks, N, K, q)
    wq = blocks.reshape(N, K // 32, 34)[:, :, 2:].view(np.int8).astype(np.int64)
    want = np.einsum("nbt,mbt->mnb", wq, q.reshape(M, K // 32, 32).astype(np.int64))
    assert np.array_equal(dots, want.astype(np.int32))
    wd = blocks.reshape(N, K // 32, 34)[:, :, :2].copy().view(np.float16)[..., 0].astype(np.float32)
    # engine order with one segment == the MMQ order on the same scales
    y1 = orc.gemm_engine(blocks, N, K, q, d, ksplit=1)
    y_mmq = orc.matmul_mmq(blocks, N, K, x)
    assert np.array_equal(y1, y_mmq)
    # split partials add up in ascending order
    y4, parts = orc.gemm_engine(blocks, N, K, q, d, ksplit=4, want_partials=True)
    acc = parts[0].copy()
    for s in range(1, 4):
        acc = acc + parts[s]
    assert np.array_equal(acc, y4)
    exact = np.einsum("mnb,nb,bm->mn", want.astype(np.float64), wd.astype(np.float64), d.astype(np.float64))
    for y in (y1, y4):
        assert np.allclose(y, exact, rtol=1e-4, atol=1e-5)
    # the mmvq path quantises the activations differently (fp16 scale, x/d rounding): same product
    # up to that quantisation noise
    assert np.allclose(orc.matmul_mmvq(blocks, N, K, x), exact, rtol=2e-2, atol=5e-3)


def test_ksplit_policy_is_shape_only(orc, qb):
    for (N, K) in [(5120, 6144), (5120, 17408), (14336, 5120), (34816, 5120), (151936, 5120), (5120, 10240), (256, 256), (768, 256)]:
        S = orc.ksplit_policy(N, K)
        assert 1 <= S <= 8 and S <= K // 128
        assert S == qb.lib().qb_ksplit_policy(N, K)   # host function of the library, no GPU needed


def test_argmax_tie_break(orc):
    x = np.zeros((3, 100), np.float32)
    x[0, [7, 50]] = 3.0
    x[1, 99] = 1.0
    x[2, :] = -1.0
    assert orc.argmax_rows(x).tolist() == [7, 99, 0]


def test_deltanet_checkpoints_equal_stepwise(orc):
    """State after row t written in checkpoint mode == state after t+1 single-row calls
    (src/gated_delta_net.cu:165-176)."""
    rng = np.random.default_rng(6)
    nk, nv, hd, T = 2, 4, 64, 4
    C = (2 * nk + nv) * hd
    stride = C + nv * hd + 2 * nv
    proj = rng.standard_normal((T, stride)).astype(np.float32)
    conv_w = rng.uniform(-0.5, 0.5, (C, 4)).astype(np.float32)
    ssm_a = -np.exp(rng.uniform(0, np.log(16), nv)).astype(np.float32)
    dt = rng.uniform(-4, -1, nv).astype(np.float32)
    nw = np.ones(hd, np.float32)
    st0 = (rng.standard_normal((T, nv, hd, hd)) * 0.1).astype(np.float32)
    cv0 = rng.standard_normal((T, C, 3)).astype(np.float32)
    st_a, cv_a = st0.copy(), cv0.copy()
    core_a = orc.deltanet_rows(proj, conv_w, ssm_a, dt, nw, nk, nv, hd, 1e-6, st_a, cv_a, slot_in=2, write_all=True)
    st_b, cv_b = st0.copy(), cv0.copy()
    st_b[0], cv_b[0] = st0[2], cv0[2]
    for t in range(T):
        core_t = orc.deltanet_rows(proj[t:t + 1], conv_w, ssm_a, dt, nw, nk, nv, hd, 1e-6, st_b, cv_b, slot_in=0, write_all=False)
        assert np.array_equal(core_t[0], core_a[t])
        assert np.array_equal(st_b[0], st_a[t]) and np.array_equal(cv_b[0], cv_a[t])


def test_golden_tiny_streams_and_losslessness(orc, qb):
    """Config 1: greedy stream, MTP k=1 stream and first logits of the oracle match the committed
    fixture; speculative == greedy (lossless) for k=1 and for forced 70% drafts at k=3."""
    g = np.load(os.path.join(GOLD, "tiny_streams.npz"))
    m = orc.Model(tiny_ocfg(orc, qb), qb.configs.MODEL_SEED)
    prompt = orc.synth_prompt(qb.configs.PROMPT_SEED + 1, 4096, 64)
    assert np.array_equal(prompt, g["prompt"])
    s = orc.Seq(m, 256)
    s.prefill(prompt, 16)    # chunking must not matter
    lg = s.last_logits(1)[0]
    assert int(np.argmax(lg)) == int(g["logits0_argmax"])
    assert np.allclose(lg[::64], g["logits0_sample"], rtol=1e-4, atol=1e-5)
    greedy = [s.cur_token]
    while len(greedy) < 32:
        greedy.append(s.greedy_step())
    assert greedy == g["greedy"].tolist()
    s2 = orc.Seq(m, 256)
    s2.prefill(prompt, 64)
    out = [s2.cur_token]
    while len(out) < 32:
        out += s2.mtp_step(1)[0]
    assert out[:32] == greedy == g["mtp_k1"].tolist()
    # forced drafts at k=3: draft i is the true continuation with probability 0.7
    rng = np.random.default_rng(7)
    s3 = orc.Seq(m, 256)
    s3.prefill(prompt, 64)
    out = [s3.cur_token]
    accepted = 0
    while len(out) < 28:
        base = len(out)
        forced = [greedy[base + i] if (base + i < 32 and rng.random() < 0.7) else 1 for i in range(3)]
        toks, _, _ = s3.mtp_step(3, forced)
        accepted += len(toks) - 1
        out += toks
    assert out[:28] == greedy[:28] and accepted > 0


def _np_distribution(l, temp, top_p, top_k, min_p):
    """Independent numpy statement of the sampling distribution (stable descending order)."""
    n = len(l)
    e = np.exp(((l - l.max()) * np.float32(1.0 / temp)).astype(np.float32)).astype(np.float32)
    p = (e * np.float32(1.0 / e.astype(np.float64).sum())).astype(np.float32)
    if not ((0 < top_k < n) or (0 < top_p < 1) or min_p > 0):
        return p
    order = np.argsort(-l.astype(np.float64), kind="stable")
    keep = top_k if 0 < top_k < n else n
    if min_p > 0:
        keep = min(keep, int((p[order] >= p[order[0]] * np.float32(min_p)).sum()))
    if 0 < top_p < 1:
        cum = np.cumsum(p[order[:keep]].astype(np.float64))
        hit = np.nonzero(cum >= np.float32(top_p))[0]
        if len(hit):
            keep = int(hit[0]) + 1
    out = np.zeros(n, np.float32)
    ks = p[order[:keep]].astype(np.float64).sum()
    out[order[:keep]] = p[order[:keep]] * np.float32(1.0 / ks)
    return out


@pytest.mark.parametrize("temp,top_p,top_k,min_p", [(1.0, 1.0, 0, 0.0), (0.7, 0.9, 0, 0.0), (0.5, 1.0, 5, 0.0), (1.3, 0.8, 50, 0.05),
                                                     (0.2, 0.0, 0, 0.3), (1.0, 0.5, 1, 0.0), (1.0, 1e-6, 0, 0.0), (1.0, 1.0, 10**9, 0.0)])
def test_sampling_acceptance_oracle(orc, temp, top_p, top_k, min_p):
    """The oracle's sampling-mode acceptance against an independent numpy statement: p[draft], the accept decision, and the
    inverse-CDF draw over the nonzero entries in index order."""
    rng = np.random.default_rng(17)
    rows, V = 12, 3000
    x = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    x[3, 100] = x[3, 2000] = x[3].max() + 1          # a tie at the top
    draft = np.where(np.arange(rows) % 3 == 2, -1, x.argmax(1)).astype(np.int32)
    draft[4] = 7                                      # an unlikely draft
    ua, ur = rng.random(rows), rng.random(rows)
    tok, acc, pd = orc.sample_rows(x, draft, ua, ur, temp, top_p, top_k, min_p)
    for r in range(rows):
        p = _np_distribution(x[r], temp, top_p, top_k, min_p)
        assert abs(p.astype(np.float64).sum() - 1) < 1e-4
        d = int(draft[r])
        if d >= 0:
            assert np.isclose(pd[r], p[d], rtol=1e-5, atol=1e-9)
            assert acc[r] == int(ua[r] < p[d])
            if acc[r]:
                assert tok[r] == d
                continue
            p[d] = 0
        nz = np.nonzero(p > 0)[0]
        if len(nz) == 0:
            assert tok[r] == d
            continue
        cp = np.cumsum(p[nz].astype(np.float64) / p[nz].astype(np.float64).sum())
        cp[-1] = 1.0
        want = nz[np.searchsorted(cp, ur[r], side="left")]
        assert tok[r] == want, (r, tok[r], want)
        assert d < 0 or tok[r] != d
