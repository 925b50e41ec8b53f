"""The reference's own engine as the end-to-end comparator: a seeded synthetic GGUF checkpoint is read by the reference
(its GGUF reader, tokenizer, QwenExecutor, native backend generate loops on its CUDA DeviceBackend, built from the
reference sources into oracle/_ref/qw3ref_engine), by the product (qb_model_load_gguf) and by the CPU oracle; greedy
decoding and the MTP speculative loop (draft chain, 4-row verify, acceptance, checkpoint restore, MTP prefix) are
compared on the token streams and on the counters of the reference's `native mtp_spec_summary:` / `mtp_accept_hist:`
lines.  Skipped when the comparator has not been built (it needs the reference tree)."""
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, top2_margin

sys.path.insert(0, os.path.join(ROOT, "oracle"))
pytestmark = pytest.mark.gpu
ENGINE = os.path.join(ROOT, "oracle", "_ref", "qw3ref_engine")
K, N_NEW, PROMPT_LEN, CTX = 3, 48, 40, 512


def pin_config(qb):
    """Reduced 27B-class shape: the head sizes the reference's kernels are written for (attention 256, DeltaNet 128),
    4 layers (DeltaNet x3 + full attention) and one MTP layer; small enough for a file of a few tens of MB."""
    return qb.ModelConfig(n_layers=4, n_embd=1024, n_ff=2048, n_heads=8, n_kv_heads=2, head_dim=256, rope_dim=64,
                          rope_theta=1e7, rms_eps=1e-6, ssm_conv_kernel=4, ssm_num_k_heads=4, ssm_num_v_heads=8,
                          ssm_head_dim=128, full_attention_interval=4, vocab_size=4096, mtp_layers=1, weight_sigma=0.02)


def run_reference(path, mode, prompt, n_new, sampling=None):
    import gguf_synth as G
    env = dict(os.environ, QW3_PAGED_KV_PREFILL="0", QW3_Q8_BF16_MAIN="0", QW3_FATTN_NSPLIT="1")
    for key, v in (sampling or {}).items():          # temperature, top_p, top_k, min_p, seed (see oracle/ref_engine_main.cpp)
        env["QW3REF_" + key.upper()] = repr(v)
    cmd = [ENGINE, path, mode, str(K), str(n_new), str(CTX)] + [str(int(t)) for t in prompt]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, "reference engine failed:\n" + r.stderr[-3000:]
    m = re.search(r"^QW3REF_TEXT (.*)$", r.stdout, re.M)
    assert m, r.stdout[-2000:]
    toks = G.parse_token_text(m.group(1).strip())
    log = r.stderr + r.stdout
    summary, hist = parse_summary(log)
    return toks, summary, hist, log


def parse_summary(log):
    """The `native mtp_spec_summary:` / `native mtp_accept_hist:` lines of a log (the reference's, or the product's
    Batch.spec_summary_lines())."""
    summary = {}
    sm = re.search(r"native mtp_spec_summary:(.*)", log)
    if sm:
        summary = dict(kv.split("=", 1) for kv in sm.group(1).split() if "=" in kv)
    hm = re.search(r"native mtp_accept_hist:(.*)", log)
    hist = [int(v.split("=")[1]) for v in hm.group(1).split()] if hm else None
    return summary, hist


def engine_streams(qb, model, prompt, n_new):
    """(greedy tokens, speculative tokens, accepted length per step) of the product with the reference's chain policy:
    depth min(K, tokens still wanted)."""
    g = qb.Batch(model, 1, CTX, 0)
    g.prefill(0, prompt)
    greedy = list(g.read_output()[0])
    while len(greedy) < n_new:
        g.greedy_step()
        greedy += g.read_output()[0]
    g.close()
    b = qb.Batch(model, 1, CTX, K)
    b.prefill(0, prompt)
    spec, acc = list(b.read_output()[0]), []
    while len(spec) < n_new:
        b.set_draft_policy([max(1, min(K, n_new - len(spec)))])
        b.mtp_step()
        t = b.read_output()[0]
        acc.append(len(t) - 1)
        spec += t
    st = b.stats()
    st["summary"], st["hist"] = parse_summary("\n".join(b.spec_summary_lines()))
    b.close()
    return greedy[:n_new], spec[:n_new], acc, st


def oracle_streams(orc, om, prompt, n_new):
    s = orc.Seq(om, CTX)
    s.prefill(prompt, 0)
    greedy, margins = [s.cur_token], [top2_margin(s.last_logits(1)[0])]
    while len(greedy) < n_new:
        s.greedy_step()
        greedy.append(s.cur_token)
        margins.append(top2_margin(s.last_logits(1)[0]))
    s = orc.Seq(om, CTX)
    s.prefill(prompt, 0)
    spec, acc = [s.cur_token], []
    while len(spec) < n_new:
        out, _, _ = s.mtp_step(max(1, min(K, n_new - len(spec))))
        acc.append(len(out) - 1)
        spec += out
    return greedy, margins, spec[:n_new], acc


def common_prefix(a, b):
    n = 0
    while n < min(len(a), len(b)) and a[n] == b[n]:
        n += 1
    return n


@pytest.mark.skipif(not os.path.exists(ENGINE), reason="oracle/_ref/qw3ref_engine not built (make -C oracle ref-engine REF=<reference tree>)")
@pytest.mark.parametrize("predictable", [False, True])
def test_reference_engine_greedy_and_mtp(qb, orc, ctx, tmp_path, predictable):
    """predictable = False: the seeded model with random gains (MTP acceptance ~ 0: pins the greedy path and that a
    rejecting speculative loop is lossless).  predictable = True: residual branches scaled down and eh_proj = [I | 0] + noise,
    which gives the untrained MTP head a real acceptance rate, so the accepted-length histogram depends on the whole
    wiring of the head."""
    import gguf_synth as G
    cfg = pin_config(qb)
    ocfg = orc.ModelConfig(**cfg.as_dict())
    kw = dict(gain_sigma=0.05, branch_scale=0.01, eh_identity=True) if predictable else dict(gain_sigma=0.1)
    t = G.seeded_model_tensors(ocfg, 0x5EED + int(predictable), **kw)
    path = G.write_gguf(str(tmp_path / "pin.gguf"), ocfg, t, context_length=CTX)
    prompt = orc.synth_prompt(4242, cfg.vocab_size, PROMPT_LEN)

    model = qb.Model.from_gguf(ctx, path)
    e_greedy, e_spec, e_acc, e_stats = engine_streams(qb, model, prompt, N_NEW)
    model.close()
    assert e_spec == e_greedy                                          # lossless on the product itself
    o_greedy, o_margin, o_spec, o_acc = oracle_streams(orc, orc.Model.from_tensors(ocfg, t), prompt, N_NEW)

    r_greedy, _, _, log_g = run_reference(path, "greedy", prompt, N_NEW)
    r_spec, summ, hist, log_m = run_reference(path, "mtp", prompt, N_NEW)
    print("reference greedy  :", r_greedy[:16], "...")
    print("product greedy    :", e_greedy[:16], "...")
    print("reference summary :", {k_: summ.get(k_) for k_ in ("batches", "drafted", "accepted", "rejected", "rollbacks")}, "hist", hist)
    print("product           : steps %d drafted %d accepted %d, accepted lengths %s" % (len(e_acc), e_stats["drafted"], e_stats["accepted"], np.bincount(e_acc, minlength=K + 1).tolist()))
    print("oracle            : accepted lengths %s" % np.bincount(o_acc, minlength=K + 1).tolist())

    # greedy: the three streams agree up to the first position where the oracle's top-2 margin is inside the numeric
    # differences of the implementations (the reference quantises matvec activations as round(x/d), its attention is fp32)
    n_ro = common_prefix(r_greedy, o_greedy)
    n_re = common_prefix(r_greedy, e_greedy)
    print("greedy agreement: reference/oracle %d, reference/product %d of %d tokens" % (n_ro, n_re, N_NEW))
    assert len(r_greedy) == N_NEW
    assert n_ro >= 8 and n_re >= 8
    if n_ro < N_NEW:
        assert o_margin[n_ro] < 2e-2, (n_ro, o_margin[n_ro])
    n_eo = common_prefix(e_greedy, o_greedy)
    if n_eo < N_NEW:
        assert o_margin[n_eo] < 2e-2, (n_eo, o_margin[n_eo])
    # the reference's own speculative loop is lossless against its own greedy decode
    assert r_spec == r_greedy
    # counters of the speculative loop
    assert summ.get("enabled") == "true" and hist is not None
    r_batches, r_drafted, r_accepted = int(summ["batches"]), int(summ["drafted"]), int(summ["accepted"])
    assert sum(hist) == r_batches
    if n_re == N_NEW:
        # same token stream: the step structure must be the same too
        assert r_batches == len(e_acc) and r_drafted == e_stats["drafted"]
        # the product's own summary lines, read by the same parser: same step structure, field by field
        for key in ("enabled", "batches", "drafted"):
            assert e_stats["summary"][key] == summ[key], key
        if r_accepted == e_stats["accepted"]:
            assert e_stats["hist"] == hist and e_stats["summary"]["rejected"] == summ["rejected"]
        tol = max(2, r_drafted // 10)
        assert abs(r_accepted - e_stats["accepted"]) <= tol
        assert abs(r_accepted - sum(o_acc)) <= tol
    if predictable:
        assert r_accepted >= r_drafted // 5, "the predictable model should accept a good share of its drafts"
        assert e_stats["accepted"] >= e_stats["drafted"] // 5


@pytest.mark.skipif(not os.path.exists(ENGINE), reason="oracle/_ref/qw3ref_engine not built (make -C oracle ref-engine REF=<reference tree>)")
def test_reference_engine_sampled_mtp(qb, orc, ctx, tmp_path):
    """A sampling request (temperature > 0) through the reference's speculative loop and through the product's, on the
    same generator: the reference seeds one std::mt19937_64 per request with options.seed; the product is handed that
    generator's draws (oracle/ref_sampling.py replays the engine and libstdc++'s conversion to a uniform) through a
    DrawQueue -- the first draw picks the token after the prompt, a step is handed k + 1 and returns the unused ones.
    While both implementations see the same logits up to their numeric noise, the two token streams are the same; a
    draw that lands inside that noise at a boundary of the cumulative distribution ends the common prefix (from there on
    the two requests are different texts).  The sampler's functions themselves are pinned bit-exactly on the reference
    in tests/test_sampling_ref_pin_cpu.py; this test pins the order in which the loop consumes the generator."""
    import gguf_synth as G
    import ref_sampling as R
    cfg = pin_config(qb)
    ocfg = orc.ModelConfig(**cfg.as_dict())
    t = G.seeded_model_tensors(ocfg, 0x5EED + 1, gain_sigma=0.05, branch_scale=0.01, eh_identity=True)
    path = G.write_gguf(str(tmp_path / "pin_s.gguf"), ocfg, t, context_length=CTX)
    prompt = orc.synth_prompt(4242, cfg.vocab_size, PROMPT_LEN)
    model = qb.Model.from_gguf(ctx, path)
    temp, top_p, top_k = 0.7, 1.0, 6
    prefixes, n_new = [], 32
    for seed in (11, 12, 13, 14):
        r_tok, summ, hist, _ = run_reference(path, "mtp", prompt, n_new, dict(temperature=temp, top_p=top_p, top_k=top_k, seed=seed))
        assert len(r_tok) == n_new and summ.get("enabled") == "true"
        b = qb.Batch(model, 1, CTX, K)
        dq = qb.serve.DrawQueue(R.MT64(seed), K + 1)
        b.prefill_sampled(0, prompt, dq.take(), temp, top_p, top_k)
        e_tok, e_acc = list(b.read_output()[0]), []
        while len(e_tok) < n_new:
            depth = max(1, min(K, n_new - len(e_tok)))
            b.set_draft_policy([depth])
            b.mtp_step_sampled(np.array([dq.peek()], np.float64), temp, top_p, top_k)
            out = b.read_output()[0]
            dq.consume_step(len(out), depth)
            e_acc.append(len(out) - 1)
            e_tok += out
        b.close()
        n = common_prefix(r_tok, e_tok[:n_new])
        prefixes.append(n)
        print("seed %d: common prefix %d of %d; reference hist %s accepted %s/%s; product accepted lengths %s"
              % (seed, n, n_new, hist, summ.get("accepted"), summ.get("drafted"), np.bincount(e_acc, minlength=K + 1).tolist()))
    model.close()
    # a wrong draw order would break every stream within its first step or two; numeric noise breaks one only where a
    # draw falls next to a boundary
    # (measured: all four requests equal to the reference's for all 32 tokens, accepted-length histograms equal)
    assert sorted(prefixes)[1] == n_new and min(prefixes) >= 4, prefixes
