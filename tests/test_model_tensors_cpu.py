"""CPU tests of the checkpoint path: the synthetic GGUF writer (test infrastructure) against the product's GGUF
parser, the oracle built from named tensors against the seeded oracle model, and the noise floor of the tiny model."""
import os
import struct
import sys

import numpy as np
import pytest

from conftest import ROOT, tiny_ocfg

sys.path.insert(0, os.path.join(ROOT, "oracle"))


@pytest.fixture(scope="module")
def G(orc):
    import gguf_synth
    return gguf_synth


def test_gguf_writer_and_product_parser_agree(qb, orc, G, tmp_path):
    ocfg = tiny_ocfg(orc, qb)
    t = G.seeded_model_tensors(ocfg, 0x5EED, gain_sigma=0.1)
    path = G.write_gguf(str(tmp_path / "tiny.gguf"), ocfg, t)
    cfg, n, nbytes = qb.binding.gguf_read_config(path)
    want = qb.configs.tiny().as_dict()
    got = cfg.as_dict()
    for key in want:
        if key == "weight_sigma":
            continue
        assert got[key] == pytest.approx(want[key]), key
    assert n == len(t) and nbytes == sum(a.nbytes for a in t.values())


def test_gguf_parser_rejects_bad_files(qb, orc, G, tmp_path):
    ocfg = tiny_ocfg(orc, qb)
    t = {"output_norm.weight": np.ones(ocfg.n_embd, np.float32)}
    path = G.write_gguf(str(tmp_path / "a.gguf"), ocfg, t)
    raw = open(path, "rb").read()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"XXXX" + raw[4:])
    with pytest.raises(qb.QbError, match="magic"):
        qb.binding.gguf_read_config(str(bad))
    bad.write_bytes(raw[:4] + struct.pack("<I", 2) + raw[8:])
    with pytest.raises(qb.QbError, match="version"):
        qb.binding.gguf_read_config(str(bad))
    bad.write_bytes(raw[:200])
    with pytest.raises(qb.QbError):
        qb.binding.gguf_read_config(str(bad))
    bad.write_bytes(raw.replace(b"qwen35.ssm.group_count", b"qwen35.ssm.group_counx"))
    with pytest.raises(qb.QbError, match="ssm.group_count"):
        qb.binding.gguf_read_config(str(bad))
    bad.write_bytes(raw[:8] + struct.pack("<Q", 2 ** 61) + raw[16:])          # an absurd tensor count
    with pytest.raises(qb.QbError, match="more tensors"):
        qb.binding.gguf_read_config(str(bad))
    with pytest.raises(qb.QbError, match="cannot open"):
        qb.binding.gguf_read_config(str(tmp_path / "missing.gguf"))


def test_oracle_from_named_tensors_equals_seeded_model(qb, orc, G):
    """The seeded model written out as named tensors (unit gains) and bound by name gives the seeded model's bits:
    prefill logits and the logits of speculative steps."""
    ocfg = tiny_ocfg(orc, qb)
    a = orc.Model(ocfg, qb.configs.MODEL_SEED)
    b = orc.Model.from_tensors(ocfg, G.seeded_model_tensors(ocfg, qb.configs.MODEL_SEED))
    prompt = orc.synth_prompt(5, ocfg.vocab_size, 40)
    got = []
    for m in (a, b):
        s = orc.Seq(m, 128)
        s.prefill(prompt, 0)
        lg = [s.last_logits(1).copy()]
        for _ in range(3):
            s.mtp_step(1)
            lg.append(s.last_logits(2).copy())
        got.append(lg)
    for x, y in zip(*got):
        assert np.array_equal(x, y)
    with pytest.raises(RuntimeError):
        t = G.seeded_model_tensors(ocfg, 1)
        del t["blk.1.ssm_a"]
        orc.Model.from_tensors(ocfg, t)


def test_gain_vectors_are_bound_to_their_own_norms(qb, orc, G):
    """Every gain vector matters: changing any one of them changes the logits of a speculative step."""
    ocfg = tiny_ocfg(orc, qb)
    base = G.seeded_model_tensors(ocfg, 3, gain_sigma=0.1)
    prompt = orc.synth_prompt(6, ocfg.vocab_size, 24)

    def run(t):
        s = orc.Seq(orc.Model.from_tensors(ocfg, t), 64)
        s.prefill(prompt, 0)
        drafts = []
        for _ in range(8):
            drafts += s.mtp_step(3)[1]
        return s.last_logits(4).copy(), drafts

    ref_lg, ref_drafts = run(base)
    L = ocfg.n_layers
    for name in ["blk.0.attn_norm.weight", "blk.0.ffn_norm.weight", "blk.0.ssm_norm.weight", "blk.3.attn_q_norm.weight", "blk.3.attn_k_norm.weight",
                 "output_norm.weight", "blk.%d.nextn.enorm.weight" % L, "blk.%d.nextn.hnorm.weight" % L,
                 "blk.%d.nextn.shared_head_norm.weight" % L, "blk.%d.attn_norm.weight" % L]:
        t = dict(base)
        t[name] = (base[name] * np.where(np.arange(base[name].size) % 2, 3.0, 1.0 / 3.0)).astype(np.float32)
        lg, drafts = run(t)
        assert not np.array_equal(lg, ref_lg) or drafts != ref_drafts, name


def test_tiny_model_noise_floor_under_one_ulp(qb, orc):
    """How far the logits of the 256-wide tiny model move when every attn_norm gain of layer 0 moves by one unit in
    the last place: the activations are re-quantised to int8 before every projection, so the change flips rounding
    decisions and the two runs differ by the rounding noise itself.  Any fp32 implementation that is not the same
    instruction sequence sits somewhere inside this band; a bound below it cannot be tested on this model."""
    ocfg = tiny_ocfg(orc, qb)
    prompt = orc.synth_prompt(qb.configs.PROMPT_SEED + 1, ocfg.vocab_size, 64)
    m = orc.Model(ocfg, qb.configs.MODEL_SEED)
    a = orc.Seq(m, 256)
    a.prefill(prompt, 64)
    la = [a.last_logits(1)[0].copy()]
    toks = [a.cur_token]
    for _ in range(31):
        a.greedy_step()
        la.append(a.last_logits(1)[0].copy())
        toks.append(a.cur_token)
    m.nudge_attn_norm(0, 1)
    b = orc.Seq(m, 256)
    b.prefill(prompt, 64)
    errs = []
    for i in range(32):
        if i:
            b.greedy_step()
        lb = b.last_logits(1)[0]
        errs.append(float(np.abs(lb - la[i]).max() / np.abs(la[i]).max()))
        b.set_cur_token(toks[i])
    print("tiny model, one-ulp nudge of one norm: logit max-rel-err max %.3g mean %.3g" % (max(errs), float(np.mean(errs))))
    assert 1e-4 < max(errs) < 0.2
