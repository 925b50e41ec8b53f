"""GPU tests of a model built from the caller's tensors (qb_model_create) and from a GGUF file (qb_model_load_gguf):
the seeded model as named tensors equals the seeded constructor bit for bit; a model with non-unit RMSNorm gains
matches the oracle built from the same tensors; the file path gives the bits of the in-memory path."""
import os
import sys

import numpy as np
import pytest

from conftest import ROOT, rel_err, tiny_ocfg, top2_margin

sys.path.insert(0, os.path.join(ROOT, "oracle"))
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G(orc):
    import gguf_synth
    return gguf_synth


def run_stream(qb, model, prompt, k, steps):
    """Prefill logits, then `steps` speculative steps: (logit blocks, drafts per step, emitted tokens)."""
    b = qb.Batch(model, 1, 256, k)
    b.prefill(0, prompt)
    lg, drafts, toks = [b.last_logits(1).copy()], [], list(b.read_output()[0])
    for _ in range(steps):
        b.mtp_draft()
        drafts.append(b.last_drafts()[0].tolist())
        b.mtp_verify()
        lg.append(b.last_logits(k + 1).copy())
        b.mtp_accept_commit()
        toks += b.read_output()[0]
    b.close()
    return lg, drafts, toks


def test_seeded_tensors_give_the_seeded_model_bits(qb, orc, ctx, G):
    cfg, ocfg = qb.configs.tiny(), tiny_ocfg(orc, qb)
    prompt = orc.synth_prompt(11, cfg.vocab_size, 48)
    a = qb.Model(ctx, cfg, qb.configs.MODEL_SEED)
    b = qb.Model.from_tensors(ctx, cfg, G.seeded_model_tensors(ocfg, qb.configs.MODEL_SEED))
    assert a.weight_bytes == b.weight_bytes
    ra, rb = run_stream(qb, a, prompt, 3, 4), run_stream(qb, b, prompt, 3, 4)
    assert ra[1] == rb[1] and ra[2] == rb[2]
    for x, y in zip(ra[0], rb[0]):
        assert np.array_equal(x, y)
    a.close(); b.close()


def test_model_with_gains_matches_oracle_and_gguf_path(qb, orc, ctx, G, tmp_path):
    """Non-unit gains on every norm (each vector its own draws): engine vs oracle from the same tensors, then the
    same model through a GGUF file must reproduce the in-memory model's bits."""
    cfg, ocfg = qb.configs.tiny(), tiny_ocfg(orc, qb)
    t = G.seeded_model_tensors(ocfg, 0xBEEF, gain_sigma=0.1)
    prompt = orc.synth_prompt(12, cfg.vocab_size, 40)
    model = qb.Model.from_tensors(ctx, cfg, t)
    om = orc.Model.from_tensors(ocfg, t)
    lg, drafts, toks = run_stream(qb, model, prompt, 3, 5)
    s = orc.Seq(om, 256)
    s.prefill(prompt, 0)
    e0 = rel_err(lg[0][0], s.last_logits(1)[0])
    assert e0 < 1e-2, e0
    assert toks[0] == s.cur_token or top2_margin(s.last_logits(1)[0]) < 2e-2
    s.set_cur_token(toks[0])
    worst, draft_agree, n_drafts = e0, 0, 0
    for step in range(5):
        otoks, odrafts, orows = s.mtp_step(3, drafts[step])          # the oracle verifies the GPU's drafts
        olg = s.last_logits(4)
        per_row = [rel_err(lg[step + 1][r], olg[r]) for r in range(4)]
        worst = max(worst, max(per_row))
        assert per_row[0] < 1e-2 and max(per_row) < 2.5e-2, (step, per_row)     # later rows: inside the tiny model's one-ulp noise band (1.6 % measured)
        rows = np.argmax(lg[step + 1], 1).tolist()
        if rows != orows:
            assert all(rows[r] == orows[r] or top2_margin(olg[r]) < 2e-2 for r in range(4))
            break
    # the MTP head's own drafts against the oracle's on a fresh sequence (first step: same inputs on both sides)
    s2 = orc.Seq(om, 256)
    s2.prefill(prompt, 0)
    s2.set_cur_token(toks[0])
    _, od, _ = s2.mtp_step(3)
    assert od == drafts[0], (od, drafts[0])
    print("gains model: worst logit rel err %.3g" % worst)

    path = G.write_gguf(str(tmp_path / "gains.gguf"), ocfg, t)
    fm = qb.Model.from_gguf(ctx, path)
    got = fm.cfg.as_dict()
    assert all(got[k] == pytest.approx(v) for k, v in cfg.as_dict().items() if k != "weight_sigma")
    lg2, drafts2, toks2 = run_stream(qb, fm, prompt, 3, 5)
    assert drafts2 == drafts and toks2 == toks
    for x, y in zip(lg, lg2):
        assert np.array_equal(x, y)
    model.close(); fm.close()


def test_one_checkpoint_file_feeds_tokenizer_and_model(qb, orc, ctx, G, tmp_path):
    """Text in, text out through one GGUF file: its token and merge tables build the tokenizer, its tensors the model; the
    stream of the text's ids equals the stream of the same ids on the model built from the tensors in memory."""
    cfg, ocfg = qb.configs.tiny(), tiny_ocfg(orc, qb)
    t = G.seeded_model_tensors(ocfg, 0xF11E, gain_sigma=0.1)
    tokens, merges = G.synth_bpe_vocab(0x70C)
    assert len(tokens) <= cfg.vocab_size
    eos = tokens.index(b"<|im_end|>")
    path = G.write_gguf(str(tmp_path / "chat.gguf"), ocfg, t, eos_id=eos, tokens=tokens, merges=merges)
    tok = qb.binding.Tokenizer.from_gguf(path)
    assert tok.vocab_size == cfg.vocab_size and tok.eos_id == eos
    text = "<|im_start|>user\nthe rate is 42 percent, isn't it?<|im_end|>\n<|im_start|>assistant\n"
    ids = tok.encode(text)
    assert ids.size < len(text) and int(ids.max()) < len(tokens) and ids[0] == tokens.index(b"<|im_start|>")
    assert tok.decode(ids) == text.encode()
    fm, mm = qb.Model.from_gguf(ctx, path), qb.Model.from_tensors(ctx, cfg, t)
    a, b = run_stream(qb, fm, ids.tolist(), 3, 4), run_stream(qb, mm, ids.tolist(), 3, 4)
    assert a[2] == b[2] and a[1] == b[1]
    out = tok.decode(np.array(a[2], np.int32))                # tokens beyond the tables decode to their placeholder names
    assert isinstance(out, bytes) and len(out) > 0
    fm.close(); mm.close(); tok.close()


def test_own_mtp_tables_and_tied_output(qb, orc, ctx, G):
    """nextn.embed_tokens / nextn.shared_head_head of their own, and a checkpoint without output.weight (LM head =
    token_embd): drafts and tokens equal the oracle's from the same tensors."""
    cfg, ocfg = qb.configs.tiny(), tiny_ocfg(orc, qb)
    t = G.seeded_model_tensors(ocfg, 0xFACE, gain_sigma=0.05)
    L = cfg.n_layers
    t["blk.%d.nextn.embed_tokens.weight" % L] = orc.synth_q8_0(1, 901, cfg.vocab_size, cfg.n_embd).reshape(cfg.vocab_size, -1)
    t["blk.%d.nextn.shared_head_head.weight" % L] = orc.synth_q8_0(1, 902, cfg.vocab_size, cfg.n_embd).reshape(cfg.vocab_size, -1)
    del t["output.weight"]
    prompt = orc.synth_prompt(13, cfg.vocab_size, 33)
    model = qb.Model.from_tensors(ctx, cfg, t)
    lg, drafts, toks = run_stream(qb, model, prompt, 3, 1)
    s = orc.Seq(orc.Model.from_tensors(ocfg, t), 128)
    s.prefill(prompt, 0)
    assert rel_err(lg[0][0], s.last_logits(1)[0]) < 1e-2
    s.set_cur_token(toks[0])
    _, od, _ = s.mtp_step(3)
    assert od == drafts[0]
    model.close()


def test_missing_or_misshaped_tensor_is_named(qb, orc, ctx, G):
    cfg, ocfg = qb.configs.tiny(), tiny_ocfg(orc, qb)
    t = G.seeded_model_tensors(ocfg, 5)
    bad = dict(t)
    del bad["blk.2.ssm_dt.bias"]
    with pytest.raises(qb.QbError, match="blk.2.ssm_dt.bias"):
        qb.Model.from_tensors(ctx, cfg, bad)
    bad = dict(t)
    bad["blk.3.attn_k_norm.weight"] = np.ones(7, np.float32)
    with pytest.raises(qb.QbError, match="blk.3.attn_k_norm.weight"):
        qb.Model.from_tensors(ctx, cfg, bad)
    bad = dict(t)
    bad["blk.0.ffn_down.weight"] = np.zeros((cfg.n_embd, cfg.n_ff), np.float32)      # F32 where Q8_0 is required
    with pytest.raises(qb.QbError, match="Q8_0"):
        qb.Model.from_tensors(ctx, cfg, bad)
