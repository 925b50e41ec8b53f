"""GPU tests of the whole step through the C ABI: logits vs the oracle, speculative == greedy
(lossless), forced-acceptance runs, paging and batch invariance."""
import numpy as np
import pytest

from conftest import tiny_ocfg

pytestmark = pytest.mark.gpu

LOGIT_TOL = 1e-2     # max |gpu - oracle| / max |oracle|, the bound the step is specified to


@pytest.fixture(scope="module")
def tiny(qb, orc, ctx):
    cfg = qb.configs.tiny()
    model = qb.Model(ctx, cfg, qb.configs.MODEL_SEED)
    omodel = orc.Model(tiny_ocfg(orc, qb), qb.configs.MODEL_SEED)
    prompt = orc.synth_prompt(qb.configs.PROMPT_SEED + 1, cfg.vocab_size, 64)
    yield dict(cfg=cfg, model=model, omodel=omodel, prompt=prompt)
    model.close()


def greedy_stream(qb, model, prompt, n, page_order=0, n_seqs=1, max_ctx=256):
    b = qb.Batch(model, n_seqs, max_ctx, 0, page_order=page_order)
    for s in range(n_seqs):
        b.prefill(s, prompt)
    outs = [list(b.read_output()[s]) for s in range(n_seqs)]
    while len(outs[0]) < n:
        b.greedy_step()
        for s, t in enumerate(b.read_output()):
            outs[s] += t
    b.close()
    return outs


def test_prefill_logits_and_greedy_stream_vs_oracle(qb, orc, ctx, tiny):
    b = qb.Batch(tiny["model"], 1, 256, 1)
    b.prefill(0, tiny["prompt"])
    got = list(b.read_output()[0])
    lg = b.last_logits(1)[0]
    s = orc.Seq(tiny["omodel"], 256)
    s.prefill(tiny["prompt"], 64)
    want_lg = s.last_logits(1)[0]
    assert np.abs(lg - want_lg).max() / np.abs(want_lg).max() < LOGIT_TOL
    want = [s.cur_token]
    for _ in range(31):
        b.greedy_step()
        got += b.read_output()[0]
        want.append(s.greedy_step())
        lg, want_lg = b.last_logits(1)[0], s.last_logits(1)[0]
        assert np.abs(lg - want_lg).max() / np.abs(want_lg).max() < LOGIT_TOL
    assert got == want
    assert b.position(0) == 64 + 31
    b.close()


def test_config1_mtp_k1_is_lossless(qb, orc, ctx, tiny):
    """BASELINE config 1: prompt 64, decode 32, k=1: speculative stream == greedy stream exactly."""
    want = greedy_stream(qb, tiny["model"], tiny["prompt"], 32)[0][:32]
    b = qb.Batch(tiny["model"], 1, 256, 1)
    b.prefill(0, tiny["prompt"])
    got = list(b.read_output()[0])
    while len(got) < 32:
        b.mtp_step()
        got += b.read_output()[0]
    assert got[:32] == want
    st = b.stats()
    assert st["steps"] > 0 and st["drafted"] == st["steps"]
    b.close()


def test_mtp_drafts_and_row_argmax_match_oracle_step(qb, orc, ctx, tiny):
    """One k=3 step compared piecewise with the oracle: emitted tokens and verify logits."""
    b = qb.Batch(tiny["model"], 1, 256, 3)
    b.prefill(0, tiny["prompt"])
    s = orc.Seq(tiny["omodel"], 256)
    s.prefill(tiny["prompt"], 64)
    for _ in range(4):
        b.mtp_draft()
        b.mtp_verify()
        lg = b.last_logits(4)
        b.mtp_accept_commit()
        toks = b.read_output()[0]
        otoks, odrafts, orows = s.mtp_step(3)
        olg = s.last_logits(4)
        assert toks == otoks
        assert np.abs(lg - olg).max() / np.abs(olg).max() < LOGIT_TOL
        assert np.argmax(lg, 1).tolist() == orows
    b.close()


@pytest.mark.parametrize("k", [1, 3])
def test_forced_acceptance_run_is_lossless(qb, orc, ctx, tiny, k):
    """Drafts forced to the true continuation at a seeded 70% rate exercise accept, partial accept and
    rollback; the emitted stream must still equal plain greedy decoding."""
    n = 48
    want = greedy_stream(qb, tiny["model"], tiny["prompt"], n + k + 2)[0]
    stream = np.zeros(64 + len(want) + 8, np.int32)
    stream[:64] = tiny["prompt"]
    stream[64:64 + len(want)] = want       # stream[p] = token at absolute position p
    sdev = ctx.array(stream)
    b = qb.Batch(tiny["model"], 1, 256, k)
    b.prefill(0, tiny["prompt"])
    got = list(b.read_output()[0])
    hist = []
    while len(got) < n:
        b.mtp_draft()
        b.mtp_force_drafts(sdev, len(stream), 0.7, 1234)
        b.mtp_verify()
        b.mtp_accept_commit()
        t = b.read_output()[0]
        hist.append(len(t) - 1)
        got += t
    assert got[:n] == want[:n]
    assert max(hist) == k and min(hist) < k        # both full acceptance and rejection happened
    st = b.stats()
    assert st["accepted"] == sum(hist) and st["emitted"] >= n
    b.close()


def test_page_order_invariance(qb, orc, ctx, tiny):
    """Identical token stream under identity / reverse / shuffled page tables (page 16)."""
    a = greedy_stream(qb, tiny["model"], tiny["prompt"], 24, page_order=0)[0]
    assert a == greedy_stream(qb, tiny["model"], tiny["prompt"], 24, page_order=1)[0]
    assert a == greedy_stream(qb, tiny["model"], tiny["prompt"], 24, page_order=2)[0]


def test_batch_invariance_and_ragged_batch(qb, orc, ctx, tiny):
    """Continuous-batching shape: several sequences with different prompt lengths in one batch give
    each sequence the stream it gets alone, greedy and speculative."""
    cfg = tiny["cfg"]
    prompts = [orc.synth_prompt(qb.configs.PROMPT_SEED + 10 + i, cfg.vocab_size, n) for i, n in enumerate([64, 17, 40])]
    alone = [greedy_stream(qb, tiny["model"], p, 20)[0][:20] for p in prompts]
    b = qb.Batch(tiny["model"], 3, 256, 3)
    for s, p in enumerate(prompts):
        b.prefill(s, p)
    outs = [list(t) for t in b.read_output()]
    while min(len(o) for o in outs) < 20:
        b.mtp_step()
        for s, t in enumerate(b.read_output()):
            outs[s] += t
    for s in range(3):
        assert outs[s][:20] == alone[s]
    b.close()


def test_capacity_error_is_reported_not_faulted(qb, orc, ctx, tiny):
    b = qb.Batch(tiny["model"], 1, 70, 1)
    b.prefill(0, tiny["prompt"])
    with pytest.raises(qb.QbError):
        for _ in range(10):
            b.mtp_step()
            b.read_output()
    with pytest.raises(qb.QbError):
        b.prefill(0, tiny["prompt"])
    b.close()
