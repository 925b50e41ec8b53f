"""Continuous batching on the GPU: requests admitted at different steps into recycled sequence slots get exactly the
token stream each gets alone (qb_seq_reset + the batch-invariant kernels), greedy and speculative."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def alone(qb, model, prompt, n, k):
    b = qb.Batch(model, 1, 256, k)
    b.prefill(0, prompt)
    out = list(b.read_output()[0])
    while len(out) < n:
        if k:
            b.mtp_step()
        else:
            b.greedy_step()
        out += b.read_output()[0]
    b.close()
    return out[:n]


@pytest.fixture(scope="module")
def model(qb, ctx):
    m = qb.Model(ctx, qb.configs.tiny(), qb.configs.MODEL_SEED)
    yield m
    m.close()


def test_reset_slot_equals_fresh_batch(qb, orc, ctx, model):
    V = model.cfg.vocab_size
    p1, p2 = orc.synth_prompt(91, V, 40), orc.synth_prompt(92, V, 23)
    want = alone(qb, model, p2, 16, 1)
    b = qb.Batch(model, 2, 256, 1)
    b.prefill(0, p1); b.prefill(1, p1)
    for _ in range(9):
        b.mtp_step()
    b.read_output()
    b.reset(1)
    assert b.position(1) == 0 and b.position(0) > 40
    b.prefill(1, p2)
    got = list(b.read_output()[1])
    while len(got) < 16:
        b.mtp_step()
        got += b.read_output()[1]
    assert got[:16] == want
    b.close()


@pytest.mark.parametrize("k,slots", [(1, 2), (0, 3), (1, 1)])
def test_served_requests_match_their_solo_streams(qb, orc, ctx, model, k, slots):
    V = model.cfg.vocab_size
    spec = [(64, 12, 0), (17, 30, 0), (40, 9, 0), (5, 20, 3), (33, 14, 25), (8, 1, 26)]
    reqs = [qb.serve.Request(i, orc.synth_prompt(200 + i, V, n), new, arrival_step=a) for i, (n, new, a) in enumerate(spec)]
    b = qb.Batch(model, slots, 256, k)
    done = qb.serve.run(b, reqs, speculative=k > 0)
    b.close()
    assert sorted(r.rid for r in done) == list(range(len(spec)))
    for r in done:
        assert r.tokens == alone(qb, model, r.prompt, r.max_new_tokens, k), r.rid
    assert len({r.slot for r in done}) <= slots


def test_idle_slot_survives_a_long_run(qb, orc, ctx, model):
    """One request in a two-slot batch whose context is short: the idle slot is reset before it overflows."""
    V = model.cfg.vocab_size
    p = orc.synth_prompt(300, V, 10)
    b = qb.Batch(model, 2, 96, 1)
    done = qb.serve.run(b, [qb.serve.Request(0, p, 70), qb.serve.Request(1, p, 70, arrival_step=200)])
    b.close()
    want = alone(qb, model, p, 70, 1)
    assert done[0].tokens == want and done[1].tokens == want


def test_sampled_serving_reproduces_each_request_alone(qb, orc, ctx, model):
    """Sampling mode through the loop: a request with its own generator gets the same tokens in a shared batch with delayed
    admission as alone in a one-slot batch (decisions depend only on the request's logits and its own draws)."""
    V = model.cfg.vocab_size
    samp = dict(temp=0.9, top_p=0.95, top_k=40, min_p=0.0)
    spec = [(30, 14, 0), (12, 20, 0), (21, 10, 2), (9, 16, 5)]
    mk = lambda: [qb.serve.Request(i, orc.synth_prompt(400 + i, V, n), new, arrival_step=a) for i, (n, new, a) in enumerate(spec)]
    rng_of = lambda r: np.random.default_rng(1000 + r.rid)
    b = qb.Batch(model, 2, 256, 1)
    together = {r.rid: r.tokens for r in qb.serve.run(b, mk(), sampling=samp, rng_of=rng_of)}
    b.close()
    for req in mk():
        b1 = qb.Batch(model, 1, 256, 1)
        req.arrival_step = 0
        solo = qb.serve.run(b1, [req], sampling=samp, rng_of=rng_of)[0].tokens
        b1.close()
        assert together[req.rid] == solo, req.rid
    # and top_k = 1 collapses to the greedy stream whatever the draws
    b = qb.Batch(model, 2, 256, 1)
    done = qb.serve.run(b, mk(), sampling=dict(temp=0.7, top_p=1.0, top_k=1, min_p=0.0), rng_of=rng_of)
    b.close()
    for r in done:
        assert r.tokens == alone(qb, model, r.prompt, r.max_new_tokens, 1), r.rid


def test_swap_and_active_prefix(qb, orc, ctx, model):
    """Three requests in a 3-slot batch; after some steps slots 0 and 2 are exchanged and only the first two slots stay
    active: the exchanged requests continue their own streams, the parked one resumes unchanged later."""
    V = model.cfg.vocab_size
    prompts = [orc.synth_prompt(500 + i, V, n) for i, n in enumerate([30, 12, 21])]
    want = [alone(qb, model, p, 40, 1) for p in prompts]
    b = qb.Batch(model, 3, 256, 1)
    outs = []
    for s, p in enumerate(prompts):
        b.prefill(s, p)
        outs.append(list(b.read_output()[s]))
    for _ in range(5):
        b.mtp_step()
        for s, t in enumerate(b.read_output()):
            outs[s] += t
    b.swap(0, 2)
    outs[0], outs[2] = outs[2], outs[0]
    want[0], want[2] = want[2], want[0]
    b.set_active(2)
    for _ in range(6):
        b.mtp_step()
        o = b.read_output()
        for s in range(2):
            outs[s] += o[s]
    parked = len(outs[2])
    b.set_active(3)
    while min(len(o) for o in outs) < 40:
        b.mtp_step()
        for s, t in enumerate(b.read_output()):
            outs[s] += t
    for s in range(3):
        assert outs[s][:40] == want[s], s
    assert parked < 40
    b.close()


@pytest.mark.parametrize("k,slots,chunk", [(1, 2, 0), (1, 3, 8), (0, 2, 5)])
def test_compacting_loop_matches_solo_streams(qb, orc, ctx, model, k, slots, chunk):
    V = model.cfg.vocab_size
    spec = [(64, 12, 0), (17, 30, 0), (40, 9, 0), (5, 20, 3), (33, 14, 25), (8, 1, 26), (29, 11, 27)]
    reqs = [qb.serve.Request(i, orc.synth_prompt(600 + i, V, n), new, arrival_step=a) for i, (n, new, a) in enumerate(spec)]
    b = qb.Batch(model, slots, 256, k)
    done = qb.serve.run_compact(b, reqs, speculative=k > 0, prefill_chunk=chunk)
    b.close()
    assert sorted(r.rid for r in done) == list(range(len(spec)))
    for r in done:
        assert r.tokens == alone(qb, model, r.prompt, r.max_new_tokens, k), r.rid


def test_compacting_loop_sampled_with_penalties(qb, orc, ctx, model):
    V = model.cfg.vocab_size
    samp = dict(temp=0.9, top_p=0.95, top_k=40, min_p=0.0, presence=0.5, repetition=1.2)
    spec = [(30, 14, 0), (12, 20, 0), (21, 10, 2), (9, 16, 5)]
    mk = lambda: [qb.serve.Request(i, orc.synth_prompt(700 + i, V, n), new, arrival_step=a) for i, (n, new, a) in enumerate(spec)]
    rng_of = lambda r: np.random.default_rng(2000 + r.rid)
    b = qb.Batch(model, 2, 256, 1)
    together = {r.rid: r.tokens for r in qb.serve.run_compact(b, mk(), sampling=samp, rng_of=rng_of, prefill_chunk=7)}
    b.close()
    for req in mk():
        b1 = qb.Batch(model, 1, 256, 1)
        req.arrival_step = 0
        solo = qb.serve.run_compact(b1, [req], sampling=samp, rng_of=rng_of)[0].tokens
        b1.close()
        assert together[req.rid] == solo, req.rid


def test_reset_then_read_keeps_the_slot_at_position_zero(qb, orc, ctx, model):
    """A recycled slot stays at position 0 for the host as well, whatever step records are read before its prefill."""
    V = model.cfg.vocab_size
    b = qb.Batch(model, 2, 128, 1)
    b.prefill(0, orc.synth_prompt(1, V, 90)); b.prefill(1, orc.synth_prompt(2, V, 70))
    b.mtp_step(); b.read_output()
    b.reset(1)
    b.read_output()                                      # refreshes the host's position mirror from the records
    b.prefill(1, orc.synth_prompt(3, V, 100))            # would not fit behind the old request's 70 tokens
    assert b.position(1) == 100
    b.close()
