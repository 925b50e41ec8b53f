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
