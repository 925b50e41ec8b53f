"""Sampling-mode speculative acceptance on the device (qb_sample_rows, qb_mtp_sample_rows) against the oracle's restatement
of sampling_distribution + speculative_accept_pointmass (src/qwen_native_backend.cpp:282-467), same logits, same draws."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PARAMS = [(1.0, 1.0, 0, 0.0), (0.7, 0.9, 0, 0.0), (0.5, 1.0, 5, 0.0), (1.3, 0.8, 50, 0.05), (0.2, 0.0, 0, 0.3), (1.0, 0.5, 1, 0.0),
          (0.05, 0.95, 40, 0.0), (2.0, 0.999, 0, 0.0),
          (1.0, 1e-6, 0, 0.0), (1.0, 1.0, 0, 1.5), (1.0, 1.0, 10**9, 0.0), (1.0, 0.3, 3, 0.9)]      # one-token nucleus, min_p above 1 (collapses to the top token), top_k beyond the vocabulary


def gpu_sample(qb, ctx, x, draft, ua, ur, temp, top_p, top_k, min_p):
    rows, V = x.shape
    tok, acc, pd = ctx.empty((rows,), np.int32), ctx.empty((rows,), np.int32), ctx.empty((rows,), np.float32)
    d = ctx.array(np.ascontiguousarray(draft, np.int32)) if draft is not None else None
    a = ctx.array(np.ascontiguousarray(ua, np.float64)) if ua is not None else None
    qb.binding.check(qb.lib().qb_sample_rows(ctx.h, ctx.array(x).ptr, rows, V, V, d.ptr if d else None, a.ptr if a else None,
                                             ctx.array(np.ascontiguousarray(ur, np.float64)).ptr, temp, top_p, top_k, min_p,
                                             tok.ptr, acc.ptr, pd.ptr))
    ctx.sync()
    return tok.download(), acc.download(), pd.download()


@pytest.mark.parametrize("temp,top_p,top_k,min_p", PARAMS)
@pytest.mark.parametrize("V", [3000, 151936])
def test_sample_rows_vs_oracle(qb, orc, ctx, V, temp, top_p, top_k, min_p):
    rng = np.random.default_rng(100 + V % 97 + int(temp * 10))
    rows = 8
    x = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    x[3, 100] = x[3, V - 5] = x[3].max() + 1                      # a tie at the top: lowest index first
    x[5, :] = np.round(x[5, :] * 2) / 2                           # many ties everywhere
    draft = np.where(np.arange(rows) % 3 == 2, -1, x.argmax(1)).astype(np.int32)
    draft[4] = 7                                                  # a draft the target gives almost no mass
    ua, ur = rng.random(rows), rng.random(rows)
    ur[0], ur[1] = 0.0, 1.0 - 1e-12                               # ends of the inverse CDF
    want = orc.sample_rows(x, draft, ua, ur, temp, top_p, top_k, min_p)
    got = gpu_sample(qb, ctx, x, draft, ua, ur, temp, top_p, top_k, min_p)
    assert np.allclose(got[2], want[2], rtol=2e-5, atol=1e-9), (got[2], want[2])
    assert np.array_equal(got[1], want[1]), (got[1], want[1])
    assert np.array_equal(got[0], want[0]), (got[0], want[0])


def test_plain_sampling_rows_follow_the_distribution(qb, orc, ctx):
    """No drafts: 4000 draws of one 50-token row reproduce its truncated distribution (chi-square-sized bound)."""
    rng = np.random.default_rng(5)
    V, n = 50, 4000
    row = (rng.standard_normal(V) * 2).astype(np.float32)
    x = np.tile(row, (n, 1))
    ur = rng.random(n)
    tok, _, _ = gpu_sample(qb, ctx, x, None, None, ur, 0.8, 0.9, 0, 0.0)
    want, _, _ = orc.sample_rows(x[:1], np.array([-1], np.int32), np.zeros(1), ur[:1], 0.8, 0.9, 0, 0.0)
    assert tok[0] == want[0]
    e = np.exp((row - row.max()) / 0.8); p = e / e.sum()
    order = np.argsort(-p); keep = order[:np.nonzero(np.cumsum(p[order]) >= 0.9)[0][0] + 1]
    q = np.zeros(V); q[keep] = p[keep] / p[keep].sum()
    freq = np.bincount(tok, minlength=V) / n
    assert set(np.nonzero(freq)[0]) <= set(keep)
    assert np.abs(freq - q).max() < 4 * np.sqrt(0.25 / n)


@pytest.fixture(scope="module")
def model(qb, ctx):
    m = qb.Model(ctx, qb.configs.tiny(), qb.configs.MODEL_SEED)
    yield m
    m.close()


def test_top_k_one_is_greedy(qb, orc, ctx, model):
    """top_k = 1 makes the target a point mass at the argmax: whatever the draws, the sampled speculative stream is the greedy one."""
    V = model.cfg.vocab_size
    prompt = orc.synth_prompt(77, V, 48)
    g = qb.Batch(model, 1, 256, 0)
    g.prefill(0, prompt)
    want = list(g.read_output()[0])
    while len(want) < 24:
        g.greedy_step()
        want += g.read_output()[0]
    g.close()
    b = qb.Batch(model, 1, 256, 3)
    b.prefill(0, prompt)
    got = list(b.read_output()[0])
    rng = np.random.default_rng(1)
    while len(got) < 24:
        b.mtp_step_sampled(rng.random((1, 4)), temp=0.9, top_k=1)
        got += b.read_output()[0]
    b.close()
    assert got[:24] == want[:24]


@pytest.mark.parametrize("temp,top_p,top_k", [(1.0, 1.0, 0), (0.6, 0.9, 20)])
def test_sampled_step_matches_the_reference_accept_loop(qb, orc, ctx, model, temp, top_p, top_k):
    """Each step: the verifier's logits and the drafts go through the oracle's accept loop with the same draws (row i accepts
    with u[i], a rejection at row i draws with u[i+1], the bonus draw is u[k]); the step must emit exactly those tokens."""
    V, k, ns = model.cfg.vocab_size, 3, 2
    b = qb.Batch(model, ns, 256, k)
    for s in range(ns):
        b.prefill(s, orc.synth_prompt(80 + s, V, 30 + 7 * s))
    rng = np.random.default_rng(3)
    n_acc = 0
    for step in range(12):
        u = rng.random((ns, k + 1))
        if step % 3 == 0:
            u[:, 0] = 0.0                                        # force some acceptances of the first draft
        b.mtp_draft()
        b.mtp_verify()
        logits = b.last_logits(ns * (k + 1)).reshape(ns, k + 1, V).copy()
        drafts = b.last_drafts()
        b.mtp_sample_rows(u, temp, top_p, top_k)
        b.mtp_accept_commit()
        out = b.read_output()
        for s in range(ns):
            want = []
            for i in range(k + 1):
                d = int(drafts[s, i]) if i < k else -1
                tok, acc, _ = orc.sample_rows(logits[s, i:i + 1], np.array([d], np.int32), u[s, i:i + 1], u[s, min(i + 1, k):min(i + 1, k) + 1],
                                              temp, top_p, top_k, 0.0)
                want.append(int(tok[0]))
                if d < 0 or not acc[0]:
                    break
                n_acc += 1
            assert out[s] == want, (step, s, out[s], want)
    if top_k == 0:
        assert n_acc > 0          # untruncated: every draft has some mass, and u = 0 accepts it
    b.close()


def test_token_penalties_follow_the_running_prefix(qb, orc, ctx, model):
    """presence / repetition penalties: row i of a step is penalised on the request's prompt and emitted tokens plus the
    step's drafts 0..i-1 (apply_token_penalties against the running prefix of the accept loop)."""
    V, k, ns = model.cfg.vocab_size, 3, 2
    pres, rep = 0.7, 1.3
    temp, top_p, top_k = 0.8, 0.95, 0
    b = qb.Batch(model, ns, 256, k)
    b.set_penalties(pres, rep)
    seen = []
    for s in range(ns):
        prompt = orc.synth_prompt(90 + s, V, 25 + 9 * s)
        b.prefill(s, prompt)
        seen.append(set(int(t) for t in prompt) | set(b.read_output()[s]))
    rng = np.random.default_rng(4)

    def penalise(row, toks):
        row = row.copy()
        idx = np.array(sorted(toks), np.int64)
        v = row[idx]
        v = np.where(v >= 0, v / np.float32(rep), v * np.float32(rep)).astype(np.float32) - np.float32(pres)
        row[idx] = v
        return row

    changed = 0
    for step in range(10):
        u = rng.random((ns, k + 1))
        if step % 2 == 0:
            u[:, 0] = 0.0
        b.mtp_draft()
        b.mtp_verify()
        logits = b.last_logits(ns * (k + 1)).reshape(ns, k + 1, V).copy()
        drafts = b.last_drafts()
        b.mtp_sample_rows(u, temp, top_p, top_k)
        b.mtp_accept_commit()
        out = b.read_output()
        for s in range(ns):
            want, ctxset = [], set(seen[s])
            for i in range(k + 1):
                d = int(drafts[s, i]) if i < k else -1
                row = penalise(logits[s, i], ctxset)
                ui = min(i + 1, k)
                tok, acc, _ = orc.sample_rows(row[None], np.array([d], np.int32), u[s, i:i + 1], u[s, ui:ui + 1], temp, top_p, top_k, 0.0)
                plain, _, _ = orc.sample_rows(logits[s, i][None], np.array([d], np.int32), u[s, i:i + 1], u[s, ui:ui + 1], temp, top_p, top_k, 0.0)
                changed += int(plain[0] != tok[0])
                want.append(int(tok[0]))
                if d < 0 or not acc[0]:
                    break
                ctxset.add(d)
            assert out[s] == want, (step, s, out[s], want)
            seen[s] |= set(out[s])
    assert changed > 0            # the penalties did change decisions in this run
    # a recycled slot starts with an empty record
    b.reset(0)
    p2 = orc.synth_prompt(95, V, 11)
    b.prefill(0, p2)
    seen0 = set(int(t) for t in p2) | set(b.read_output()[0])
    u = rng.random((ns, k + 1))
    b.mtp_draft(); b.mtp_verify()
    logits = b.last_logits(ns * (k + 1)).reshape(ns, k + 1, V).copy()
    drafts = b.last_drafts()
    b.mtp_sample_rows(u, temp, top_p, top_k); b.mtp_accept_commit()
    d = int(drafts[0, 0])
    tok, acc, _ = orc.sample_rows(penalise(logits[0, 0], seen0)[None], np.array([d], np.int32), u[0, 0:1], u[0, 1:2], temp, top_p, top_k, 0.0)
    assert b.read_output()[0][0] == int(tok[0])
    b.close()


@pytest.mark.parametrize("penalties", [False, True])
def test_sampled_stream_replays_through_one_continuous_generator(qb, orc, ctx, model, penalties):
    """A whole sampled request, first token included, against the reference's generator order: ONE generator per request;
    the first draw picks the token after the prompt (pick_from_last_logits), then every step draws one uniform per
    acceptance test and one for the residual or bonus token (speculative_accept_pointmass).  The host loop hands the
    step k+1 draws from a DrawQueue and returns the unused ones; the replay below consumes a fresh copy of the same
    generator strictly in sequence through the oracle's sampler and must produce the same tokens."""
    V, k = model.cfg.vocab_size, 3
    temp, top_p, top_k, pres, rep = 0.9, 0.95, 0, 0.6, 1.25
    prompt = orc.synth_prompt(321, V, 37)
    b = qb.Batch(model, 1, 256, k)
    if penalties:
        b.set_penalties(pres, rep)
    dq = qb.serve.DrawQueue(np.random.default_rng(77), k + 1)
    replay = np.random.default_rng(77)

    def penalise(row, toks):
        if not penalties:
            return row
        row = row.copy()
        idx = np.array(sorted(toks), np.int64)
        v = row[idx]
        row[idx] = np.where(v >= 0, v / np.float32(rep), v * np.float32(rep)).astype(np.float32) - np.float32(pres)
        return row

    one = lambda: np.array([replay.random()], np.float64)
    # chunked ingestion: the parts of the prompt that are not its end choose no token and count nothing
    b.prefill(0, prompt[:16], more=True)
    b.prefill(0, prompt[16:30], more=True)
    assert b.stats()["emitted"] == 0
    b.prefill_sampled(0, prompt[30:], dq.take(), temp, top_p, top_k)
    first = b.read_output()[0]
    seen = set(int(t) for t in prompt)
    tok, _, _ = orc.sample_rows(penalise(b.last_logits(1)[0], seen)[None], np.array([-1], np.int32), np.zeros(1), one(), temp, top_p, top_k, 0.0)
    assert first == [int(tok[0])]
    assert b.stats()["emitted"] == 1
    seen |= set(first)
    emitted, rejected, full = list(first), 0, 0
    for step in range(16):
        depth = (k, 1, 2, k)[step % 4]                      # the chain policy: the row after the last draft is the bonus row
        b.set_draft_policy([depth])
        u = np.array([dq.peek()], np.float64)
        b.mtp_draft()
        b.mtp_verify()
        logits = b.last_logits(k + 1).copy()
        drafts = b.last_drafts()[0]
        b.mtp_sample_rows(u, temp, top_p, top_k)
        b.mtp_accept_commit()
        out = b.read_output()[0]
        dq.consume_step(len(out), depth)
        # the reference's loop on the continuous generator
        want, ctxset = [], set(seen)
        for i in range(depth + 1):
            d = int(drafts[i]) if i < depth else -1
            row = penalise(logits[i], ctxset)
            if d >= 0:
                ua = one()
                _, acc, _ = orc.sample_rows(row[None], np.array([d], np.int32), ua, ua, temp, top_p, top_k, 0.0)
                if acc[0]:
                    want.append(d)
                    ctxset.add(d)
                    continue
                t, _, _ = orc.sample_rows(row[None], np.array([d], np.int32), np.array([2.0]), one(), temp, top_p, top_k, 0.0)   # rejected: residual draw
                want.append(int(t[0]))
                rejected += 1
                break
            t, _, _ = orc.sample_rows(row[None], np.array([-1], np.int32), np.zeros(1), one(), temp, top_p, top_k, 0.0)               # bonus draw
            want.append(int(t[0]))
            full += 1
        assert out == want, (step, out, want)
        seen |= set(out)
        emitted += out
    assert rejected > 0
    b.close()
