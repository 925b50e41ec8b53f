"""Pooled K/V pages and shared prompt prefixes through the C ABI (the reference's GlobalKvPagePool and prefix cache,
src/qwen_native_backend.cpp:1155-1265, 6603-6709, 9785-10410): a pooled batch must produce the bits of a batch with
private pages, report an exhausted pool before launching anything, recycle pages most recently freed first, and let a
request continue from another request's prefix without ingesting it."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
PAGE = 16


@pytest.fixture(scope="module")
def tiny_model(qb, ctx):
    m = qb.Model(ctx, qb.configs.tiny(), qb.configs.MODEL_SEED)
    yield m
    m.close()


def run_steps(b, n_steps, speculative=True):
    outs = [list(t) for t in b.read_output()]
    logits = []
    for _ in range(n_steps):
        b.mtp_step() if speculative else b.greedy_step()
        logits.append(b.last_logits(b.n_seqs * (b.k + 1 if speculative else 1)).copy())
        for s, t in enumerate(b.read_output()):
            outs[s] += t
    return outs, logits


def test_pooled_batch_has_the_bits_of_private_pages(qb, orc, ctx, tiny_model):
    V, k = tiny_model.cfg.vocab_size, 3
    prompts = [orc.synth_prompt(700 + s, V, n) for s, n in enumerate((37, 5, 64))]
    ref = qb.Batch(tiny_model, 3, 192, k)
    pooled = qb.Batch(tiny_model, 3, 192, k, pool_pages=24)          # 3 x 13 pages would be the private form
    assert pooled.pool_info() == dict(free=24, total=24, page_size=PAGE)
    for b in (ref, pooled):
        for s, p in enumerate(prompts):
            b.prefill(s, p)
    assert [len(pooled.seq_pages(s)) for s in range(3)] == [3, 1, 4]
    assert pooled.seq_pages(0) == [0, 1, 2] and pooled.seq_pages(1) == [3]      # handed out in order of need
    want, want_logits = run_steps(ref, 10)
    got, got_logits = run_steps(pooled, 10)
    assert got == want
    for a, c in zip(got_logits, want_logits):
        assert np.array_equal(a, c)
    used = sum(len(pooled.seq_pages(s)) for s in range(3))
    assert pooled.pool_info()["free"] == 24 - used
    # a sequence never holds more than its position bound needs: positions + the k + 1 rows of the next step
    st = pooled.stats()
    assert used <= sum((len(p) + len(o) + k + 1 + PAGE - 1) // PAGE + 1 for p, o in zip(prompts, got)), st
    ref.close()
    pooled.close()


def test_exhaustion_is_reported_and_pages_come_back(qb, orc, ctx, tiny_model):
    V = tiny_model.cfg.vocab_size
    b = qb.Batch(tiny_model, 3, 128, 1, pool_pages=6)
    b.set_active(0)
    b.prefill(0, orc.synth_prompt(1, V, 40))             # 3 pages
    b.prefill(1, orc.synth_prompt(2, V, 30))             # 2 pages
    assert b.pool_info()["free"] == 1
    with pytest.raises(qb.QbError, match="page pool exhausted"):
        b.prefill(2, orc.synth_prompt(3, V, 40))         # needs 3, 1 free: refused before any launch
    assert b.pool_info()["free"] == 1 and b.seq_pages(2) == []
    first = b.seq_pages(0)
    b.reset(0)                                           # the request retires: its pages return
    assert b.pool_info()["free"] == 4
    b.prefill(2, orc.synth_prompt(3, V, 40))
    assert b.seq_pages(2) == first                       # most recently freed first, the retired request's first page on top
    # the refused call left the context usable: decode goes on and equals a batch with private pages
    solo = qb.Batch(tiny_model, 1, 128, 1)
    solo.prefill(0, orc.synth_prompt(3, V, 40))
    b.swap(0, 2)
    b.set_active(1)
    want, _ = run_steps(solo, 6)
    got, _ = run_steps(b, 6)
    assert got[0] == want[0]
    # decoding past the pool: the step that needs a page nobody can give is refused, the sequence stays where it was
    b.reset(1)
    hog = qb.Batch(tiny_model, 1, 128, 1, pool_pages=3)
    hog.prefill(0, orc.synth_prompt(3, V, 40))
    with pytest.raises(qb.QbError, match="page pool exhausted"):
        for _ in range(40):
            hog.mtp_step()
            hog.read_output()
    qb.lib().qb_synchronize(ctx.h)
    hog.close()
    solo.close()
    b.close()


@pytest.mark.parametrize("penalties", [False, True])
def test_request_continues_from_a_shared_prefix(qb, orc, ctx, tiny_model, penalties):
    V, k = tiny_model.cfg.vocab_size, 3
    prefix = orc.synth_prompt(41, V, 2 * PAGE)
    rest_a, rest_b = orc.synth_prompt(42, V, 9), orc.synth_prompt(43, V, 21)
    samp = dict(temp=0.8, top_p=0.95, top_k=0)
    u = np.random.default_rng(5).random((12, 1, k + 1))

    def decode(b, seq_prompt_done):
        outs = list(b.read_output()[0])
        for i in range(12):
            if penalties:
                b.mtp_step_sampled(np.tile(u[i], (b.n_seqs, 1)), **samp)
            else:
                b.mtp_step()
            outs += b.read_output()[0]
        return outs, b.last_logits(k + 1).copy()

    # what request B gives when it ingests its whole prompt itself
    solo = qb.Batch(tiny_model, 1, 192, k)
    if penalties:
        solo.set_penalties(0.7, 1.3)
    solo.prefill(0, np.concatenate([prefix, rest_b]))
    want, want_logits = decode(solo, None)
    solo.close()

    b = qb.Batch(tiny_model, 2, 192, k, pool_pages=16)
    if penalties:
        b.set_penalties(0.7, 1.3)
    b.set_active(0)
    b.prefill(0, prefix, more=True)                       # request A: the prefix, then an entry of it, then its own tokens
    entry = b.prefix_capture(0, prefix)
    assert qb.lib().qb_prefix_tokens(entry) == 2 * PAGE
    b.prefill(0, rest_a)
    with pytest.raises(qb.QbError, match="not at the end"):
        b.prefix_capture(0, prefix)                       # A has moved on
    b.prefix_attach(1, entry)                             # request B: no ingestion of the prefix
    assert b.seq_pages(1) == b.seq_pages(0)[:2]
    b.prefill(1, rest_b)
    assert b.seq_pages(1)[2] not in b.seq_pages(0)        # B's own tokens go to pages of its own
    b.swap(0, 1)
    b.set_active(1)
    got, got_logits = decode(b, None)
    assert got == want
    assert np.array_equal(got_logits, want_logits)
    # the entry keeps the prefix pages alive when both requests are gone; releasing it frees them
    b.reset(0)
    b.reset(1)
    assert b.pool_info()["free"] == 16 - 2
    with pytest.raises(qb.QbError, match="not empty"):
        b.prefill(0, rest_a)
        b.prefix_attach(0, entry)
    b.reset(0)
    b.prefix_release(entry)
    assert b.pool_info()["free"] == 16
    b.close()


def test_serving_loop_with_prefix_cache_and_page_pool(qb, orc, ctx, tiny_model):
    """The compacting loop on a pooled batch with the prefix-cache policy: requests that share a system prompt start from
    the cached entry (fewer prompt tokens ingested), pages are reserved at admission, and every request still gets exactly
    the token stream it gets alone."""
    V, k = tiny_model.cfg.vocab_size, 3
    system = [int(t) for t in orc.synth_prompt(500, V, 40)]
    tails = [[int(t) for t in orc.synth_prompt(510 + i, V, n)] for i, n in enumerate((5, 17, 9, 30))]
    prompts = [system + tails[0], system + tails[1], [int(t) for t in orc.synth_prompt(520, V, 50)], system + tails[2], system[:33] + tails[3]]

    def alone(prompt, n):
        b = qb.Batch(tiny_model, 1, 256, k)
        b.prefill(0, prompt)
        out = list(b.read_output()[0])
        while len(out) < n:
            b.mtp_step()
            out += b.read_output()[0]
        b.close()
        return out[:n]

    want = [alone(p, 12) for p in prompts]
    eng = qb.Batch(tiny_model, 2, 256, k, pool_pages=20)
    counted = {"n": 0}
    raw_prefill = eng.prefill

    def counting_prefill(seq, tokens, more=False):
        counted["n"] += len(tokens)
        raw_prefill(seq, tokens, more)

    eng.prefill = counting_prefill
    cache = qb.serve.PrefixCache(eng, max_entries=3)
    reqs = [qb.serve.Request(i, p, 12, arrival_step=3 * i) for i, p in enumerate(prompts)]
    done = qb.serve.run_compact(eng, reqs, prefix_cache=cache)
    assert sorted(r.rid for r in done) == list(range(len(prompts)))
    for r in done:
        assert r.tokens == want[r.rid], r.rid
    assert cache.hits == 3                                   # requests 1, 3 and 4 start from the 32-token entry of request 0
    assert counted["n"] == sum(len(p) for p in prompts) - 3 * 32
    cache.clear()
    assert eng.pool_info()["free"] == 20                     # every page is back: requests retired, entries released
    eng.close()


def test_sequence_being_ingested_survives_the_steps_of_the_others(qb, orc, ctx, tiny_model):
    """A request whose prompt arrives in parts while another request decodes and the host reads every step record: the
    host's position bound of the ingesting sequence must stay where its last chunk left it (it decides which pages the next
    chunk gets), and the request must end with the stream it gets alone."""
    V, k = tiny_model.cfg.vocab_size, 3
    pa, pb = orc.synth_prompt(801, V, 30), orc.synth_prompt(802, V, 61)
    solo = qb.Batch(tiny_model, 1, 192, k)
    solo.prefill(0, pb)
    want, _ = run_steps(solo, 6)
    solo.close()
    b = qb.Batch(tiny_model, 2, 192, k, pool_pages=12)
    b.set_active(0)
    b.prefill(0, pa)
    b.read_output()
    b.set_active(1)
    for lo, hi in ((0, 20), (20, 48), (48, 61)):
        if hi < 61:
            b.prefill(1, pb[lo:hi], more=True)
        else:
            b.prefill(1, pb[lo:hi])
        assert len(b.seq_pages(1)) == -(-hi // PAGE)
        b.mtp_step()                      # request A decodes in between; its record is read
        b.read_output()
    b.swap(0, 1)
    b.set_active(1)
    b.reset(1)
    # (the first token of B was emitted by its last prefill call, before A's step overwrote nothing of it)
    got = [b.current_token(0)] if hasattr(b, "current_token") else None
    outs = []
    for _ in range(6):
        b.mtp_step()
        outs += b.read_output()[0]
    assert outs == want[0][1:1 + len(outs)]
    b.close()
