"""Host logic of the continuous-batching loop (kvmem-qw3_b200/serve.py) against a fake engine whose token streams are a
pure function of the prompt: admission order, slot reuse, delayed arrival, EOS / budget trimming, idle-slot resets."""
import sys
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def stream(prompt, n):
    """The tokens a request with this prompt gets alone: a hash chain."""
    out, h = [], sum((i + 1) * t for i, t in enumerate(prompt)) % 9973
    for _ in range(n):
        h = (h * 31 + 7) % 9973
        out.append(h % 1000)
    return out


class FakeEngine:
    """Mimics binding.Batch: every step emits 1..k+1 tokens per slot (the count cycles), slots keep independent state."""

    def __init__(self, n_seqs, k, max_ctx):
        self.n_seqs, self.k, self.max_ctx = n_seqs, k, max_ctx
        self.prompt = [None] * n_seqs
        self.emitted = [0] * n_seqs
        self.pos = [0] * n_seqs
        self.out = [[] for _ in range(n_seqs)]
        self.resets, self.steps = [], 0

    def reset(self, s):
        self.prompt[s], self.emitted[s], self.pos[s] = None, 0, 0
        self.resets.append(s)

    def prefill(self, s, tokens, more=False):
        assert self.pos[s] == 0, "prefill into a slot that was not reset"
        assert not more, "the fixed-slot loop ingests whole prompts"
        self.prompt[s] = list(tokens)
        self.pos[s] = len(tokens)
        self.out[s] = stream(self.prompt[s], 1)
        self.emitted[s] = 1

    def prefill_sampled(self, s, tokens, u, **kw):
        self.first_draws = getattr(self, "first_draws", {})
        self.first_draws[tuple(tokens)] = u
        self.prefill(s, tokens)

    def _step(self, width):
        self.steps += 1
        for s in range(self.n_seqs):
            n = 1 + (self.steps + s) % width
            assert self.pos[s] + width <= self.max_ctx + width and self.pos[s] < self.max_ctx, "slot ran out of context"
            self.pos[s] += n
            if self.prompt[s] is None:
                self.out[s] = [0] * n
                continue
            full = stream(self.prompt[s], self.emitted[s] + n)
            self.out[s] = full[self.emitted[s]:]
            self.emitted[s] += n

    def mtp_step(self):
        self._step(self.k + 1)

    def greedy_step(self):
        self._step(1)

    def read_output(self):
        return [list(o) for o in self.out]


def test_requests_get_the_stream_they_get_alone_with_delayed_admission():
    serve = entry.load_package().serve
    eng = FakeEngine(2, 3, 512)
    reqs = [serve.Request(i, [i + 1, 2 * i + 3, 5], 5 + 3 * i, arrival_step=a) for i, a in enumerate([0, 0, 0, 4, 30])]
    done = serve.run(eng, reqs)
    assert sorted(r.rid for r in done) == [0, 1, 2, 3, 4]
    for r in done:
        assert r.tokens == stream(r.prompt, r.max_new_tokens), r.rid
        assert r.admitted_step >= r.arrival_step and r.finished_step >= r.admitted_step
    by = {r.rid: r for r in done}
    assert by[0].slot == 0 and by[1].slot == 1            # slot 0 first
    assert by[2].admitted_step > 0                        # had to wait for a slot
    first_free = min(by[0].finished_step, by[1].finished_step)
    assert by[2].admitted_step == first_free              # admitted in the iteration after a slot was freed
    assert by[3].admitted_step >= max(4, first_free)
    assert by[4].admitted_step >= 30


def test_eos_trims_and_frees_the_slot():
    serve = entry.load_package().serve
    eng = FakeEngine(1, 3, 256)
    full = stream([9, 9], 40)
    eos = full[6]
    first = full.index(eos)
    done = serve.run(eng, [serve.Request("a", [9, 9], 40, eos=eos), serve.Request("b", [1], 3)])
    assert done[0].rid == "a" and done[0].tokens == full[:first + 1]
    assert done[1].tokens == stream([1], 3)


def test_idle_slots_are_reset_before_they_run_out_of_context():
    serve = entry.load_package().serve
    eng = FakeEngine(2, 3, 64)
    done = serve.run(eng, [serve.Request(0, [1, 2, 3], 40)], speculative=True)      # slot 1 idles through many steps
    assert done[0].tokens == stream([1, 2, 3], 40)
    done = serve.run(eng, [serve.Request(1, [4], 50), serve.Request(2, [5], 50, arrival_step=3)])
    assert [r.tokens for r in sorted(done, key=lambda r: r.rid)] == [stream([4], 50), stream([5], 50)]
    assert eng.resets.count(1) >= 2


def test_greedy_mode_and_budget_of_one():
    serve = entry.load_package().serve
    eng = FakeEngine(2, 0, 128)
    done = serve.run(eng, [serve.Request(0, [3], 1), serve.Request(1, [4], 6), serve.Request(2, [8], 2)], speculative=False)
    assert {r.rid: r.tokens for r in done} == {0: stream([3], 1), 1: stream([4], 6), 2: stream([8], 2)}


def test_request_that_cannot_fit_is_refused():
    import pytest
    serve = entry.load_package().serve
    with pytest.raises(ValueError):
        serve.run(FakeEngine(1, 3, 32), [serve.Request(0, list(range(20)), 20)])


def test_sampled_serving_hands_each_request_its_draws_in_order():
    """The first draw of a request picks the token after its prompt; a sampled step gets k+1 draws per slot and consumes
    n_out + 1 of them when it rejected (n_out - 1 acceptance tests that passed, the one that failed and the residual draw),
    all k + 1 when the whole chain was accepted; the rest lead the next step."""
    serve = entry.load_package().serve

    class Counter:
        def __init__(self, base):
            self.n = base

        def random(self):
            self.n += 1
            return self.n / 1000.0

    class Eng(FakeEngine):
        def __init__(self, *a):
            super().__init__(*a)
            self.seen = []

        def mtp_step_sampled(self, u, **kw):
            assert kw == dict(temp=0.8, top_p=0.9, top_k=0, min_p=0.0)
            self.seen.append([list(r) for r in u])
            self.mtp_step()

    eng = Eng(2, 3, 256)
    reqs = [serve.Request(0, [1, 2], 9), serve.Request(1, [3], 7, arrival_step=2)]
    done = serve.run(eng, reqs, sampling=dict(temp=0.8, top_p=0.9, top_k=0, min_p=0.0), rng_of=lambda r: Counter(100 * r.rid))
    assert {r.rid: r.tokens for r in done} == {0: stream([1, 2], 9), 1: stream([3], 7)}
    used, emitted, budget = {0: [], 1: []}, {0: 1, 1: 1}, {0: 9, 1: 7}      # the prefill gave each its first token
    # replay: what each step consumed is the head of what it was handed, and the heads chain into 1, 2, 3, ... per request
    eng2 = FakeEngine(2, 3, 256)
    eng2.prefill(0, [1, 2])
    for step, u in enumerate(eng.seen):
        if step == 2:
            eng2.reset(1)
            eng2.prefill(1, [3])
        eng2.mtp_step()
        out = eng2.read_output()
        for s in (0, 1):
            if eng2.prompt[s] is not None and emitted[s] < budget[s]:
                n = len(out[s])
                used[s] += u[s][:4 if n == 4 else n + 1]
                emitted[s] += n
    assert eng.first_draws == {(1, 2): 0.001, (3,): 0.101}
    for s, base in ((0, 0), (1, 100)):
        got = [round(v * 1000) for v in used[s]]
        assert len(got) >= budget[s] - 1 and got == list(range(base + 2, base + 2 + len(got)))


class CompactEngine(FakeEngine):
    """FakeEngine with the active-prefix count, slot swap and appending prefill of binding.Batch."""

    def __init__(self, *a):
        super().__init__(*a)
        self.n_active = self.n_seqs
        self.stepped = 0                                  # sequence-steps actually computed

    def set_active(self, n):
        assert 0 <= n <= self.n_seqs
        self.n_active = n

    def swap(self, a, b):
        for arr in (self.prompt, self.emitted, self.pos, self.out):
            arr[a], arr[b] = arr[b], arr[a]

    def prefill(self, s, tokens, more=False):
        assert s >= self.n_active, "prefill into a slot the decode steps are running"
        self.prompt[s] = (self.prompt[s] or []) + list(tokens)
        self.pos[s] += len(tokens)
        if more:                                          # a part of the prompt: no token is chosen
            self.out[s], self.emitted[s] = [], 0
            return
        assert self.emitted[s] == 0, "a token was chosen before the prompt was complete"
        self.out[s] = stream(self.prompt[s], 1)
        self.emitted[s] = 1

    def reset(self, s):
        super().reset(s)
        self.emitted[s] = 0

    def _step(self, width):
        self.steps += 1
        for s in range(self.n_active):
            assert self.prompt[s] is not None, "an empty slot inside the active range"
            n = 1 + (self.steps + s) % width
            assert self.pos[s] < self.max_ctx
            self.pos[s] += n
            full = stream(self.prompt[s], self.emitted[s] + n)
            self.out[s] = full[self.emitted[s]:]
            self.emitted[s] += n
            self.stepped += 1


import pytest as _pytest


@_pytest.mark.parametrize("chunk", [0, 3])
def test_compacting_loop_keeps_live_requests_in_the_first_slots(chunk):
    serve = entry.load_package().serve
    eng = CompactEngine(3, 3, 512)
    spec = [(5, 9, 0), (11, 30, 0), (2, 4, 0), (7, 12, 1), (9, 6, 2), (4, 1, 3), (13, 20, 40)]
    reqs = [serve.Request(i, list(range(i, i + n)), new, arrival_step=a) for i, (n, new, a) in enumerate(spec)]
    done = serve.run_compact(eng, reqs, prefill_chunk=chunk)
    assert sorted(r.rid for r in done) == list(range(len(spec)))
    for r in done:
        assert r.tokens == stream(r.prompt, r.max_new_tokens), r.rid
    assert eng.n_active == 0
    # no sequence-step was spent on an empty slot: the steps computed are bounded by what the requests needed
    assert eng.stepped <= sum(new for _, new, _ in spec)


def test_compacting_loop_sampled_draws_follow_the_request_through_swaps():
    serve = entry.load_package().serve

    class Eng(CompactEngine):
        def __init__(self, *a):
            super().__init__(*a)
            self.first = {}

        def mtp_step_sampled(self, u, **kw):
            for s in range(self.n_active):
                key = tuple(self.prompt[s])
                self.first.setdefault(key, []).append(u[s][0])
            self.mtp_step()

    class Counter:
        def __init__(self, base):
            self.n = base

        def random(self):
            self.n += 1
            return float(self.n)

    eng = Eng(2, 1, 256)
    reqs = [serve.Request(i, [i + 1], new, arrival_step=0) for i, new in enumerate([3, 12, 7])]
    done = serve.run_compact(eng, reqs, sampling=dict(temp=1.0, top_p=1.0, top_k=0, min_p=0.0), rng_of=lambda r: Counter(1000 * r.rid))
    assert {r.rid: r.tokens for r in done} == {i: stream([i + 1], new) for i, new in enumerate([3, 12, 7])}
    for i in range(3):
        heads = eng.first[(i + 1,)]
        assert eng.first_draws[(i + 1,)] == 1000 * i + 1        # the request's first draw picked its first token
        assert heads[0] == 1000 * i + 2 and all(b > a for a, b in zip(heads, heads[1:])) and all(1000 * i < h < 1000 * (i + 1) for h in heads)


def test_pooled_engine_admits_only_what_its_page_pool_can_hold():
    """With one page pool for all slots a request is admitted when the pages of its whole life fit beside those promised to
    the requests already in; the others wait in arrival order, and everybody still gets the stream they get alone."""
    serve = entry.load_package().serve

    class Pooled(CompactEngine):
        page_size, pool_pages = 16, 6

        def __init__(self, *a):
            super().__init__(*a)
            self.held = [0] * self.n_seqs
            self.peak = 0

        def _pages(self, s):
            return -(-(self.pos[s] + self.k + 1) // self.page_size) if self.prompt[s] is not None else 0

        def _account(self):
            used = sum(self._pages(s) for s in range(self.n_seqs))
            assert used <= self.pool_pages, "the loop let the pool run dry"
            self.peak = max(self.peak, used)

        def prefill(self, s, tokens, more=False):
            super().prefill(s, tokens, more)
            self._account()

        def _step(self, width):
            super()._step(width)
            self._account()

    eng = Pooled(4, 3, 256)
    # lives of 3, 3, 2 and 4 pages: the third waits for a retirement although a slot is free, the fourth for two
    spec = [(20, 20), (30, 10), (10, 14), (40, 16)]
    reqs = [serve.Request(i, list(range(i, i + n)), new) for i, (n, new) in enumerate(spec)]
    done = serve.run_compact(eng, reqs)
    assert sorted(r.rid for r in done) == [0, 1, 2, 3]
    for r in done:
        assert r.tokens == stream(r.prompt, r.max_new_tokens), r.rid
    assert reqs[2].admitted_step > 0 and reqs[3].admitted_step >= reqs[2].admitted_step
    assert eng.peak <= 6
    with _pytest.raises(ValueError, match="pages"):
        serve.run_compact(Pooled(4, 3, 256), [serve.Request(9, list(range(100)), 20)])


def test_prefix_cache_policy_hits_longest_prefix_and_evicts_least_recently_used():
    """Requests whose prompts share page-aligned prefixes: a later one starts from the longest cached prefix (it ingests only
    the rest), everybody gets the stream they get alone, the table evicts its least recently used entry when it is full,
    and cached prefixes give way before a request has to wait for pages."""
    serve = entry.load_package().serve

    class Eng(CompactEngine):
        page_size, pool_pages = 16, 40

        def __init__(self, *a):
            super().__init__(*a)
            self.ingested = 0                      # prompt tokens that went through prefill
            self.entries = {}                      # handle -> tokens
            self.next_handle = 1

        def prefill(self, s, tokens, more=False):
            self.ingested += len(tokens)
            super().prefill(s, tokens, more)

        def prefix_capture(self, s, tokens):
            assert self.prompt[s] == list(tokens) and self.emitted[s] == 0 and len(tokens) % self.page_size == 0
            h = self.next_handle
            self.next_handle += 1
            self.entries[h] = list(tokens)
            return h

        def prefix_attach(self, s, h):
            assert self.prompt[s] is None and self.pos[s] == 0, "attach into a slot that is not empty"
            self.prompt[s] = list(self.entries[h])
            self.pos[s] = len(self.entries[h])
            self.out[s], self.emitted[s] = [], 0

        def prefix_release(self, h):
            del self.entries[h]

    system = list(range(1000, 1040))                          # 40 shared tokens: 2 whole pages
    prompts = [system + [7, 8, 9], system + [7, 8, 9, 10, 11], system[:20] + [5] * 30, system + [1], list(range(50))]
    eng = Eng(2, 3, 512)
    cache = serve.PrefixCache(eng, max_entries=2)
    reqs = [serve.Request(i, p, 6, arrival_step=4 * i) for i, p in enumerate(prompts)]
    done = serve.run_compact(eng, reqs, prefix_cache=cache)
    assert sorted(r.rid for r in done) == list(range(len(prompts)))
    for r in done:
        assert r.tokens == stream(r.prompt, r.max_new_tokens), r.rid
    # request 0 misses and leaves an entry of 32 tokens; 1 and 3 hit it (45 - 32 and 41 - 32 tokens ingested); 2 shares only
    # 20 tokens with the system prompt and no entry of 16 tokens exists: a miss that leaves its own entry (48 tokens); 4 is
    # unrelated: its entry pushes out the least recently used one, which is request 2's
    assert cache.hits == 2 and cache.misses == 3
    assert eng.ingested == 43 + (45 - 32) + 50 + (41 - 32) + 50
    assert cache.evictions == 1 and len(cache.table) == 2 and len(eng.entries) == 2
    # the entry the hits keep using survives the evictions
    assert tuple(system[:32]) in cache.table
    cache.clear()
    assert eng.entries == {}
    # pool pressure: with the pool nearly promised away a cached prefix is released rather than a request kept waiting
    eng2 = Eng(2, 3, 512)
    eng2.pool_pages = 7
    cache2 = serve.PrefixCache(eng2)
    a = serve.Request(0, list(range(100, 170)), 20)           # 70 + 20 + 4 -> 6 pages; leaves an entry of 64 tokens = 4 pages
    b = serve.Request(1, list(range(300, 340)), 20, arrival_step=40)   # 4 pages: fits only if the entry goes
    done2 = serve.run_compact(eng2, [a, b], prefix_cache=cache2)
    assert [r.rid for r in done2] == [0, 1] and cache2.evictions >= 1
    assert done2[1].tokens == stream(b.prompt, 20)
