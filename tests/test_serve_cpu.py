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

    def prefill(self, s, tokens):
        assert self.pos[s] == 0, "prefill into a slot that was not reset"
        self.prompt[s] = list(tokens)
        self.pos[s] = len(tokens)
        self.out[s] = stream(self.prompt[s], 1)
        self.emitted[s] = 1

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
