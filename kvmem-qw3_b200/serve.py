"""Continuous-batching loop around the MTP step: request queue, admission into free sequence slots, retirement.

The host side of the reference's continuous_batch_worker_loop (src/qwen_native_backend.cpp:6711-6866: pending queue,
`max_active` slots, admission when a slot is free, retirement at EOS or at the token budget) over the fixed-slot batch of
this library: a batch has `n_slots` sequences; a retired request's slot is recycled with Batch.reset (position 0, zero
recurrent state) and the next pending request is prefilled into it while the others keep decoding.  Every step runs all
slots (an idle slot decodes from its reset state and is reset again before it runs out of context); because a row's
result never depends on which other rows share a launch, a request's tokens are the ones it would get alone.

`engine` is anything with n_seqs, k, max_ctx, prefill(seq, tokens, more=False), prefill_sampled(seq, tokens, u, **sampling),
mtp_step() / mtp_step_sampled(u, **sampling) or greedy_step(), read_output(), reset(seq):
binding.Batch on the GPU, a fake in the CPU tests.
"""
import collections


class Request:
    def __init__(self, rid, prompt, max_new_tokens, arrival_step=0, eos=None):
        self.rid, self.prompt, self.max_new_tokens = rid, list(prompt), int(max_new_tokens)
        self.arrival_step, self.eos = int(arrival_step), eos
        self.tokens = []            # emitted tokens (the first one comes from the prefill's last row)
        self.admitted_step = self.finished_step = None
        self.slot = None

    def done(self):
        return len(self.tokens) >= self.max_new_tokens or (self.eos is not None and self.eos in self.tokens)

    def _trim(self):
        if self.eos is not None and self.eos in self.tokens:
            self.tokens = self.tokens[:self.tokens.index(self.eos) + 1]
        self.tokens = self.tokens[:self.max_new_tokens]


class SlotScheduler:
    """FIFO admission into a fixed number of slots; free slots are reused last-freed-first (the LIFO order of the
    reference's page pool, src/qwen_native_backend.cpp:1155-1265)."""

    def __init__(self, n_slots):
        self.free = list(range(n_slots - 1, -1, -1))     # pop() hands out slot 0 first
        self.pending = collections.deque()
        self.active = {}                                 # slot -> Request

    def submit(self, req):
        self.pending.append(req)

    def admissible(self, step):
        """Requests that can be admitted now: arrived, in arrival order, one per free slot."""
        out = []
        while self.pending and self.free and self.pending[0].arrival_step <= step:
            req = self.pending.popleft()
            req.slot = self.free.pop()
            req.admitted_step = step
            self.active[req.slot] = req
            out.append(req)
        return out

    def retire(self, slot, step):
        req = self.active.pop(slot)
        req.finished_step = step
        self.free.append(slot)
        return req

    def idle(self):
        return not self.pending and not self.active


class DrawQueue:
    """Uniform draws of one request in the order the reference consumes its generator (one std::mt19937_64 per request,
    src/qwen_native_backend.cpp:399-467): the first draw picks the token after the prompt (pick_from_last_logits,
    :15399-15428); a sampled step is handed k+1 draws; one that rejects after a acceptances has used a + 2 of them (a + 1
    acceptance tests and the residual draw), a fully accepted chain all k + 1; the rest stay at the head of the queue."""

    def __init__(self, rng, width):
        self.rng, self.width, self.buf = rng, width, []

    def peek(self):
        while len(self.buf) < self.width:
            self.buf.append(float(self.rng.random()))
        return self.buf[:self.width]

    def consume(self, n):
        del self.buf[:n]

    def consume_step(self, n_out, depth=None):
        """Draws used by a speculative step of chain depth `depth` (default: the full width - 1) that emitted n_out tokens
        (accepted drafts + the residual or bonus token): a fully accepted chain depth + 1, a rejecting one n_out + 1."""
        depth = self.width - 1 if depth is None else min(depth, self.width - 1)
        self.consume(depth + 1 if n_out >= depth + 1 else n_out + 1)

    def take(self):
        v = self.peek()[0]
        self.consume(1)
        return v


class PrefixCache:
    """Host policy over the engine's shared-prefix entries (prefix_capture / prefix_attach / prefix_release), the role of the
    reference server's prefix cache (src/qwen_native_backend.cpp:9785-10410): a prompt is looked up by its page-aligned
    prefixes, longest first; a hit seeds the request from the entry instead of ingesting those tokens; a miss ingests the
    prompt in two parts so that an entry of its page-aligned prefix can be taken; entries nobody has used for longest are
    released first when the page pool runs short or the table is full.  Entries hold K/V pages: `pages_held` is what the
    admission control of run_compact counts against the pool."""

    def __init__(self, engine, max_entries=16, min_tokens=None):
        self.engine, self.max_entries = engine, max_entries
        self.page = engine.page_size
        self.min_tokens = self.page if min_tokens is None else max(self.page, min_tokens)
        self.table = collections.OrderedDict()          # tuple(tokens) -> entry handle, least recently used first
        self.hits = self.misses = self.evictions = 0

    def aligned(self, n_prompt):
        """Longest prefix length an entry may have for a prompt of n_prompt tokens: whole pages, at least one token left."""
        n = (n_prompt - 1) // self.page * self.page
        return n if n >= self.min_tokens else 0

    def lookup(self, prompt):
        """(entry, n_tokens) of the longest cached page-aligned prefix of `prompt`, or (None, 0)."""
        n = self.aligned(len(prompt))
        while n >= self.min_tokens:
            key = tuple(prompt[:n])
            if key in self.table:
                self.table.move_to_end(key)
                self.hits += 1
                return self.table[key], n
            n -= self.page
        self.misses += 1
        return None, 0

    def wants(self, prompt):
        """Prefix length to take an entry of while this prompt is ingested (0: none, or already there)."""
        n = self.aligned(len(prompt))
        return n if n and tuple(prompt[:n]) not in self.table else 0

    def insert(self, slot, tokens):
        while len(self.table) >= self.max_entries and self.evict_one():
            pass
        if len(self.table) >= self.max_entries:
            return False
        self.table[tuple(tokens)] = self.engine.prefix_capture(slot, list(tokens))
        return True

    def evict_one(self):
        if not self.table:
            return False
        _, entry = self.table.popitem(last=False)
        self.engine.prefix_release(entry)
        self.evictions += 1
        return True

    def pages_held(self):
        return sum(len(k) // self.page for k in self.table)

    def clear(self):
        while self.evict_one():
            pass


def run_compact(engine, requests, speculative=True, max_steps=1 << 30, sampling=None, rng_of=None, prefill_chunk=0, prefix_cache=None):
    """The loop for engines with set_active(n) and swap(s1, s2): live requests are kept in slots [0, n_live) and only those
    are decoded; a retiring request's slot is filled by the last live one (swap), a new request is ingested in a slot
    beyond the live range -- `prefill_chunk` tokens per iteration when that is set, so decoding goes on meanwhile -- and
    swapped to the end of the live range when its prompt is in.  prefix_cache: a PrefixCache over the same (pooled) engine:
    admitted requests start from the longest cached prefix of their prompt, and leave an entry of their own."""
    pending = collections.deque(sorted(requests, key=lambda r: (r.arrival_step, r.rid)))
    per_step = engine.k + 1 if speculative else 1
    if sampling is not None:
        if not speculative:
            raise ValueError("sampled decode runs through the speculative step")
        sampling = dict(sampling)
        presence, repetition = sampling.pop("presence", 0.0), sampling.pop("repetition", 1.0)
        if presence != 0.0 or repetition != 1.0:
            engine.set_penalties(presence, repetition)
    live = []                                            # live[s] = request in slot s
    ingest = {}                                          # slot -> [request, tokens ingested]
    draws = {}                                           # rid -> DrawQueue
    finished, step = [], 0
    engine.set_active(0)
    # an engine with one K/V page pool for all slots (binding.Batch(pool_pages=...)): a request is admitted only when the
    # pages of its whole life (prompt + budget + one step's rows) fit beside those promised to the requests already in,
    # so a decode step never finds the pool empty; requests wait in arrival order
    pool_pages = getattr(engine, "pool_pages", 0)
    reserved = {}                                        # rid -> pages promised

    def pages_of(req):
        return -(-(len(req.prompt) + req.max_new_tokens + per_step) // engine.page_size)

    def retire(s):
        req = live[s]
        reserved.pop(req.rid, None)
        req.finished_step = step
        req._trim()
        finished.append(req)
        last = len(live) - 1
        if s != last:
            engine.swap(s, last)
            live[s] = live[last]
            live[s].slot = s
        live.pop()
        engine.set_active(len(live))
        if pool_pages:
            engine.reset(last)                           # the retired request's pages go back to the pool now, not at the next admission

    while (pending or live or ingest) and step < max_steps:
        # admission: a free slot beyond the live range per arrived request
        while pending and pending[0].arrival_step <= step and len(live) + len(ingest) < engine.n_seqs:
            req = pending[0]
            if len(req.prompt) + req.max_new_tokens + per_step > engine.max_ctx:
                raise ValueError("request %r does not fit max_ctx %d" % (req.rid, engine.max_ctx))
            if pool_pages:
                if pages_of(req) > pool_pages:
                    raise ValueError("request %r needs %d pages, the pool has %d" % (req.rid, pages_of(req), pool_pages))
                held = prefix_cache.pages_held() if prefix_cache else 0
                while sum(reserved.values()) + held + pages_of(req) > pool_pages and prefix_cache and prefix_cache.evict_one():
                    held = prefix_cache.pages_held()               # cached prefixes make room before a request has to wait
                if sum(reserved.values()) + held + pages_of(req) > pool_pages:
                    break                                          # waits for a retirement
                reserved[req.rid] = pages_of(req)
            pending.popleft()
            slot = next(s for s in range(len(live), engine.n_seqs) if s not in ingest)
            engine.reset(slot)
            req.slot, req.admitted_step = slot, step
            done_n = 0
            if prefix_cache:
                entry, done_n = prefix_cache.lookup(req.prompt)
                if entry is not None:
                    engine.prefix_attach(slot, entry)
            ingest[slot] = [req, done_n]
        # ingestion: one chunk per request and iteration (the whole prompt when prefill_chunk is 0)
        for slot in sorted(ingest):
            if slot not in ingest:                                 # moved by a swap earlier in this iteration
                continue
            req, done_n = ingest[slot]
            n = len(req.prompt) - done_n if not prefill_chunk else min(prefill_chunk, len(req.prompt) - done_n)
            cut = prefix_cache.wants(req.prompt) if prefix_cache else 0
            if cut > done_n:                                       # stop at the page-aligned prefix: an entry is taken there
                n = min(n, cut - done_n)
            final = done_n + n == len(req.prompt)
            if not final:
                engine.prefill(slot, req.prompt[done_n:done_n + n], more=True)     # no token is chosen, nothing counted
            elif sampling is not None:
                draws[req.rid] = DrawQueue(rng_of(req), per_step)
                engine.prefill_sampled(slot, req.prompt[done_n:], draws[req.rid].take(), **sampling)
            else:
                engine.prefill(slot, req.prompt[done_n:])
            ingest[slot][1] = done_n + n
            if prefix_cache and cut and done_n + n == cut:
                prefix_cache.insert(slot, req.prompt[:cut])
            if not final:
                continue
            req.tokens.extend(engine.read_output()[slot])          # the prefill's last row gives the first token
            del ingest[slot]
            target = len(live)
            if slot != target:                                     # to the end of the live range
                engine.swap(slot, target)
                if target in ingest:
                    ingest[slot] = ingest.pop(target)
                    ingest[slot][0].slot = slot
            req.slot = target
            live.append(req)
            engine.set_active(len(live))
            if req.done():
                retire(target)
        if not live:
            step += 1
            continue
        if sampling is not None:
            u = [draws[live[s].rid].peek() if s < len(live) else [0.5] * per_step for s in range(engine.n_seqs)]
            engine.mtp_step_sampled(u, **sampling)
        elif speculative:
            engine.mtp_step()
        else:
            engine.greedy_step()
        out = engine.read_output()
        step += 1
        for s in range(len(live) - 1, -1, -1):           # from the end: retiring swaps the last live request in
            req = live[s]
            req.tokens.extend(out[s])
            if sampling is not None:
                draws[req.rid].consume_step(len(out[s]))
            if req.done():
                retire(s)
    return finished


def run(engine, requests, speculative=True, max_steps=1 << 30, sampling=None, rng_of=None):
    """Serve `requests` (a list of Request) to completion; returns them in completion order.
    One loop iteration = admissions (a prefill each) + one decode step of the whole batch.
    sampling: None (greedy) or dict(temp=, top_p=, top_k=, min_p=[, presence=, repetition=]) for engine.mtp_step_sampled (the
    penalties go to engine.set_penalties); rng_of(request) gives the
    request's generator (anything with .random() -> float in [0, 1))."""
    sched = SlotScheduler(engine.n_seqs)
    for r in sorted(requests, key=lambda r: (r.arrival_step, r.rid)):
        sched.submit(r)
    per_step = engine.k + 1 if speculative else 1
    idle_pos = [0] * engine.n_seqs                       # upper bound of the position of slots that hold no request
    if sampling is not None and not speculative:
        raise ValueError("sampled decode runs through the speculative step")
    draws = {}                                           # slot -> DrawQueue of the request it holds
    if sampling is not None:
        sampling = dict(sampling)
        presence, repetition = sampling.pop("presence", 0.0), sampling.pop("repetition", 1.0)
        if presence != 0.0 or repetition != 1.0:
            engine.set_penalties(presence, repetition)   # before any prefill: the prompts count as seen tokens
    finished, step = [], 0
    while not sched.idle() and step < max_steps:
        for req in sched.admissible(step):
            if len(req.prompt) + req.max_new_tokens + per_step > engine.max_ctx:
                raise ValueError("request %r does not fit max_ctx %d" % (req.rid, engine.max_ctx))
            engine.reset(req.slot)
            if sampling is not None:
                draws[req.slot] = DrawQueue(rng_of(req), per_step)
                engine.prefill_sampled(req.slot, req.prompt, draws[req.slot].take(), **sampling)
            else:
                engine.prefill(req.slot, req.prompt)
            req.tokens.extend(engine.read_output()[req.slot])      # the prefill's last row gives the first token
            if req.done():
                req._trim()
                finished.append(sched.retire(req.slot, step))
                idle_pos[req.slot] = len(req.prompt) + per_step
        if not sched.active:                             # nothing to decode yet: wait for the next arrival
            step += 1
            continue
        for s in range(engine.n_seqs):                   # idle slots must not run out of context
            if s not in sched.active and idle_pos[s] + 2 * per_step >= engine.max_ctx:
                engine.reset(s)
                idle_pos[s] = 0
        if sampling is not None:
            u = [draws[s].peek() if s in sched.active else [0.5] * per_step for s in range(engine.n_seqs)]
            engine.mtp_step_sampled(u, **sampling)
        elif speculative:
            engine.mtp_step()
        else:
            engine.greedy_step()
        out = engine.read_output()
        step += 1
        for s in range(engine.n_seqs):
            req = sched.active.get(s)
            if req is None:
                idle_pos[s] += per_step
                continue
            req.tokens.extend(out[s])
            if sampling is not None:
                draws[s].consume_step(len(out[s]))
            if req.done():
                req._trim()
                finished.append(sched.retire(s, step))
                idle_pos[s] = len(req.prompt) + len(req.tokens) + per_step
    return finished
