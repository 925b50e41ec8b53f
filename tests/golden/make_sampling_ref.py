"""Golden vectors of the reference's sampler for the speculative acceptance in sampling mode.

The cases are seeded (cases() below builds them from numpy generators, so only the RESULTS are stored); the results come
from the reference's own functions -- apply_token_penalties, sampling_distribution, sample_from, sample_token and
speculative_accept_pointmass of src/qwen_native_backend.cpp -- called through oracle/_ref/libqw3ref_sampling.so
(oracle/Makefile target ref-sampling, which compiles that source file where it lies).  Run where the reference tree is
present:

    make -C oracle ref-sampling REF=<reference tree> && python tests/golden/make_sampling_ref.py

Writes tests/golden/sampling_ref.npz: per case the accepted length, the residual / bonus token, the number of generator
outputs consumed, and for the first row of the case the count of nonzero probabilities, their float64 sum and p[draft].
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "sampling_ref.npz")
N_CASES = 240


def cases():
    """Seeded case list: dict(rows [k+1][V] f32, drafts [k], temp, top_p, top_k, min_p, presence, repetition, seen, seed, skip)."""
    out = []
    for c in range(N_CASES):
        g = np.random.default_rng(0xACCE97 + c)
        V = int(g.choice([50, 1000, 4096, 4096, 32000])) if c % 40 else 151936
        k = int(g.choice([1, 3, 3, 5]))
        scale = float(g.choice([0.5, 2.0, 4.0, 8.0]))
        rows = (g.standard_normal((k + 1, V)) * scale).astype(np.float32)
        ties = c % 7 == 3
        if ties:
            rows = (np.round(rows * 2.0) / 2.0).astype(np.float32)      # many exactly equal logits
        temp = float(g.choice([0.3, 0.6, 1.0, 1.5]))
        if ties:
            top_k, top_p = 0, 1.0                                       # the order of equal logits is the sort's own business
            min_p = float(g.choice([0.0, 0.2]))
        else:
            top_k = int(g.choice([0, 0, 1, 2, 20, 200, V + 5]))
            top_p = float(g.choice([1.0, 0.95, 0.8, 0.5, 0.05]))
            min_p = float(g.choice([0.0, 0.0, 0.05, 0.5]))
        pen = c % 3 == 1
        presence = float(g.choice([0.5, 1.5])) if pen else 0.0
        repetition = float(g.choice([1.0, 1.2, 0.8])) if pen else 1.0
        seen = sorted(set(int(t) for t in g.integers(0, V, size=int(g.integers(0, 60)))))
        drafts = []
        for i in range(k):
            order = np.argsort(-rows[i], kind="stable")
            how = int(g.integers(0, 4))
            drafts.append(int(order[0]) if how < 2 else int(order[int(g.integers(0, 5))]) if how == 2 else int(g.integers(0, V)))
        if pen and seen and k > 1:
            drafts[1] = drafts[0] if c % 2 else drafts[1]                # an accepted draft penalises itself in the next row
        out.append(dict(rows=rows, drafts=np.array(drafts, np.uint32), temp=temp, top_p=top_p, top_k=top_k, min_p=min_p,
                        presence=presence, repetition=repetition, seen=seen, seed=int(g.integers(0, 2 ** 62)), skip=int(g.integers(0, 700))))
    return out


def penalise(row, toks, presence, repetition):
    """apply_token_penalties (src/qwen_native_backend.cpp:262-280) in float32."""
    use_rep = repetition > 0.0 and repetition != 1.0
    if not toks or (presence == 0.0 and not use_rep):
        return row
    row = row.copy()
    idx = np.array(sorted(t for t in toks if t < row.size), np.int64)
    v = row[idx]
    if use_rep:
        v = np.where(v >= 0, v / np.float32(repetition), v * np.float32(repetition)).astype(np.float32)
    if presence != 0.0:
        v = (v - np.float32(presence)).astype(np.float32)
    row[idx] = v
    return row


def oracle_spec_accept(orc, case, gen):
    """The accept loop on the CPU oracle's sampler with the draws taken from `gen` (an MT64) in the reference's order: one
    uniform per acceptance test; one for the residual or bonus token unless fewer than two tokens are left to choose
    from (std::discrete_distribution draws nothing then).  Returns (accepted, extra token, draws consumed)."""
    c, start = case, gen.count
    ctxset, accepted = set(c["seen"]), 0
    args = (c["temp"], c["top_p"], c["top_k"], c["min_p"])
    k = len(c["drafts"])
    for i in range(k + 1):
        row = penalise(c["rows"][i], ctxset, c["presence"], c["repetition"])
        p = orc.sampling_distribution(row, *args)
        nnz = int(np.count_nonzero(p > 0))
        if i == k:
            u = gen.unit() if nnz >= 2 else 0.5
            tok, _, _ = orc.sample_rows(row[None], np.array([-1], np.int32), np.zeros(1), np.array([u]), *args)
            return accepted, int(tok[0]), gen.count - start
        d = int(c["drafts"][i])
        ua = np.array([gen.unit()])
        _, acc, _ = orc.sample_rows(row[None], np.array([d], np.int32), ua, ua, *args)
        if acc[0]:
            ctxset.add(d)
            accepted += 1
            continue
        left = nnz - int(p[d] > 0)
        u = gen.unit() if left >= 2 else 0.5
        tok, _, _ = orc.sample_rows(row[None], np.array([d], np.int32), np.array([2.0]), np.array([u]), *args)
        return accepted, int(tok[0]), gen.count - start
    raise AssertionError("unreachable")


def main():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_sampling as R
    if not R.available():
        raise SystemExit("oracle/_ref/libqw3ref_sampling.so is missing: make -C oracle ref-sampling REF=<reference tree>")
    cs = cases()
    acc, extra, used, nnz, psum, pd = [], [], [], [], [], []
    for c in cs:
        a, e, n = R.spec_accept(c["rows"], c["drafts"], c["temp"], c["top_p"], c["top_k"], c["min_p"], c["presence"], c["repetition"],
                                c["seen"], c["seed"], c["skip"])
        p = R.distribution(c["rows"][0], c["temp"], c["top_p"], c["top_k"], c["min_p"], c["presence"], c["repetition"], c["seen"])
        acc.append(a); extra.append(e); used.append(n)
        nnz.append(int(np.count_nonzero(p > 0))); psum.append(float(p.astype(np.float64).sum())); pd.append(p[int(c["drafts"][0])])
    # the generator itself: outputs 1, 2, 10000 of a default-seeded engine are checked in the test against the
    # value the C++ standard states; here the first draws of a few seeds as the reference's distribution object makes them
    seeds = np.array([0, 1, 5489, 123456789012345], np.uint64)
    draws = np.stack([R.unit_draws(int(s), 3, 8) for s in seeds])
    np.savez(OUT, accepted=np.array(acc, np.int32), extra=np.array(extra, np.int32), consumed=np.array(used, np.int32),
             nnz=np.array(nnz, np.int64), psum=np.array(psum, np.float64), p_draft=np.array(pd, np.float32), draw_seeds=seeds, draws=draws)
    print("wrote", OUT, "accepted histogram", np.bincount(acc).tolist(), "consumed histogram", np.bincount(used).tolist())


if __name__ == "__main__":
    main()
