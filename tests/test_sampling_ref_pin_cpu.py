"""Pins the CPU oracle's sampler (sampling_distribution, the acceptance test, the residual / bonus / first-token draw and
the order in which they consume one generator) on the reference's own functions: against the committed results of
tests/golden/sampling_ref.npz everywhere, and against oracle/_ref/libqw3ref_sampling.so itself (the reference's
src/qwen_native_backend.cpp compiled where it lies) when that library has been built.  No GPU."""
import os
import sys

import numpy as np
import pytest

from conftest import ROOT

sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
import make_sampling_ref as G  # noqa: E402
import ref_sampling as R  # noqa: E402

GOLD = os.path.join(ROOT, "tests", "golden", "sampling_ref.npz")


def test_mt64_replay_known_answer():
    """The C++ standard fixes the 10000th output of a default-constructed std::mt19937_64."""
    g = R.MT64()
    g.discard(9999)
    assert g.next_u64() == 9981545732273789042
    # the draws of uniform_real_distribution<double>(0, 1) as the reference's build makes them
    gold = np.load(GOLD)
    for seed, want in zip(gold["draw_seeds"], gold["draws"]):
        g = R.MT64(int(seed))
        g.discard(3)
        assert [g.unit() for _ in range(8)] == want.tolist()


def test_oracle_accept_loop_matches_reference_golden(orc):
    gold = np.load(GOLD)
    cs = G.cases()
    assert len(cs) == gold["accepted"].size
    seen_consumed = set()
    for i, c in enumerate(cs):
        gen = R.MT64(c["seed"])
        gen.discard(c["skip"])
        gen.count = 0
        a, e, n = G.oracle_spec_accept(orc, c, gen)
        assert (a, e, n) == (int(gold["accepted"][i]), int(gold["extra"][i]), int(gold["consumed"][i])), (i, a, e, n)
        row = G.penalise(c["rows"][0], set(c["seen"]), c["presence"], c["repetition"])
        p = orc.sampling_distribution(row, c["temp"], c["top_p"], c["top_k"], c["min_p"])
        assert int(np.count_nonzero(p > 0)) == int(gold["nnz"][i]), i
        assert abs(float(p.astype(np.float64).sum()) - float(gold["psum"][i])) < 1e-6
        assert p[int(c["drafts"][0])] == gold["p_draft"][i], i
        seen_consumed.add((a, n - a))
    # the vectors cover rejections with and without a residual draw, and full acceptance with and without a bonus draw
    assert {1, 2} <= {n for _, n in seen_consumed}, seen_consumed
    assert np.bincount(gold["accepted"]).size >= 4


@pytest.mark.skipif(not R.available(), reason="oracle/_ref/libqw3ref_sampling.so not built (make -C oracle ref-sampling REF=<reference tree>)")
def test_oracle_sampler_matches_reference_library_live(orc):
    """Bit-exact distributions row by row, the acceptance result, and plain sampling (sample_token) on one generator."""
    cs = G.cases()
    for i, c in enumerate(cs[:120]):
        ctxset = set(c["seen"])
        for r in range(c["rows"].shape[0]):
            want = R.distribution(c["rows"][r], c["temp"], c["top_p"], c["top_k"], c["min_p"], c["presence"], c["repetition"], ctxset)
            got = orc.sampling_distribution(G.penalise(c["rows"][r], ctxset, c["presence"], c["repetition"]), c["temp"], c["top_p"], c["top_k"], c["min_p"])
            assert np.array_equal(want.view(np.uint32), got.view(np.uint32)), (i, r, np.abs(want - got).max())
        gen = R.MT64(c["seed"]); gen.discard(c["skip"]); gen.count = 0
        assert G.oracle_spec_accept(orc, c, gen) == R.spec_accept(c["rows"], c["drafts"], c["temp"], c["top_p"], c["top_k"], c["min_p"],
                                                                  c["presence"], c["repetition"], c["seen"], c["seed"], c["skip"]), i
        if not c["presence"] and c["repetition"] == 1.0:
            # sample_token on every row from one generator (the plain decode loop's pick_next)
            want_tok, used = R.sample_tokens(c["rows"], c["temp"], c["top_p"], c["top_k"], c["min_p"], c["seed"], c["skip"])
            gen = R.MT64(c["seed"]); gen.discard(c["skip"]); gen.count = 0
            got = []
            for row in c["rows"]:
                p = orc.sampling_distribution(row, c["temp"], c["top_p"], c["top_k"], c["min_p"])
                u = gen.unit() if np.count_nonzero(p > 0) >= 2 else 0.5
                t, _, _ = orc.sample_rows(row[None], np.array([-1], np.int32), np.zeros(1), np.array([u]), c["temp"], c["top_p"], c["top_k"], c["min_p"])
                got.append(int(t[0]))
            assert got == want_tok.tolist() and gen.count == used, i
