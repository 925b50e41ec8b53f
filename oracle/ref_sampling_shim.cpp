// TEST INFRASTRUCTURE ONLY.  The reference's own sampler as a callable comparator: this translation unit includes
// src/qwen_native_backend.cpp where it lies (nothing is copied), which makes the file-local functions of its unnamed
// namespace reachable: apply_token_penalties (:262-280), sampling_distribution (:290-367), sample_from (:371-380),
// sample_token (:385-397) and speculative_accept_pointmass (:414-467).  The entry points below call them unchanged with
// a std::mt19937_64 seeded the way the generate loops seed theirs (options.seed, :11630 / :15390) and advanced by
// `skip` engine outputs, and report how many engine outputs the call consumed.  Linked against the reference's other
// host objects (oracle/Makefile target ref-sampling); nothing here is part of the product.
#include "qwen_native_backend.cpp"

#include <cstdint>

namespace {
uint64_t consumed_since(std::mt19937_64 before, const std::mt19937_64 &after, uint64_t limit) {
    for (uint64_t n = 0; n <= limit; ++n) {
        if (before == after) return n;
        before.discard(1);
    }
    return UINT64_MAX;
}
std::unordered_map<uint32_t, uint32_t> seen_map(const uint32_t *tok, const uint32_t *cnt, uint32_t n) {
    std::unordered_map<uint32_t, uint32_t> m;
    for (uint32_t i = 0; i < n; ++i) m[tok[i]] += cnt ? cnt[i] : 1u;
    return m;
}
}  // namespace

extern "C" {

// sampling_distribution on one row (penalties first when a seen set is given).
void rs_distribution(const float *logits, uint32_t n, float temp, float top_p, int32_t top_k, float min_p, float presence,
                     float repetition, const uint32_t *seen_tok, uint32_t n_seen, float *out) {
    std::vector<float> row(logits, logits + n);
    qw3::apply_token_penalties(row, seen_map(seen_tok, nullptr, n_seen), presence, repetition);
    const std::vector<float> p = qw3::sampling_distribution(row, temp, top_p, top_k, min_p);
    for (uint32_t i = 0; i < n; ++i) out[i] = p[i];
}

// `count` successive sample_token calls on the rows of `logits` ([count][n]) from one generator.
void rs_sample_tokens(const float *logits, uint32_t count, uint32_t n, float temp, float top_p, int32_t top_k, float min_p,
                      uint64_t seed, uint64_t skip, int32_t *tokens, uint64_t *consumed) {
    std::mt19937_64 rng(seed);
    rng.discard(skip);
    const std::mt19937_64 start = rng;
    for (uint32_t r = 0; r < count; ++r) {
        std::vector<float> row(logits + (size_t)r * n, logits + (size_t)(r + 1) * n);
        tokens[r] = qw3::sample_token(row, temp, top_p, top_k, min_p, rng);
    }
    if (consumed) *consumed = consumed_since(start, rng, 4ull * count + 16);
}

// One speculative_accept_pointmass call: rows [n_drafts + 1][n]; result[0] = accepted, result[1] = extra token.
void rs_spec_accept(const float *rows, uint32_t n_drafts, uint32_t n, const uint32_t *drafts, float temp, float top_p, int32_t top_k,
                    float min_p, float presence, float repetition, const uint32_t *seen_tok, uint32_t n_seen, uint64_t seed,
                    uint64_t skip, int32_t *result, uint64_t *consumed) {
    std::vector<std::vector<float>> target(n_drafts + 1);
    for (uint32_t r = 0; r <= n_drafts; ++r) target[r].assign(rows + (size_t)r * n, rows + (size_t)(r + 1) * n);
    const std::vector<uint32_t> d(drafts, drafts + n_drafts);
    std::mt19937_64 rng(seed);
    rng.discard(skip);
    const std::mt19937_64 start = rng;
    const qw3::SpecAcceptResult r = qw3::speculative_accept_pointmass(target, d, temp, top_p, top_k, min_p, presence, repetition,
                                                                      seen_map(seen_tok, nullptr, n_seen), rng);
    result[0] = (int32_t)r.accepted;
    result[1] = r.extra_token;
    if (consumed) *consumed = consumed_since(start, rng, 2ull * n_drafts + 16);
}

// The generator as the reference's loops see it: `count` outputs of uniform_real_distribution<double>(0, 1) after `skip`
// engine outputs (the accept test's draw, :423 / :448); pins the replay of the generator used by the tests.
void rs_unit_draws(uint64_t seed, uint64_t skip, uint32_t count, double *out) {
    std::mt19937_64 rng(seed);
    rng.discard(skip);
    std::uniform_real_distribution<double> unit(0.0, 1.0);
    for (uint32_t i = 0; i < count; ++i) out[i] = unit(rng);
}

}  // extern "C"
