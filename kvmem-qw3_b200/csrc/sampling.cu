// Sampling-mode speculative acceptance on the device.
//
// The reference pulls the verifier's logits to the host for non-greedy requests and runs
// sampling_distribution + speculative_accept_pointmass there (src/qwen_native_backend.cpp:282-370, 399-467).
// Here one CTA per logits row builds the same distribution in place -- softmax(logits / temp), then the top-k,
// min-p and nucleus truncations, each a prefix of the descending order, renormalised over the kept set -- and
// takes the row's decision: accept the (greedy, point-mass) draft with probability p[draft]; on rejection draw
// from p with the draft removed; a row without a draft draws from p (the bonus token, or plain sampling).
// The uniform draws come from the caller, in the order the reference's generator would be consumed.
//
// The kept set is found without sorting: the descending order is the order of a monotone 32-bit key of the
// logit, and "the shortest prefix that reaches top_p or the count limit" is a bisection over that key with one
// pass over the row per step (count and probability mass of the keys at or above the probe).  Ties at the
// boundary key are taken lowest index first.
#include "qb_internal.h"

#include <cfloat>

namespace {

constexpr int ST = 1024;                      // threads per row

struct SampleParams {
    float inv_t, top_p, min_p;
    int top_k;
};

__device__ __forceinline__ uint32_t okey(float f) {      // ascending key order == ascending float order
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

template <typename T, typename Op>
__device__ T block_reduce(T v, Op op, T *scratch) {       // all threads get the result; scratch: 32 entries
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();                                       // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    T r = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = op(r, __shfl_xor_sync(0xffffffffu, r, o));
    return r;
}

struct OpSumD { __device__ double operator()(double a, double b) const { return a + b; } };
struct OpSumU { __device__ unsigned long long operator()(unsigned long long a, unsigned long long b) const { return a + b; } };
struct OpMaxF { __device__ float operator()(float a, float b) const { return fmaxf(a, b); } };
struct OpMinI { __device__ int operator()(int a, int b) const { return a < b ? a : b; } };
struct OpMaxI { __device__ int operator()(int a, int b) const { return a > b ? a : b; } };

// exclusive prefix over the threads of the block (thread order) of a double and a count; totals returned too
__device__ void block_exscan(double v, unsigned int c, double &ex_v, unsigned int &ex_c, double &tot_v, unsigned int &tot_c,
                             double *sv, unsigned int *sc) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    double iv = v;
    unsigned int ic = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double nv = __shfl_up_sync(0xffffffffu, iv, o);
        const unsigned int nc = __shfl_up_sync(0xffffffffu, ic, o);
        if (lane >= (uint32_t)o) { iv += nv; ic += nc; }
    }
    __syncthreads();
    if (lane == 31) { sv[warp] = iv; sc[warp] = ic; }
    __syncthreads();
    double wv = 0.0;
    unsigned int wc = 0;
    tot_v = 0.0; tot_c = 0;
    for (uint32_t w = 0; w < ST / 32; ++w) {               // 32 entries, warp order = the summation order of a serial scan
        if (w < warp) { wv += sv[w]; wc += sc[w]; }
        tot_v += sv[w]; tot_c += sc[w];
    }
    ex_v = wv + (iv - v);
    ex_c = wc + (ic - c);
}

__device__ __forceinline__ float key_to_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// One CTA per row.  draft[row] < 0: no draft (bonus / plain sampling row).
__global__ void __launch_bounds__(ST)
sample_rows_kernel(const float *__restrict__ logits, uint32_t V, uint32_t stride, const int32_t *__restrict__ draft,
                   const double *__restrict__ u_acc, const double *__restrict__ u_res, SampleParams p, int32_t *token,
                   int32_t *accepted, float *p_draft, float *pval, int32_t *pidx, uint32_t nblk, uint32_t K1) {
    __shared__ double s_d[32];
    __shared__ unsigned long long s_u[32];
    __shared__ float s_f[32];
    __shared__ int s_i[32];
    __shared__ unsigned int s_c[32];
    QB_PDL_ENTER();
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const float *x = logits + (size_t)row * stride;

    // softmax(logits / temp): max, then the denominator in double (src/qwen_native_backend.cpp:296-303)
    float mx = -INFINITY;
    for (uint32_t i = tid; i < V; i += ST) mx = fmaxf(mx, x[i]);
    mx = block_reduce(mx, OpMaxF(), s_f);
    int top_idx = 0x7fffffff;
    double sum = 0.0;
    for (uint32_t i = tid; i < V; i += ST) {
        const float l = x[i];
        if (l == mx && (int)i < top_idx) top_idx = (int)i;
        sum += (double)expf((l - mx) * p.inv_t);
    }
    sum = block_reduce(sum, OpSumD(), s_d);
    top_idx = block_reduce(top_idx, OpMinI(), s_i);
    const float norm = (float)(1.0 / (sum > 0.0 ? sum : 1.0));
    auto prob = [&](float l) -> float { return expf((l - mx) * p.inv_t) * norm; };

    const bool use_k = p.top_k > 0 && (uint32_t)p.top_k < V, use_p = p.top_p < 1.0f && p.top_p > 0.0f, use_m = p.min_p > 0.0f;
    const bool trunc = use_k || use_p || use_m;
    uint32_t B = 0;                 // boundary key: keys above it are kept, r_ties of the n_ties equal to it
    unsigned int r_ties = 0, n_ties = 0;
    float kn = 1.0f;
    bool degenerate = false;
    if (trunc) {
        unsigned long long L1 = use_k ? (unsigned long long)p.top_k : (unsigned long long)V;
        if (use_m) {                // min-p keeps the prefix whose probability is at least min_p times the top one (:333-338)
            const float cutoff = prob(mx) * p.min_p;
            unsigned long long c = 0;
            for (uint32_t i = tid; i < V; i += ST) c += prob(x[i]) >= cutoff ? 1u : 0u;
            c = block_reduce(c, OpSumU(), s_u);
            L1 = c < L1 ? c : L1;
        }
        if (L1 == 0) {
            degenerate = true;
        } else {
            // largest key t such that the elements with key >= t already hit the count limit or the nucleus mass
            uint32_t lo = 0, hi = 0xffffffffu;
            while (lo < hi) {
                const uint32_t mid = lo + (uint32_t)(((unsigned long long)(hi - lo) + 1) >> 1);
                unsigned long long c = 0;
                double m = 0.0;
                for (uint32_t i = tid; i < V; i += ST) {
                    const float l = x[i];
                    if (okey(l) >= mid) { ++c; if (use_p) m += (double)prob(l); }
                }
                c = block_reduce(c, OpSumU(), s_u);
                bool ok = c >= L1;
                if (use_p && !ok) { m = block_reduce(m, OpSumD(), s_d); ok = m >= (double)p.top_p; }
                if (ok) lo = mid; else hi = mid - 1;
            }
            B = lo;
            unsigned long long c_above = 0, c_eq = 0;
            double m_above = 0.0;
            for (uint32_t i = tid; i < V; i += ST) {
                const float l = x[i];
                const uint32_t k = okey(l);
                if (k > B) { ++c_above; m_above += (double)prob(l); }
                else if (k == B) ++c_eq;
            }
            c_above = block_reduce(c_above, OpSumU(), s_u);
            c_eq = block_reduce(c_eq, OpSumU(), s_u);
            m_above = block_reduce(m_above, OpSumD(), s_d);
            n_ties = (unsigned int)c_eq;
            const float pB = prob(key_to_float(B));
            double cum = m_above;
            unsigned int j = 0;
            while (j < n_ties) {     // ties enter one at a time, as the sorted walk of the reference does (:340-348)
                ++j;
                cum += (double)pB;
                if (c_above + j >= L1) break;
                if (use_p && cum >= (double)p.top_p) break;
            }
            r_ties = j;
            if (cum <= 0.0) degenerate = true;
            else kn = (float)(1.0 / cum);
        }
    }
    const bool rank_ties = trunc && !degenerate && r_ties < n_ties;
    // probability of element i of the final distribution; tie_rank only matters when rank_ties
    auto out_of = [&](uint32_t i, float l, unsigned int tie_rank) -> float {
        if (degenerate) return (int)i == top_idx ? 1.0f : 0.0f;
        if (!trunc) return prob(l);
        const uint32_t k = okey(l);
        if (k > B || (k == B && (!rank_ties || tie_rank < r_ties))) return prob(l) * kn;
        return 0.0f;
    };
    // contiguous chunk of this thread (index order = the order sample_from walks the nonzero entries, :373-383)
    const uint32_t CH = (V + ST - 1) / ST, i0 = tid * CH, i1 = (i0 + CH < V) ? i0 + CH : V;
    unsigned int tie_ex = 0;
    if (rank_ties) {
        unsigned int c = 0;
        for (uint32_t i = i0; i < i1; ++i) c += okey(x[i]) == B ? 1u : 0u;
        double dv, dt;
        unsigned int tot;
        block_exscan(0.0, c, dv, tie_ex, dt, tot, s_d, s_c);
    }
    // accept the draft with probability p[draft] (:436-443)
    // K1 = 0: one draft entry per row; K1 > 0: rows are [sequence][K1] and drafts [sequence][K1 - 1], the last row of a
    // sequence has none
    const int d = !draft ? -1 : K1 == 0 ? draft[row] : (row % K1 + 1 < K1 ? draft[(row / K1) * (K1 - 1) + row % K1] : -1);
    int acc = 0;
    float pd = 0.0f;
    if (d >= 0 && (uint32_t)d < V) {
        unsigned int rk = 0;
        if (rank_ties && okey(x[d]) == B) {                 // rank of the draft among the boundary ties
            unsigned long long c = 0;
            for (uint32_t i = tid; i < (uint32_t)d; i += ST) c += okey(x[i]) == B ? 1u : 0u;
            rk = (unsigned int)block_reduce(c, OpSumU(), s_u);
        }
        pd = out_of((uint32_t)d, x[d], rk);
        acc = u_acc[row] < (double)pd ? 1 : 0;
    }
    int tok = d;
    if (!acc) {
        // draw from the distribution with the rejected draft removed: inverse CDF over the nonzero entries in index
        // order, cumulative sums of weight / total, the last one forced to 1 (std::discrete_distribution)
        double wsum = 0.0;
        unsigned int tr = tie_ex;
        for (uint32_t i = i0; i < i1; ++i) {
            const float l = x[i];
            const bool tie = rank_ties && okey(l) == B;
            if ((int)i != d) wsum += (double)out_of(i, l, tr);
            if (tie) ++tr;
        }
        double ex, total;
        unsigned int ec, tc;
        block_exscan(wsum, 0u, ex, ec, total, tc, s_d, s_c);
        int cand = 0x7fffffff, last_nz = -1;
        if (total > 0.0) {
            const double u = u_res[row];
            double run = ex;
            tr = tie_ex;
            for (uint32_t i = i0; i < i1; ++i) {
                const float l = x[i];
                const bool tie = rank_ties && okey(l) == B;
                const float w = (int)i != d ? out_of(i, l, tr) : 0.0f;
                if (tie) ++tr;
                if (w > 0.0f) {
                    run += (double)w;
                    last_nz = (int)i;
                    if (cand == 0x7fffffff && run / total >= u) cand = (int)i;
                }
            }
        }
        cand = block_reduce(cand, OpMinI(), s_i);
        last_nz = block_reduce(last_nz, OpMaxI(), s_i);
        if (cand != 0x7fffffff) tok = cand;
        else if (last_nz >= 0) tok = last_nz;
        else if (d < 0) tok = top_idx;                      // cannot happen for a proper distribution
    }
    if (tid == 0) {
        if (token) token[row] = tok;
        if (accepted) accepted[row] = acc;
        if (p_draft) p_draft[row] = pd;
    }
    if (pval)                                               // the row's "argmax" for the commit kernel: the decided token
        for (uint32_t j = tid; j < nblk; j += ST) {
            pval[(size_t)row * nblk + j] = j == 0 ? INFINITY : -INFINITY;
            pidx[(size_t)row * nblk + j] = j == 0 ? tok : 0x7fffffff;
        }
}

}  // namespace

int qb_launch_sample_rows(qb_ctx *ctx, const float *logits, uint32_t rows, uint32_t V, uint32_t stride, const int32_t *draft,
                          uint32_t K1, const double *u_acc, const double *u_res, float temp, float top_p, int32_t top_k,
                          float min_p, int32_t *token, int32_t *accepted, float *p_draft, float *pval, int32_t *pidx,
                          uint32_t nblk) {
    QB_REQUIRE(temp > 0.0f, "sampling needs temp > 0 (temp <= 0 is the argmax path)");
    QB_REQUIRE(rows > 0 && V > 0 && u_res != nullptr, "qb_launch_sample_rows: bad arguments");
    SampleParams p;
    p.inv_t = 1.0f / temp; p.top_p = top_p; p.min_p = min_p; p.top_k = top_k;
    QB_CUDA(qb_launch_pdl(ctx->stream, sample_rows_kernel, dim3(rows), dim3(ST), (size_t)0, logits, V, stride, draft, u_acc, u_res, p,
                          token, accepted, p_draft, pval, pidx, nblk, K1));
    QB_LAUNCHED(ctx, "sample_rows_kernel");
    return QB_OK;
}

extern "C" int qb_sample_rows(qb_ctx *ctx, const float *logits_dev, uint32_t rows, uint32_t V, uint32_t stride,
                              const int32_t *draft_dev, const double *u_acc_dev, const double *u_res_dev, float temp, float top_p,
                              int32_t top_k, float min_p, int32_t *token_dev, int32_t *accepted_dev, float *p_draft_dev) {
    QB_REQUIRE(ctx && logits_dev && token_dev, "qb_sample_rows: null argument");
    QB_REQUIRE(draft_dev == nullptr || u_acc_dev != nullptr, "qb_sample_rows: drafts need acceptance draws");
    QB_CUDA(cudaSetDevice(ctx->device));
    return qb_launch_sample_rows(ctx, logits_dev, rows, V, stride, draft_dev, 0, u_acc_dev, u_res_dev, temp, top_p, top_k, min_p,
                                 token_dev, accepted_dev, p_draft_dev, nullptr, nullptr, 0);
}
