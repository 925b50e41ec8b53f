// Sampling-mode speculative acceptance on the device.
//
// The reference pulls the verifier's logits to the host for non-greedy requests and runs
// sampling_distribution + speculative_accept_pointmass there (src/qwen_native_backend.cpp:282-370, 399-467).
// Here a cluster of 8 CTAs per logits row builds the same distribution -- softmax(logits / temp), then the top-k,
// min-p and nucleus truncations, each a prefix of the descending order, renormalised over the kept set -- and
// takes the row's decision: accept the (greedy, point-mass) draft with probability p[draft]; on rejection draw
// from p with the draft removed; a row without a draft draws from p (the bonus token, or plain sampling).
// The uniform draws come from the caller, in the order the reference's generator would be consumed.
//
// Every thread keeps its (at most 20) consecutive logits and their exponentials in registers, so the row is read
// once.  The kept set is found without sorting: the descending order is the order of a monotone 32-bit key of the
// logit, and "the shortest prefix that reaches top_p or the count limit" is a radix descent over that key, two
// bits per pass: a 4-bin histogram (count and probability mass) of the elements under the current prefix, reduced
// over the block and exchanged between the CTAs through distributed shared memory.  Ties at the boundary key are
// taken lowest index first.
#include "qb_internal.h"

#include <cfloat>

namespace {

constexpr int ST = 1024;                      // threads per CTA
constexpr int CL = 8;                         // CTAs per row (one cluster)
constexpr int EPT = 20;                       // elements per thread at most: rows up to CL * ST * EPT = 163840 logits
constexpr int NB = 4;                         // histogram bins per pass (two key bits)

struct SampleParams {
    float inv_t, top_p, min_p;
    int top_k;
    float presence, repetition;               // token penalties (0 / 1 = off)
    const uint32_t *seen;                     // bitmap [sequence][seen_words] of the tokens a request has seen, or null
    uint32_t seen_words;
    const int32_t *chain_limit;               // [sequence] draft depth of this step (K1 > 0 form), or null = K1 - 1 everywhere
    int32_t eos;                              // a chain ends before the first draft equal to this token (-1: none)
};

__device__ __forceinline__ uint32_t okey(float f) {      // ascending key order == ascending float order
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Shared memory of a CTA: per-warp partials of a block reduction and the exchange area the CTAs of the cluster write
// into (two buffers, used alternately: a CTA that is one exchange ahead never overwrites what a slower one still reads).
struct Smem {
    double wd[ST / 32][NB];
    long long wi[ST / 32][NB];
    double xd[2][CL][NB];
    long long xi[2][CL][NB];
};

struct Comm {
    Smem *sm;
    uint32_t crank;
    int par;
};

__device__ __forceinline__ void push_to_cluster(Comm &c, int j, double sd, long long si) {
    const uint32_t ld = (uint32_t)__cvta_generic_to_shared(&c.sm->xd[c.par][c.crank][j]);
    const uint32_t li = (uint32_t)__cvta_generic_to_shared(&c.sm->xi[c.par][c.crank][j]);
    for (uint32_t r = 0; r < CL; ++r) {
        uint32_t rd, ri;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rd) : "r"(ld), "r"(r));
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ri) : "r"(li), "r"(r));
        asm volatile("st.shared::cluster.f64 [%0], %1;" ::"r"(rd), "d"(sd) : "memory");
        asm volatile("st.shared::cluster.s64 [%0], %1;" ::"r"(ri), "l"(si) : "memory");
    }
}
__device__ __forceinline__ int cluster_turn(Comm &c) {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    const int buf = c.par;
    c.par ^= 1;
    return buf;
}

// Sum over the block of N (<= NB) doubles and N integers per thread (warp shuffles, then the 32 warp rows added in warp
// order), handed to every CTA of the cluster: afterwards c.sm->xd[buf][rank][j] / xi[buf][rank][j] hold every CTA's sums.
template <int N>
__device__ int exchange(Comm &c, double (&d)[N], long long (&i)[N]) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int j = 0; j < N; ++j) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            d[j] += __shfl_xor_sync(0xffffffffu, d[j], o);
            i[j] += __shfl_xor_sync(0xffffffffu, i[j], o);
        }
    }
    __syncthreads();                                       // the warp rows may still be read from the previous call
    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < N; ++j) { c.sm->wd[warp][j] = d[j]; c.sm->wi[warp][j] = i[j]; }
    }
    __syncthreads();
    if (threadIdx.x < N) {
        double sd = 0.0;
        long long si = 0;
        for (int w = 0; w < ST / 32; ++w) { sd += c.sm->wd[w][threadIdx.x]; si += c.sm->wi[w][threadIdx.x]; }
        push_to_cluster(c, (int)threadIdx.x, sd, si);
    }
    return cluster_turn(c);
}

// one maximum (as a double) and one minimum (as an integer) per CTA, exchanged the same way; combined by the caller
__device__ int exchange_minmax(Comm &c, double vmax, long long vmin) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        vmax = fmax(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
        const long long t = __shfl_xor_sync(0xffffffffu, vmin, o);
        vmin = t < vmin ? t : vmin;
    }
    __syncthreads();
    if (lane == 0) { c.sm->wd[warp][0] = vmax; c.sm->wi[warp][0] = vmin; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double sd = c.sm->wd[0][0];
        long long si = c.sm->wi[0][0];
        for (int w = 1; w < ST / 32; ++w) { sd = fmax(sd, c.sm->wd[w][0]); si = c.sm->wi[w][0] < si ? c.sm->wi[w][0] : si; }
        push_to_cluster(c, 0, sd, si);
    }
    return cluster_turn(c);
}

// exclusive prefix of (v, n) over the threads of this CTA in thread order, and the CTA totals
__device__ void block_exscan(Comm &c, double v, long long n, double &ex_v, long long &ex_n, double &tot_v, long long &tot_n) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    double iv = v;
    long long in = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double nv = __shfl_up_sync(0xffffffffu, iv, o);
        const long long nn = __shfl_up_sync(0xffffffffu, in, o);
        if (lane >= (uint32_t)o) { iv += nv; in += nn; }
    }
    __syncthreads();
    if (lane == 31) { c.sm->wd[warp][0] = iv; c.sm->wi[warp][0] = in; }
    __syncthreads();
    double wv = 0.0;
    long long wn = 0;
    tot_v = 0.0; tot_n = 0;
    for (uint32_t w = 0; w < ST / 32; ++w) {
        if (w < warp) { wv += c.sm->wd[w][0]; wn += c.sm->wi[w][0]; }
        tot_v += c.sm->wd[w][0]; tot_n += c.sm->wi[w][0];
    }
    ex_v = wv + (iv - v);
    ex_n = wn + (in - n);
}

// One cluster per row.  draft == nullptr or the row's draft < 0: no draft (bonus / plain sampling row).
// K1 = 0: one draft entry per row; K1 > 0: rows are [sequence][K1] and drafts [sequence][K1 - 1], the last row of a
// sequence has none.
__global__ void __launch_bounds__(ST)
sample_rows_kernel(const float *__restrict__ logits, uint32_t V, uint32_t stride, const int32_t *__restrict__ draft,
                   const double *__restrict__ u_acc, const double *__restrict__ u_res, SampleParams p, int32_t *token,
                   int32_t *accepted, float *p_draft, float *pval, int32_t *pidx, uint32_t nblk, uint32_t K1) {
    __shared__ Smem sm;
    QB_PDL_ENTER();
    Comm c;
    c.sm = &sm; c.par = 0;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(c.crank));
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");     // every CTA of the cluster runs (its shared
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");       // memory exists) before anyone writes into it
    const uint32_t row = blockIdx.x / CL, tid = threadIdx.x;
    const float *x = logits + (size_t)row * stride;
    // this CTA's slice of the row, this thread's consecutive elements of it (index order = rank, thread, j)
    const uint32_t VC = (V + CL - 1) / CL, s0 = min(V, c.crank * VC), s1 = min(V, s0 + VC);
    const uint32_t ept = (VC + ST - 1) / ST, g0 = s0 + tid * ept;
    const int nv = g0 >= s1 ? 0 : (int)min(ept, s1 - g0);
    // token penalties (apply_token_penalties, src/qwen_native_backend.cpp:262-280) against the request's seen tokens and
    // the drafts of the earlier rows of this step (the running prefix of the accept loop, :432-447)
    const uint32_t seq = K1 ? row / K1 : row, n_prior = K1 ? row % K1 : 0;
    // the row that follows the last draft of a shortened chain (depth limit, or a drafted end-of-sequence token:
    // src/qwen_native_backend.cpp:15817-15821) is that step's bonus row: no acceptance test, one plain draw -- the draw
    // the row would otherwise have tested its draft with
    bool chain_end = false;
    if (K1 && p.chain_limit && draft) {
        uint32_t kk = min(K1 - 1, (uint32_t)max(p.chain_limit[seq], 0));
        if (p.eos >= 0)
            for (uint32_t i = 0; i < kk; ++i)
                if (draft[(size_t)seq * (K1 - 1) + i] == p.eos) { kk = i; break; }
        chain_end = n_prior >= kk && n_prior + 1 < K1;
    }
    const bool pen_rep = p.repetition > 0.0f && p.repetition != 1.0f, pen_pres = p.presence != 0.0f;
    auto penalised = [&](uint32_t idx, float v) -> float {
        if (!(pen_rep || pen_pres)) return v;
        bool sn = p.seen && ((p.seen[(size_t)seq * p.seen_words + (idx >> 5)] >> (idx & 31)) & 1u);
        for (uint32_t q = 0; q < n_prior && !sn; ++q) sn = draft && (uint32_t)draft[(size_t)seq * (K1 - 1) + q] == idx;
        if (!sn) return v;
        if (pen_rep) v = v >= 0.0f ? v / p.repetition : v * p.repetition;
        if (pen_pres) v -= p.presence;
        return v;
    };
    float l[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) l[j] = j < nv ? penalised(g0 + j, x[g0 + j]) : -INFINITY;

    // largest logit and its lowest index in one exchange: max of (key, ~index) as one integer
    float mx;
    int top_idx;
    {
        unsigned long long best = 0;
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (j < nv) {
                const unsigned long long pk = ((unsigned long long)okey(l[j]) << 32) | (uint32_t)~(g0 + j);
                best = pk > best ? pk : best;
            }
        const int buf = exchange_minmax(c, 0.0, ~(long long)(best ^ 0x8000000000000000ull));
        long long m = sm.xi[buf][0][0];
        for (int r = 1; r < CL; ++r) m = sm.xi[buf][r][0] < m ? sm.xi[buf][r][0] : m;
        const unsigned long long pk = (unsigned long long)(~m) ^ 0x8000000000000000ull;
        mx = key_to_float((uint32_t)(pk >> 32));
        top_idx = (int)(~(uint32_t)pk);
    }
    // softmax denominator in double (src/qwen_native_backend.cpp:296-303)
    float norm;
    {
        double d[1] = {0.0};
        long long z[1] = {0};
#pragma unroll
        for (int j = 0; j < EPT; ++j) if (j < nv) d[0] += (double)expf((l[j] - mx) * p.inv_t);
        const int buf = exchange<1>(c, d, z);
        double sum = 0.0;
        for (int r = 0; r < CL; ++r) sum += sm.xd[buf][r][0];
        norm = (float)(1.0 / (sum > 0.0 ? sum : 1.0));
    }
    auto prob = [&](float v) -> float { return expf((v - mx) * p.inv_t) * norm; };

    const bool use_k = p.top_k > 0 && (uint32_t)p.top_k < V, use_p = p.top_p < 1.0f && p.top_p > 0.0f, use_m = p.min_p > 0.0f;
    const bool trunc = use_k || use_p || use_m;
    uint32_t B = 0;                 // boundary key: keys above it are kept, r_ties of the n_ties equal to it
    long long r_ties = 0, n_ties = 0;
    float kn = 1.0f;
    bool degenerate = false;
    if (trunc) {
        long long L1 = use_k ? (long long)p.top_k : (long long)V;
        if (use_m) {                // min-p keeps the prefix whose probability is at least min_p times the top one (:333-338)
            const float cutoff = prob(mx) * p.min_p;
            double z[1] = {0.0};
            long long n[1] = {0};
#pragma unroll
            for (int j = 0; j < EPT; ++j) if (j < nv && prob(l[j]) >= cutoff) ++n[0];
            const int buf = exchange<1>(c, z, n);
            long long cnt = 0;
            for (int r = 0; r < CL; ++r) cnt += sm.xi[buf][r][0];
            L1 = cnt < L1 ? cnt : L1;
        }
        if (L1 == 0) {
            degenerate = true;
        } else {
            // radix descent from the top key bits: the bin (walking down from the highest) in which the elements seen so
            // far first hit the count limit or the nucleus mass holds the boundary key
            long long c_above = 0;
            double m_above = 0.0;
            uint32_t pre = 0;
            for (int sh = 30; sh >= 0; sh -= 2) {
                double hm[NB] = {0.0, 0.0, 0.0, 0.0};
                long long hc[NB] = {0, 0, 0, 0};
#pragma unroll
                for (int j = 0; j < EPT; ++j) {
                    const uint32_t k = okey(l[j]);
                    if (j < nv && (sh == 30 || (k >> (sh + 2)) == pre)) {
                        const uint32_t b = (k >> sh) & 3u;
                        const double pm = (double)prob(l[j]);
#pragma unroll
                        for (int q = 0; q < NB; ++q) { hc[q] += b == (uint32_t)q ? 1 : 0; hm[q] += b == (uint32_t)q ? pm : 0.0; }
                    }
                }
                const int buf = exchange<NB>(c, hm, hc);
                long long cc = 0;
                double mc = 0.0;
                int chosen = 0;
                for (int q = NB - 1; q >= 0; --q) {
                    long long tc = 0;
                    double tm = 0.0;
                    for (int r = 0; r < CL; ++r) { tc += sm.xi[buf][r][q]; tm += sm.xd[buf][r][q]; }
                    const bool ok = c_above + cc + tc >= L1 || (use_p && m_above + mc + tm >= (double)p.top_p);
                    if (ok || q == 0) { chosen = q; n_ties = tc; break; }
                    cc += tc; mc += tm;
                }
                c_above += cc; m_above += mc;
                pre = (pre << 2) | (uint32_t)chosen;
            }
            B = pre;
            const float pB = prob(key_to_float(B));
            double cum = m_above;
            long long j = 0;
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
    // probability of element i (logit v) of the final distribution; tie_rank only matters when rank_ties
    auto out_of = [&](uint32_t i, float v, long long tie_rank) -> float {
        if (degenerate) return (int)i == top_idx ? 1.0f : 0.0f;
        if (!trunc) return prob(v);
        const uint32_t k = okey(v);
        if (k > B || (k == B && (!rank_ties || tie_rank < r_ties))) return prob(v) * kn;
        return 0.0f;
    };
    // ranks of the boundary ties in index order: this thread's first tie rank, and the rank of the draft
    const int d = !draft || chain_end ? -1 : K1 == 0 ? draft[row] : (row % K1 + 1 < K1 ? draft[(row / K1) * (K1 - 1) + row % K1] : -1);
    const bool has_d = d >= 0 && (uint32_t)d < V;
    long long tie_ex = 0, d_rank = 0;
    if (rank_ties) {
        double z[2] = {0.0, 0.0};
        long long n[2] = {0, 0};
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (j < nv && okey(l[j]) == B) { ++n[0]; if (has_d && g0 + j < (uint32_t)d) ++n[1]; }
        double ev, tv;
        long long tn;
        block_exscan(c, 0.0, n[0], ev, tie_ex, tv, tn);
        const int buf = exchange<2>(c, z, n);
        for (uint32_t r = 0; r < CL; ++r) {
            if (r < c.crank) tie_ex += sm.xi[buf][r][0];
            d_rank += sm.xi[buf][r][1];
        }
    }
    // accept the draft with probability p[draft] (:436-443)
    int acc = 0;
    float pd = 0.0f;
    if (has_d) {
        pd = out_of((uint32_t)d, penalised((uint32_t)d, x[d]), d_rank);
        acc = u_acc[row] < (double)pd ? 1 : 0;
    }
    int tok = d;
    if (!acc) {
        // draw from the distribution with the rejected draft removed: inverse CDF over the nonzero entries in index
        // order, cumulative sums of weight / total, the last one forced to 1 (std::discrete_distribution)
        double w[1] = {0.0};
        long long z[1] = {0};
        {
            long long tr = tie_ex;
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                if (j < nv) {
                    const bool tie = rank_ties && okey(l[j]) == B;
                    if ((int)(g0 + j) != d) w[0] += (double)out_of(g0 + j, l[j], tr);
                    if (tie) ++tr;
                }
        }
        double ex, tv;
        long long en, tn;
        block_exscan(c, w[0], 0, ex, en, tv, tn);
        int buf = exchange<1>(c, w, z);
        double total = 0.0, off = 0.0;
        for (uint32_t r = 0; r < CL; ++r) {
            if (r < c.crank) off += sm.xd[buf][r][0];
            total += sm.xd[buf][r][0];
        }
        long long cand = 0x7fffffff;
        double last_nz = -1.0;
        if (total > 0.0) {
            const double u = chain_end ? u_acc[row] : u_res[row];
            double run = off + ex;
            long long tr = tie_ex;
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                if (j < nv) {
                    const bool tie = rank_ties && okey(l[j]) == B;
                    const float wj = (int)(g0 + j) != d ? out_of(g0 + j, l[j], tr) : 0.0f;
                    if (tie) ++tr;
                    if (wj > 0.0f) {
                        run += (double)wj;
                        last_nz = (double)(g0 + j);
                        if (cand == 0x7fffffff && run / total >= u) cand = (long long)(g0 + j);
                    }
                }
        }
        buf = exchange_minmax(c, last_nz, cand);
        for (uint32_t r = 0; r < CL; ++r) {
            cand = sm.xi[buf][r][0] < cand ? sm.xi[buf][r][0] : cand;
            last_nz = fmax(last_nz, sm.xd[buf][r][0]);
        }
        if (cand != 0x7fffffff) tok = (int)cand;
        else if (last_nz >= 0.0) tok = (int)last_nz;
        else if (d < 0) tok = top_idx;                      // cannot happen for a proper distribution
    }
    if (c.crank == 0) {
        if (tid == 0) {
            if (token) token[row] = tok;
            if (accepted) accepted[row] = acc;
            if (p_draft) p_draft[row] = pd;
        }
        if (pval)                                           // the row's "argmax" for the commit kernel: the decided token
            for (uint32_t j = tid; j < nblk; j += ST) {
                pval[(size_t)row * nblk + j] = j == 0 ? INFINITY : -INFINITY;
                pidx[(size_t)row * nblk + j] = j == 0 ? tok : 0x7fffffff;
            }
    }
}

}  // namespace

int qb_launch_sample_rows(qb_ctx *ctx, const float *logits, uint32_t rows, uint32_t V, uint32_t stride, const int32_t *draft,
                          uint32_t K1, const double *u_acc, const double *u_res, float temp, float top_p, int32_t top_k,
                          float min_p, int32_t *token, int32_t *accepted, float *p_draft, float *pval, int32_t *pidx,
                          uint32_t nblk, float presence, float repetition, const uint32_t *seen, uint32_t seen_words,
                          const int32_t *chain_limit, int32_t eos) {
    QB_REQUIRE(temp > 0.0f, "sampling needs temp > 0 (temp <= 0 is the argmax path)");
    QB_REQUIRE(rows > 0 && V > 0 && u_res != nullptr, "qb_launch_sample_rows: bad arguments");
    SampleParams p;
    p.inv_t = 1.0f / temp; p.top_p = top_p; p.min_p = min_p; p.top_k = top_k;
    p.presence = presence; p.repetition = repetition; p.seen = seen; p.seen_words = seen_words;
    p.chain_limit = chain_limit; p.eos = eos;
    QB_REQUIRE(V <= (uint32_t)(CL * ST * EPT), "sampling: rows of %u logits exceed the kernel's %d", V, CL * ST * EPT);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * CL);
    cfg.blockDim = dim3(ST);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = CL;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    QB_CUDA(cudaLaunchKernelEx(&cfg, sample_rows_kernel, logits, V, stride, draft, u_acc, u_res, p, token, accepted, p_draft, pval,
                               pidx, nblk, K1));
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
                                 token_dev, accepted_dev, p_draft_dev, nullptr, nullptr, 0, 0.0f, 1.0f, nullptr, 0);
}
