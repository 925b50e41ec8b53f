// CPU oracle for the qwen35 MTP speculative-decode step.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain multithreaded C++, the arithmetic of
// the kvmem-qw3 reference for the one path this repository implements on the GPU.  It is the
// checker for tests/, for the smoke entry and for the CPU-baseline leg of bench.py; the CUDA
// library never links, loads or calls it.
//
// Parity status: the Q8_0 / Q8_1 quantisers, the integer block dots and the two reference
// accumulation orders (mmvq, mmq) are pinned against the reference's own CUDA kernels compiled
// from its sources (oracle/_ref, GPU tests) and against the procedures and closed forms of the
// reference's tests (tests/mmq_parity.cu, tests/mixed_linear_parity.cu).  The gated-delta rule is
// pinned against the reference's gated_delta_net.cu in the same way, and the attention math against
// the reference's native decode attention (fattn_vec_decode.cu, its own library under oracle/_ref).
// RMSNorm, per-head norm + RoPE + KV append, gated attention, the whole recurrent layer core with its
// checkpoints, argmax and embedding rows are pinned on the reference's CUDA DeviceBackend driven through
// its public interface (kernels_cuda.cu built into oracle/_ref/libqw3ref_backend.so).
// The MTP head wiring and acceptance have no golden vectors in the reference ("parity unpinned" at
// unit level); they follow the cited source lines.
//
// Every function cites the reference lines it follows (paths inside the kvmem-qw3 tree).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/qw3b200.h"
#include "../include/qw3b200_synth.h"

namespace {

constexpr int QK = 32;

inline float f16_to_f32(uint16_t h) { return qs_f16_bits_to_f32(h); }
inline uint16_t f32_to_f16(float f) { return qs_f32_to_f16_bits(f); }

// Exact int32 dot of one 32-element block (the dp4a / mma.s8 integer part:
// src/mmvq_q8.cu:156-172, src/mmq_q8.cu:1738-1748).
inline int32_t dot32(const int8_t *a, const int8_t *b) {
    int32_t s = 0;
    for (int t = 0; t < QK; ++t) s += (int32_t)a[t] * (int32_t)b[t];
    return s;
}

// Planar host copy of a Q8_0 tensor: d = fp16 bits [rows][nb], q = int8 [rows][cols].
struct Q8 {
    uint32_t rows = 0, cols = 0;
    std::vector<uint16_t> d;
    std::vector<int8_t> q;
    uint32_t nb() const { return cols / QK; }
};

void q8_from_blocks(const uint8_t *blocks, uint32_t rows, uint32_t cols, Q8 &w) {
    w.rows = rows; w.cols = cols;
    const uint32_t nb = cols / QK;
    w.d.resize((size_t)rows * nb);
    w.q.resize((size_t)rows * cols);
    for (size_t b = 0; b < (size_t)rows * nb; ++b) {
        memcpy(&w.d[b], blocks + b * 34, 2);
        memcpy(&w.q[b * 32], blocks + b * 34 + 2, 32);
    }
}

const float *normal_table() {
    static std::vector<float> t;
    if (t.empty()) { t.resize(QS_NORMAL_TABLE_SIZE); qs_build_normal_table(t.data()); }
    return t.data();
}

void q8_synth(uint64_t seed, uint32_t tensor_id, uint32_t rows, uint32_t cols, float sigma, Q8 &w) {
    w.rows = rows; w.cols = cols;
    const uint32_t nb = cols / QK;
    w.d.resize((size_t)rows * nb);
    w.q.resize((size_t)rows * cols);
    const float *tab = normal_table();
    const int64_t nblocks = (int64_t)rows * nb;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nblocks; ++b) {
        qs_synth_q8_0_block(tab, seed, tensor_id, (uint64_t)b, sigma, &w.d[b], &w.q[(size_t)b * 32]);
    }
}

// ---- activation quantisers -------------------------------------------------------------

// quantize_mmq_q8_1_kernel arithmetic (src/mmvq_q8.cu:694-721): d_inv = 127/amax,
// q = rint(x*d_inv), d = 1/d_inv kept in fp32.  Planar output q[M][K], d[K/32][M].
void quantize_act(const float *x, uint32_t M, uint32_t K, uint32_t stride, int8_t *q, float *d) {
    const uint32_t nb = K / QK;
    for (uint32_t m = 0; m < M; ++m) {
        for (uint32_t kb = 0; kb < nb; ++kb) {
            const float *xb = x + (size_t)m * stride + kb * QK;
            float amax = 0.0f;
            for (int t = 0; t < QK; ++t) amax = std::max(amax, std::fabs(xb[t]));
            const float d_inv = (amax == 0.0f) ? 0.0f : 127.0f / amax;
            for (int t = 0; t < QK; ++t)
                q[(size_t)m * K + kb * QK + t] = (amax == 0.0f) ? 0 : (int8_t)(int)rintf(xb[t] * d_inv);
            d[(size_t)kb * M + m] = (amax == 0.0f) ? 0.0f : 1.0f / d_inv;
        }
    }
}

// Segment boundaries of the engine's K split, in 128-element chunks.
inline uint32_t seg_begin(uint32_t s, uint32_t S, uint32_t nchunks) { return (uint32_t)(((uint64_t)s * nchunks) / S); }

uint32_t ksplit_policy(uint32_t N, uint32_t K) {
    const uint32_t tiles = (N + 127) / 128;
    const uint32_t nchunks = K / 128;
    uint32_t S = 296 / std::max(tiles, 1u);
    S = std::max(1u, std::min(S, 8u));
    S = std::min(S, std::max(nchunks, 1u));
    return S;
}

// Engine accumulation order: per segment a sequential fma chain over 32-blocks
// (acc = fma(d_w*d_x, float(idot), acc), the per-output update of src/mmq_q8.cu:1738-1748),
// segments added in ascending order.  y[m*y_stride + n].
void gemm_engine(const Q8 &w, const int8_t *q, const float *d, uint32_t M, uint32_t S,
                 float *y, uint32_t y_stride, float *partials /* [S][M][N] or null */) {
    const uint32_t N = w.rows, K = w.cols, nb = K / QK, nchunks = K / 128;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)N; ++n) {
        const int8_t *wq = &w.q[(size_t)n * K];
        const uint16_t *wd = &w.d[(size_t)n * nb];
        for (uint32_t m = 0; m < M; ++m) {
            const int8_t *xq = q + (size_t)m * K;
            float total = 0.0f;
            for (uint32_t s = 0; s < S; ++s) {
                const uint32_t kb0 = seg_begin(s, S, nchunks) * 4, kb1 = seg_begin(s + 1, S, nchunks) * 4;
                float acc = 0.0f;
                for (uint32_t kb = kb0; kb < kb1; ++kb) {
                    const int32_t c = dot32(wq + kb * QK, xq + kb * QK);
                    const float sc = f16_to_f32(wd[kb]) * d[(size_t)kb * M + m];
                    acc = fmaf(sc, (float)c, acc);
                }
                if (partials) partials[((size_t)s * M + m) * N + n] = acc;
                total = (s == 0) ? acc : total + acc;
            }
            if (y) y[(size_t)m * y_stride + n] = total;
        }
    }
}

// fp32 in, fp32 out with the engine's quantiser and order (DeviceBackend::q8_0_matmul,
// include/qw3/device_backend.hpp:300-539).  S_shape_N is the row count of the fused weight the
// engine launches this tensor in (the split count depends on it).
void linear(const Q8 &w, uint32_t fused_rows, const float *x, uint32_t M, uint32_t x_stride, float *y,
            uint32_t y_stride) {
    std::vector<int8_t> q((size_t)M * w.cols);
    std::vector<float> d((size_t)(w.cols / QK) * M);
    quantize_act(x, M, w.cols, x_stride, q.data(), d.data());
    gemm_engine(w, q.data(), d.data(), M, ksplit_policy(fused_rows, w.cols), y, y_stride, nullptr);
}

// ---- norms, rope, activations -----------------------------------------------------------

// rms_norm_kernel_vec (src/kernels_cuda.cu:1992-2009): y = x * rsqrt(mean(x^2)+eps) * w.
void rms_norm(const float *x, const float *w, uint32_t n, float eps, float *y) {
    double ss = 0.0;
    for (uint32_t i = 0; i < n; ++i) ss += (double)x[i] * x[i];
    const float scale = 1.0f / std::sqrt((float)(ss / n) + eps);
    for (uint32_t i = 0; i < n; ++i) y[i] = x[i] * scale * w[i];
}

inline float sigmoidf_(float x) { return 1.0f / (1.0f + std::exp(-x)); }
inline float siluf_(float x) { return x / (1.0f + std::exp(-x)); }

// rope_partial_kernel (src/kernels_cuda.cu:4697-4719): split-half pairs (i, i+rope_dim/2) on the
// first rope_dim elements, angle = pos * theta^(-2i/rope_dim).
void rope_partial(float *x, uint32_t rope_dim, int pos, const float *inv_freq) {
    const uint32_t half = rope_dim / 2;
    for (uint32_t i = 0; i < half; ++i) {
        const float ang = (float)pos * inv_freq[i];
        const float c = std::cos(ang), s = std::sin(ang);
        const float x0 = x[i], x1 = x[i + half];
        x[i] = x0 * c - x1 * s;
        x[i + half] = x0 * s + x1 * c;
    }
}

void make_inv_freq(uint32_t rope_dim, float theta, std::vector<float> &f) {
    f.resize(rope_dim / 2);
    for (uint32_t i = 0; i < rope_dim / 2; ++i)
        f[i] = (float)std::pow((double)theta, -2.0 * (double)i / (double)rope_dim);
}

// argmax_kernel tie-break (src/kernels_cuda.cu:1765-1771): strictly greater, lowest index on ties.
int argmax(const float *x, uint32_t n) {
    int best = 0; float bv = x[0];
    for (uint32_t i = 1; i < n; ++i) if (x[i] > bv) { bv = x[i]; best = (int)i; }
    return best;
}

// ---- attention ---------------------------------------------------------------------------

// One query row: gated attention of n_heads heads over keys [0, n_keys) (fattn_vec_decode.cu:118-124,
// 156-233; gate src/kernels_cuda.cu:9448-9465).  q row = [n_heads][2*hd] (q | gate).  K/V fp16 bits,
// row `t` of the cache at kv[slot(t) * nkv*hd].
template <class SlotFn>
void attention_row(const float *qrow, uint32_t n_heads, uint32_t n_kv, uint32_t hd, uint32_t n_keys,
                   const uint16_t *kc, const uint16_t *vc, SlotFn slot, float *out) {
    const float scale = 1.0f / std::sqrt((float)hd);
    const uint32_t group = n_heads / n_kv;
    std::vector<float> sc(n_keys);
    for (uint32_t h = 0; h < n_heads; ++h) {
        const uint32_t kvh = h / group;
        const float *q = qrow + (size_t)h * 2 * hd;
        float mx = -INFINITY;
        for (uint32_t t = 0; t < n_keys; ++t) {
            const uint16_t *k = kc + ((size_t)slot(t) * n_kv + kvh) * hd;
            double s = 0.0;
            for (uint32_t i = 0; i < hd; ++i) s += (double)q[i] * (double)f16_to_f32(k[i]);
            sc[t] = (float)s * scale;
            mx = std::max(mx, sc[t]);
        }
        double den = 0.0;
        std::vector<double> acc(hd, 0.0);
        for (uint32_t t = 0; t < n_keys; ++t) {
            const float p = std::exp(sc[t] - mx);
            den += p;
            const uint16_t *v = vc + ((size_t)slot(t) * n_kv + kvh) * hd;
            for (uint32_t i = 0; i < hd; ++i) acc[i] += (double)p * (double)f16_to_f32(v[i]);
        }
        for (uint32_t i = 0; i < hd; ++i) {
            const float o = (float)(acc[i] / den);
            out[(size_t)h * hd + i] = o * sigmoidf_(q[hd + i]);
        }
    }
}

// rmsnorm_per_head_kernel (src/kernels_cuda.cu:4622-4645): RMSNorm over head_dim with one shared gain.
void head_norm(float *x, const float *w, uint32_t hd, float eps) {
    double ss = 0.0;
    for (uint32_t i = 0; i < hd; ++i) ss += (double)x[i] * x[i];
    const float scale = 1.0f / std::sqrt((float)(ss / hd) + eps);
    for (uint32_t i = 0; i < hd; ++i) x[i] = x[i] * scale * w[i];
}

// ---- gated DeltaNet ----------------------------------------------------------------------

struct DnShape { uint32_t nk, nv, hd, conv_k; uint32_t qkv_dim() const { return 2 * nk * hd + nv * hd; } };

// One row of the recurrent layer (recurrent_batch, src/kernels_cuda.cu:15053-15608):
//   conv1d + SiLU with state shift (:3672-3681), L2-norm of q and k heads (:4122-4156),
//   g = exp(softplus(alpha+dt_bias)*A), beta = sigmoid(b) (src/gated_delta_net.cu:63-70),
//   delta rule per v-head (:124-164), RMSNorm(core)*w*SiLU(z) (src/kernels_cuda.cu:4617-4619).
// state = [nv][hd(col j)][hd(i)], conv = [qkv_dim][conv_k-1] oldest first.
void deltanet_row(const DnShape &sh, const float *proj /* qkv */, const float *z, const float *alpha,
                  const float *beta, const float *conv_w, const float *ssm_a, const float *dt_bias,
                  const float *norm_w, float eps, float *state, float *conv, float *core) {
    const uint32_t C = sh.qkv_dim(), K1 = sh.conv_k - 1, hd = sh.hd;
    std::vector<float> x(C);
    for (uint32_t c = 0; c < C; ++c) {
        const float *w = conv_w + (size_t)c * sh.conv_k;
        float *st = conv + (size_t)c * K1;
        const float cur = proj[c];
        float acc = w[sh.conv_k - 1] * cur;
        for (uint32_t k = 0; k < K1; ++k) acc += w[k] * st[k];
        x[c] = siluf_(acc);
        for (uint32_t k = 0; k + 1 < K1; ++k) st[k] = st[k + 1];
        st[K1 - 1] = cur;
    }
    float *qh = x.data(), *kh = x.data() + sh.nk * hd, *vh = x.data() + 2 * sh.nk * hd;
    for (uint32_t h = 0; h < sh.nk; ++h) {
        for (float *p : {qh + h * hd, kh + h * hd}) {
            double ss = 0.0;
            for (uint32_t i = 0; i < hd; ++i) ss += (double)p[i] * p[i];
            const float sc = 1.0f / std::sqrt((float)ss + eps);
            for (uint32_t i = 0; i < hd; ++i) p[i] *= sc;
        }
    }
    const float oscale = 1.0f / std::sqrt((float)hd);
    for (uint32_t v = 0; v < sh.nv; ++v) {
        const uint32_t kh_i = v % sh.nk;   // src/gated_delta_net.cu:105
        const float *q = qh + kh_i * hd, *k = kh + kh_i * hd, *vv = vh + v * hd;
        const float g = std::exp(std::log1p(std::exp(alpha[v] + dt_bias[v])) * ssm_a[v]);
        const float b = sigmoidf_(beta[v]);
        float *S = state + (size_t)v * hd * hd;
        float *o = core + (size_t)v * hd;
        for (uint32_t j = 0; j < hd; ++j) {
            float *Sj = S + (size_t)j * hd;
            double kv = 0.0;
            for (uint32_t i = 0; i < hd; ++i) kv += (double)Sj[i] * k[i];
            const float delta = (vv[j] - g * (float)kv) * b;
            double at = 0.0;
            for (uint32_t i = 0; i < hd; ++i) {
                Sj[i] = g * Sj[i] + k[i] * delta;
                at += (double)Sj[i] * q[i];
            }
            o[j] = (float)at * oscale;
        }
        double ss = 0.0;
        for (uint32_t j = 0; j < hd; ++j) ss += (double)o[j] * o[j];
        const float sc = 1.0f / std::sqrt((float)(ss / hd) + eps);
        for (uint32_t j = 0; j < hd; ++j) o[j] = o[j] * sc * norm_w[j] * siluf_(z[(size_t)v * hd + j]);
    }
}

// ---- model -------------------------------------------------------------------------------

// Tensor ids of the seeded generator: layer * 32 + kind; globals use layer index 0xFFFF.
enum TensorKind : uint32_t {
    T_ATTN_Q = 1, T_ATTN_K, T_ATTN_V, T_ATTN_OUT, T_FFN_GATE, T_FFN_UP, T_FFN_DOWN,
    T_SSM_QKV, T_SSM_Z, T_SSM_ALPHA, T_SSM_BETA, T_SSM_OUT, T_SSM_CONV, T_SSM_A, T_SSM_DT,
    T_EH_PROJ, T_TOKEN_EMBD, T_OUTPUT
};
inline uint32_t tid(uint32_t layer, uint32_t kind) { return layer * 32u + kind; }

struct Layer {
    bool recurrent = false;
    Q8 attn_q, attn_k, attn_v, attn_out, ffn_gate, ffn_up, ffn_down;
    Q8 ssm_qkv, ssm_z, ssm_alpha, ssm_beta, ssm_out;
    std::vector<float> conv_w, ssm_a, dt_bias;
    // RMSNorm gains (src/qwen_native.cpp:160-186): attn_norm, ffn_norm / post_attention_norm, attn_q_norm, attn_k_norm, ssm_norm
    std::vector<float> attn_norm, ffn_norm, q_norm, k_norm, ssm_norm;
};

struct Model {
    qb_model_config cfg;
    std::vector<Layer> layers;   // n_layers (+1 MTP layer at the end if cfg.mtp_layers)
    Q8 token_embd, output, eh_proj;
    // MTP head: its own embedding table / LM head when the checkpoint has them, else the target's
    // (src/qwen_native.cpp:288-298); empty = shared
    Q8 mtp_embd, mtp_head;
    std::vector<float> output_norm, enorm, hnorm, shared_head_norm;
    std::vector<float> ones;     // gains of the seeded model are 1.0
    std::vector<float> inv_freq;
    const Q8 &mtp_embedding() const { return mtp_embd.rows ? mtp_embd : token_embd; }
    const Q8 &mtp_lm_head() const { return mtp_head.rows ? mtp_head : output; }
    DnShape dn() const { return {cfg.ssm_num_k_heads, cfg.ssm_num_v_heads, cfg.ssm_head_dim, cfg.ssm_conv_kernel}; }
    bool is_attn(uint32_t i) const { return cfg.full_attention_interval && ((i + 1) % cfg.full_attention_interval) == 0; }
};

// Small fp32 DeltaNet tensors: ssm_a = -exp(U(log 1, log 16)) (decay must be negative, cf. the
// negative_exp transform at src/qwen_weights.cpp:93), dt_bias ~ U(-4,-1), conv1d ~ U(-1,1)*0.5.
inline double urand(uint64_t seed, uint32_t stream, uint64_t i) {
    return (double)(qs_rand_u32(seed, stream, i) >> 8) / 16777216.0;
}

void build_layer(Model &m, Layer &L, uint32_t il, bool recurrent, uint64_t seed) {
    const auto &c = m.cfg;
    const float sg = c.weight_sigma;
    L.recurrent = recurrent;
    if (!recurrent) {
        const uint32_t inner = c.n_heads * c.head_dim, kvd = c.n_kv_heads * c.head_dim;
        q8_synth(seed, tid(il, T_ATTN_Q), 2 * inner, c.n_embd, sg, L.attn_q);
        q8_synth(seed, tid(il, T_ATTN_K), kvd, c.n_embd, sg, L.attn_k);
        q8_synth(seed, tid(il, T_ATTN_V), kvd, c.n_embd, sg, L.attn_v);
        q8_synth(seed, tid(il, T_ATTN_OUT), c.n_embd, inner, sg, L.attn_out);
    } else {
        const DnShape d = m.dn();
        const uint32_t vdim = d.nv * d.hd;
        q8_synth(seed, tid(il, T_SSM_QKV), d.qkv_dim(), c.n_embd, sg, L.ssm_qkv);
        q8_synth(seed, tid(il, T_SSM_Z), vdim, c.n_embd, sg, L.ssm_z);
        q8_synth(seed, tid(il, T_SSM_ALPHA), d.nv, c.n_embd, sg, L.ssm_alpha);
        q8_synth(seed, tid(il, T_SSM_BETA), d.nv, c.n_embd, sg, L.ssm_beta);
        q8_synth(seed, tid(il, T_SSM_OUT), c.n_embd, vdim, sg, L.ssm_out);
        L.conv_w.resize((size_t)d.qkv_dim() * d.conv_k);
        for (size_t i = 0; i < L.conv_w.size(); ++i)
            L.conv_w[i] = (float)((urand(seed, tid(il, T_SSM_CONV), i) * 2.0 - 1.0) * 0.5);
        L.ssm_a.resize(d.nv); L.dt_bias.resize(d.nv);
        for (uint32_t v = 0; v < d.nv; ++v) {
            L.ssm_a[v] = (float)(-std::exp(urand(seed, tid(il, T_SSM_A), v) * std::log(16.0)));
            L.dt_bias[v] = (float)(-4.0 + 3.0 * urand(seed, tid(il, T_SSM_DT), v));
        }
    }
    q8_synth(seed, tid(il, T_FFN_GATE), c.n_ff, c.n_embd, sg, L.ffn_gate);
    q8_synth(seed, tid(il, T_FFN_UP), c.n_ff, c.n_embd, sg, L.ffn_up);
    q8_synth(seed, tid(il, T_FFN_DOWN), c.n_embd, c.n_ff, sg, L.ffn_down);
}

struct Seq {
    const Model *m = nullptr;
    uint32_t max_ctx = 0;
    int pos = 0;            // committed tokens
    int cur_tok = -1;       // next token to forward
    std::vector<std::vector<uint16_t>> kc, vc;     // per layer (attention layers only used)
    std::vector<uint16_t> mtp_k, mtp_v;
    std::vector<std::vector<float>> state, conv;   // per layer (recurrent layers only used)
    std::vector<float> h_prev;                     // target hidden (pre output norm) of position pos-1
    std::vector<float> last_logits; uint32_t last_rows = 0;
    std::vector<float> last_hidden;
    std::vector<int> last_drafts, last_row_argmax;
};

// FFN block on rows: h += W_down( silu(W_gate n) * (W_up n) ) (src/qwen_executor.cpp:6662-6693).
void ffn_rows(const Model &m, const Layer &L, float *h, uint32_t M) {
    const uint32_t H = m.cfg.n_embd, F = m.cfg.n_ff;
    std::vector<float> n((size_t)M * H), g((size_t)M * F), u((size_t)M * F), dn((size_t)M * H);
    for (uint32_t r = 0; r < M; ++r) rms_norm(h + (size_t)r * H, L.ffn_norm.data(), H, m.cfg.rms_eps, &n[(size_t)r * H]);
    linear(L.ffn_gate, 2 * F, n.data(), M, H, g.data(), F);
    linear(L.ffn_up, 2 * F, n.data(), M, H, u.data(), F);
    for (size_t i = 0; i < g.size(); ++i) g[i] = siluf_(g[i]) * u[i];
    linear(L.ffn_down, H, g.data(), M, F, dn.data(), H);
    for (size_t i = 0; i < dn.size(); ++i) h[i] += dn[i];
}

// Attention block on rows at positions base..base+M-1 writing K/V into (kc, vc)
// (src/qwen_executor.cpp:6472-6638 target; :7093-7180 MTP layer).
void attn_rows(const Model &m, const Layer &L, float *h, uint32_t M, int base,
               std::vector<uint16_t> &kc, std::vector<uint16_t> &vc, bool kv_only) {
    const auto &c = m.cfg;
    const uint32_t H = c.n_embd, hd = c.head_dim, inner = c.n_heads * hd, kvd = c.n_kv_heads * hd;
    const uint32_t fused = 2 * inner + 2 * kvd;
    std::vector<float> n((size_t)M * H), q((size_t)M * 2 * inner), k((size_t)M * kvd), v((size_t)M * kvd);
    for (uint32_t r = 0; r < M; ++r) rms_norm(h + (size_t)r * H, L.attn_norm.data(), H, c.rms_eps, &n[(size_t)r * H]);
    if (!kv_only) linear(L.attn_q, fused, n.data(), M, H, q.data(), 2 * inner);
    linear(L.attn_k, fused, n.data(), M, H, k.data(), kvd);
    linear(L.attn_v, fused, n.data(), M, H, v.data(), kvd);
    if (kc.size() < (size_t)(base + M) * kvd) { kc.resize((size_t)(base + M) * kvd); vc.resize((size_t)(base + M) * kvd); }
    for (uint32_t r = 0; r < M; ++r) {
        for (uint32_t hh = 0; hh < c.n_kv_heads; ++hh) {
            float *kp = &k[(size_t)r * kvd + hh * hd];
            head_norm(kp, L.k_norm.data(), hd, c.rms_eps);
            rope_partial(kp, c.rope_dim, base + (int)r, m.inv_freq.data());
        }
        for (uint32_t i = 0; i < kvd; ++i) {   // kv_append_*_f16 (src/kernels_cuda.cu:8921-8969)
            kc[(size_t)(base + r) * kvd + i] = f32_to_f16(k[(size_t)r * kvd + i]);
            vc[(size_t)(base + r) * kvd + i] = f32_to_f16(v[(size_t)r * kvd + i]);
        }
    }
    if (kv_only) return;
    std::vector<float> mid((size_t)M * inner), o((size_t)M * H);
#pragma omp parallel for schedule(dynamic)
    for (int64_t r = 0; r < (int64_t)M; ++r) {
        float *qr = &q[(size_t)r * 2 * inner];
        for (uint32_t hh = 0; hh < c.n_heads; ++hh) {
            head_norm(qr + (size_t)hh * 2 * hd, L.q_norm.data(), hd, c.rms_eps);
            rope_partial(qr + (size_t)hh * 2 * hd, c.rope_dim, base + (int)r, m.inv_freq.data());
        }
        attention_row(qr, c.n_heads, c.n_kv_heads, hd, (uint32_t)(base + r + 1), kc.data(), vc.data(),
                      [](uint32_t t) { return t; }, &mid[(size_t)r * inner]);
    }
    linear(L.attn_out, H, mid.data(), M, inner, o.data(), H);
    for (size_t i = 0; i < o.size(); ++i) h[i] += o[i];
}

// DeltaNet block on rows (src/qwen_executor.cpp:6300-6425).  Writes the state after each row into
// ck_state[t]/ck_conv[t] when those are given (the per-row checkpoints of
// src/gated_delta_net.cu:165-176 and src/kernels_cuda.cu:3682-3691); state/conv end at the last row.
void dn_rows(const Model &m, const Layer &L, float *h, uint32_t M, std::vector<float> &state,
             std::vector<float> &conv, std::vector<std::vector<float>> *ck_state,
             std::vector<std::vector<float>> *ck_conv) {
    const auto &c = m.cfg;
    const DnShape d = m.dn();
    const uint32_t H = c.n_embd, C = d.qkv_dim(), vdim = d.nv * d.hd;
    const uint32_t fused = C + vdim + 2 * d.nv;
    std::vector<float> n((size_t)M * H), proj((size_t)M * C), z((size_t)M * vdim), al((size_t)M * d.nv),
        be((size_t)M * d.nv), core((size_t)M * vdim), o((size_t)M * H);
    for (uint32_t r = 0; r < M; ++r) rms_norm(h + (size_t)r * H, L.attn_norm.data(), H, c.rms_eps, &n[(size_t)r * H]);
    linear(L.ssm_qkv, fused, n.data(), M, H, proj.data(), C);
    linear(L.ssm_z, fused, n.data(), M, H, z.data(), vdim);
    linear(L.ssm_alpha, fused, n.data(), M, H, al.data(), d.nv);
    linear(L.ssm_beta, fused, n.data(), M, H, be.data(), d.nv);
    for (uint32_t r = 0; r < M; ++r) {
        deltanet_row(d, &proj[(size_t)r * C], &z[(size_t)r * vdim], &al[(size_t)r * d.nv], &be[(size_t)r * d.nv],
                     L.conv_w.data(), L.ssm_a.data(), L.dt_bias.data(), L.ssm_norm.data(), c.rms_eps,
                     state.data(), conv.data(), &core[(size_t)r * vdim]);
        if (ck_state) { (*ck_state)[r] = state; (*ck_conv)[r] = conv; }
    }
    linear(L.ssm_out, H, core.data(), M, vdim, o.data(), H);
    for (size_t i = 0; i < o.size(); ++i) h[i] += o[i];
}

void embed_rows(const Q8 &w, const int *tokens, uint32_t M, float *out) {
    const uint32_t H = w.cols, nb = w.nb();
    for (uint32_t r = 0; r < M; ++r)
        for (uint32_t i = 0; i < H; ++i)   // q8_get_row_kernel (src/kernels_cuda.cu:2075-2087)
            out[(size_t)r * H + i] = f16_to_f32(w.d[(size_t)tokens[r] * nb + i / 32]) * (float)w.q[(size_t)tokens[r] * H + i];
}

struct RowCheckpoints {
    // [layer][row] -> state / conv after that row (recurrent layers only)
    std::vector<std::vector<std::vector<float>>> state, conv;
};

// forward_n_tokens (src/qwen_executor.cpp:6003-6836): M rows of one sequence at positions
// base..base+M-1.  hidden = pre-output-norm rows; logits for rows >= logits_from.
void target_forward(Seq &s, const int *tokens, uint32_t M, int base, std::vector<float> &hidden,
                    std::vector<float> *logits, uint32_t logits_from, RowCheckpoints *ck) {
    const Model &m = *s.m;
    const uint32_t H = m.cfg.n_embd, V = m.cfg.vocab_size;
    hidden.assign((size_t)M * H, 0.0f);
    embed_rows(m.token_embd, tokens, M, hidden.data());
    if (ck) { ck->state.assign(m.cfg.n_layers, {}); ck->conv.assign(m.cfg.n_layers, {}); }
    for (uint32_t il = 0; il < m.cfg.n_layers; ++il) {
        const Layer &L = m.layers[il];
        if (L.recurrent) {
            if (ck) { ck->state[il].resize(M); ck->conv[il].resize(M); }
            dn_rows(m, L, hidden.data(), M, s.state[il], s.conv[il], ck ? &ck->state[il] : nullptr,
                    ck ? &ck->conv[il] : nullptr);
        } else {
            attn_rows(m, L, hidden.data(), M, base, s.kc[il], s.vc[il], false);
        }
        ffn_rows(m, L, hidden.data(), M);
    }
    if (logits) {
        const uint32_t R = M - logits_from;
        std::vector<float> n((size_t)R * H);
        for (uint32_t r = 0; r < R; ++r)
            rms_norm(&hidden[(size_t)(logits_from + r) * H], m.output_norm.data(), H, m.cfg.rms_eps, &n[(size_t)r * H]);
        logits->assign((size_t)R * V, 0.0f);
        linear(m.output, V, n.data(), R, H, logits->data(), V);
    }
}

// MTP head on rows (forward_mtp_draft_from src/qwen_executor.cpp:7025-7255; batch prefix form
// :22690-22796): row r uses token tokens[r] and previous hidden hprev[r]; K/V written at base+r.
// kv_only: stop after the K/V append.  Returns post-layer hidden (mtp_h) and logits if asked.
void mtp_rows(Seq &s, const int *tokens, const float *hprev, uint32_t M, int base, bool kv_only,
              std::vector<float> *mtp_h_out, std::vector<float> *logits) {
    const Model &m = *s.m;
    const uint32_t H = m.cfg.n_embd, V = m.cfg.vocab_size;
    const Layer &L = m.layers[m.cfg.n_layers];
    std::vector<float> e((size_t)M * H), cat((size_t)M * 2 * H), hh((size_t)M * H);
    embed_rows(m.mtp_embedding(), tokens, M, e.data());
    for (uint32_t r = 0; r < M; ++r) {
        rms_norm(&e[(size_t)r * H], m.enorm.data(), H, m.cfg.rms_eps, &cat[(size_t)r * 2 * H]);            // enorm
        rms_norm(hprev + (size_t)r * H, m.hnorm.data(), H, m.cfg.rms_eps, &cat[(size_t)r * 2 * H + H]);    // hnorm
    }
    linear(m.eh_proj, H, cat.data(), M, 2 * H, hh.data(), H);
    attn_rows(m, L, hh.data(), M, base, s.mtp_k, s.mtp_v, kv_only);
    if (kv_only) return;
    ffn_rows(m, L, hh.data(), M);
    if (logits) {
        std::vector<float> n((size_t)M * H);
        for (uint32_t r = 0; r < M; ++r) rms_norm(&hh[(size_t)r * H], m.shared_head_norm.data(), H, m.cfg.rms_eps, &n[(size_t)r * H]);
        logits->assign((size_t)M * V, 0.0f);
        linear(m.mtp_lm_head(), V, n.data(), M, H, logits->data(), V);
    }
    if (mtp_h_out) *mtp_h_out = hh;
}

}  // namespace

// =============================================================================================
// C interface (ctypes)
// =============================================================================================
extern "C" {

void orc_normal_table(float *out) { memcpy(out, normal_table(), sizeof(float) * QS_NORMAL_TABLE_SIZE); }

// Host Q8_0 quantiser of the reference's GEMM parity test (tests/mmq_parity.cu:54-80).
void orc_quantize_q8_0(const float *w, uint32_t rows, uint32_t cols, uint8_t *blocks) {
    const uint32_t nb = cols / QK;
    for (size_t b = 0; b < (size_t)rows * nb; ++b) {
        int8_t q[32];
        const uint16_t d = qs_quantize_q8_0_block(w + b * 32, q);
        memcpy(blocks + b * 34, &d, 2);
        memcpy(blocks + b * 34 + 2, q, 32);
    }
}

void orc_dequant_q8_0(const uint8_t *blocks, uint32_t rows, uint32_t cols, float *out) {
    const uint32_t nb = cols / QK;
    for (size_t b = 0; b < (size_t)rows * nb; ++b) {
        uint16_t d; memcpy(&d, blocks + b * 34, 2);
        const int8_t *q = (const int8_t *)(blocks + b * 34 + 2);
        for (int t = 0; t < 32; ++t) out[b * 32 + t] = (float)q[t] * f16_to_f32(d);
    }
}

// Split-plane device layout of the reference (src/cuda_helpers.cuh:16-39, repack at
// src/kernels_cuda.cu:1566-1594): per row all fp16 scales, then all int8 quants.
void orc_repack_split_plane(const uint8_t *blocks, uint32_t rows, uint32_t cols, uint8_t *out) {
    const uint32_t nb = cols / QK;
    for (uint32_t r = 0; r < rows; ++r) {
        uint8_t *row = out + (size_t)r * nb * 34;
        for (uint32_t kb = 0; kb < nb; ++kb) {
            const uint8_t *src = blocks + ((size_t)r * nb + kb) * 34;
            memcpy(row + 2 * kb, src, 2);
            memcpy(row + 2 * nb + 32 * kb, src + 2, 32);
        }
    }
}

void orc_synth_q8_0(uint64_t seed, uint32_t tensor_id, uint32_t rows, uint32_t cols, float sigma, uint8_t *blocks) {
    const uint32_t nb = cols / QK;
    const float *tab = normal_table();
    const int64_t nblocks = (int64_t)rows * nb;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nblocks; ++b) {
        uint16_t d; int8_t q[32];
        qs_synth_q8_0_block(tab, seed, tensor_id, (uint64_t)b, sigma, &d, q);
        memcpy(blocks + b * 34, &d, 2);
        memcpy(blocks + b * 34 + 2, q, 32);
    }
}

// quantize_q8_1_kernel (src/mmvq_q8.cu:98-111): d = amax/127, q = rint(x/d), header {half d, half sum}.
void orc_quantize_q8_1(const float *x, uint32_t M, uint32_t K, uint32_t stride, uint8_t *out) {
    const uint32_t nb = K / QK;
    for (uint32_t m = 0; m < M; ++m)
        for (uint32_t kb = 0; kb < nb; ++kb) {
            const float *xb = x + (size_t)m * stride + kb * QK;
            float amax = 0.0f;
            for (int t = 0; t < QK; ++t) amax = std::max(amax, std::fabs(xb[t]));
            // the kernel reduces the sum with xor-shuffles 16,8,4,2,1 over the 32 lanes
            float part[32];
            for (int t = 0; t < QK; ++t) part[t] = xb[t];
            for (int off = 16; off > 0; off >>= 1)
                for (int t = 0; t < QK; ++t) if ((t & off) == 0) { const float a = part[t] + part[t | off]; part[t] = a; part[t | off] = a; }
            const float d = amax / 127.0f;
            uint8_t *blk = out + ((size_t)m * nb + kb) * 36;
            const uint16_t hd = f32_to_f16(d), hs = f32_to_f16(part[0]);
            memcpy(blk, &hd, 2); memcpy(blk + 2, &hs, 2);
            for (int t = 0; t < QK; ++t) blk[4 + t] = (uint8_t)(int8_t)((amax == 0.0f) ? 0 : (int)rintf(xb[t] / d));
        }
}

// quantize_mmq_q8_1_kernel (src/mmvq_q8.cu:669-722): 144-byte blocks {float d4[4]; int8 q[128]},
// block index sb * M + row.
void orc_quantize_q8_1_mmq(const float *x, uint32_t M, uint32_t K, uint32_t stride, uint8_t *out) {
    std::vector<int8_t> q((size_t)M * K);
    std::vector<float> d((size_t)(K / QK) * M);
    quantize_act(x, M, K, stride, q.data(), d.data());
    for (uint32_t sb = 0; sb < K / 128; ++sb)
        for (uint32_t m = 0; m < M; ++m) {
            uint8_t *blk = out + ((size_t)sb * M + m) * 144;
            for (int s4 = 0; s4 < 4; ++s4) memcpy(blk + 4 * s4, &d[(size_t)(sb * 4 + s4) * M + m], 4);
            memcpy(blk + 16, &q[(size_t)m * K + sb * 128], 128);
        }
}

void orc_quantize_act(const float *x, uint32_t M, uint32_t K, uint32_t stride, int8_t *q, float *d) {
    quantize_act(x, M, K, stride, q, d);
}

uint32_t orc_ksplit_policy(uint32_t N, uint32_t K) { return ksplit_policy(N, K); }

// out[m][n][kb] exact int32 dots.
void orc_block_dots(const uint8_t *blocks, uint32_t N, uint32_t K, const int8_t *q, uint32_t M, int32_t *out) {
    Q8 w; q8_from_blocks(blocks, N, K, w);
    const uint32_t nb = K / QK;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)N; ++n)
        for (uint32_t m = 0; m < M; ++m)
            for (uint32_t kb = 0; kb < nb; ++kb)
                out[((size_t)m * N + n) * nb + kb] = dot32(&w.q[(size_t)n * K + kb * QK], q + (size_t)m * K + kb * QK);
}

// Engine-order product from quantised activations; partials may be null.
void orc_gemm_engine(const uint8_t *blocks, uint32_t N, uint32_t K, const int8_t *q, const float *d, uint32_t M,
                     uint32_t ksplit, float *y, float *partials) {
    Q8 w; q8_from_blocks(blocks, N, K, w);
    gemm_engine(w, q, d, M, ksplit ? ksplit : ksplit_policy(N, K), y, N, partials);
}

void orc_matmul_engine(const uint8_t *blocks, uint32_t N, uint32_t K, const float *x, uint32_t M, uint32_t x_stride,
                       uint32_t ksplit, float *y) {
    Q8 w; q8_from_blocks(blocks, N, K, w);
    std::vector<int8_t> q((size_t)M * K);
    std::vector<float> d((size_t)(K / QK) * M);
    quantize_act(x, M, K, x_stride, q.data(), d.data());
    gemm_engine(w, q.data(), d.data(), M, ksplit ? ksplit : ksplit_policy(N, K), y, N, nullptr);
}

// mul_mat_vec_q8_0_kernel order (src/mmvq_q8.cu:195-280): NW warps (4 for M<=4, 2 for 5..8), thread
// tid handles 8 int8 (ints kqs, kqs+1) of block kbx = tid/4 + i*8*NW; per thread
// tmp += d_w*d_x*float(sumi); warps 1.. are added to warp 0 in warp order, then xor-shuffle
// 16,8,4,2,1.  x = q8_1 blocks (36 B).
void orc_matmul_mmvq(const uint8_t *blocks, uint32_t N, uint32_t K, const uint8_t *xq81, uint32_t M, float *y) {
    Q8 w; q8_from_blocks(blocks, N, K, w);
    const uint32_t nb = K / QK;
    const int NW = M <= 4 ? 4 : 2;
    const int nthreads = 32 * NW;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)N; ++n) {
        std::vector<float> tmp(nthreads);
        for (uint32_t m = 0; m < M; ++m) {
            for (int t = 0; t < nthreads; ++t) {
                float acc = 0.0f;
                const int kqs = 2 * (t % 4);
                for (uint32_t kbx = t / 4; kbx < nb; kbx += 8 * NW) {
                    const uint8_t *xb = xq81 + ((size_t)m * nb + kbx) * 36;
                    uint16_t hd; memcpy(&hd, xb, 2);
                    const int8_t *xq = (const int8_t *)(xb + 4) + kqs * 4;
                    const int8_t *wq = &w.q[(size_t)n * K + kbx * QK + kqs * 4];
                    int32_t sumi = 0;
                    for (int i = 0; i < 8; ++i) sumi += (int32_t)wq[i] * (int32_t)xq[i];
                    const float dw = f16_to_f32(w.d[(size_t)n * nb + kbx]);
                    // d_w * d_x * float(sumi) then +=: nvcc (-fmad=true) contracts the last mul+add
                    acc = fmaf(dw * f16_to_f32(hd), (float)sumi, acc);
                }
                tmp[t] = acc;
            }
            float lane[32];
            for (int l = 0; l < 32; ++l) {
                float v = tmp[l];
                for (int wp = 1; wp < NW; ++wp) v += tmp[wp * 32 + l];
                lane[l] = v;
            }
            for (int off = 16; off > 0; off >>= 1)
                for (int l = 0; l < 32; ++l) if ((l & off) == 0) { const float a = lane[l] + lane[l | off]; lane[l] = a; lane[l | off] = a; }
            y[(size_t)m * N + n] = lane[0];
        }
    }
}

// MMQ order (src/mmq_q8.cu:1738-1748, :1917-1964, :2164-2248): acc += d_w*d_y*float(c) over
// 32-blocks in ascending K.  x = q8_1_mmq blocks (144 B).  fma_contract: the reference is built
// with nvcc's default -fmad=true, so the update is fma(d_w*d_y, float(c), acc).
void orc_matmul_mmq(const uint8_t *blocks, uint32_t N, uint32_t K, const uint8_t *xmmq, uint32_t M, float *y) {
    Q8 w; q8_from_blocks(blocks, N, K, w);
    const uint32_t nb = K / QK;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)N; ++n)
        for (uint32_t m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (uint32_t kb = 0; kb < nb; ++kb) {
                const uint8_t *blk = xmmq + ((size_t)(kb / 4) * M + m) * 144;
                float dy; memcpy(&dy, blk + 4 * (kb % 4), 4);
                const int32_t c = dot32(&w.q[(size_t)n * K + kb * QK], (const int8_t *)(blk + 16) + (kb % 4) * 32);
                acc = fmaf(f16_to_f32(w.d[(size_t)n * nb + kb]) * dy, (float)c, acc);
            }
            y[(size_t)m * N + n] = acc;
        }
}

void orc_get_rows(const uint8_t *blocks, uint32_t rows, uint32_t cols, const int32_t *ids, uint32_t n, float *out) {
    const uint32_t nb = cols / QK;
    for (uint32_t r = 0; r < n; ++r)
        for (uint32_t i = 0; i < cols; ++i) {
            const uint8_t *blk = blocks + ((size_t)ids[r] * nb + i / 32) * 34;
            uint16_t d; memcpy(&d, blk, 2);
            out[(size_t)r * cols + i] = f16_to_f32(d) * (float)(int8_t)blk[2 + i % 32];
        }
    (void)rows;
}

void orc_rms_norm(const float *x, const float *w, uint32_t M, uint32_t n, uint32_t stride, float eps, float *out) {
    for (uint32_t m = 0; m < M; ++m) rms_norm(x + (size_t)m * stride, w, n, eps, out + (size_t)m * stride);
}

void orc_inv_freq(uint32_t rope_dim, float theta, float *out) {
    std::vector<float> f; make_inv_freq(rope_dim, theta, f);
    memcpy(out, f.data(), f.size() * sizeof(float));
}

// Per-head q/k RMSNorm + partial RoPE + paged fp16 K/V append, the fused form of
// rmsnorm_per_head_batch, rope_partial_batch(_positions), kv_append_batch_paged_device
// (src/kernels_cuda.cu:4622-4645, 4697-4799, 8921-8969).  k_cache/v_cache are fp16 bit arrays.
void orc_qk_norm_rope_append(float *qkv, uint32_t rows, uint32_t row_stride, const float *q_norm_w,
                             const float *k_norm_w, const float *inv_freq, uint32_t n_heads, uint32_t n_kv,
                             uint32_t hd, uint32_t rope_dim, float eps, const int32_t *row_seq,
                             const int32_t *row_pos, const int32_t *page_table, uint32_t pt_stride,
                             uint32_t page_size, uint16_t *k_cache, uint16_t *v_cache) {
    const uint32_t kvd = n_kv * hd;
    for (uint32_t r = 0; r < rows; ++r) {
        float *q = qkv + (size_t)r * row_stride, *k = q + (size_t)n_heads * 2 * hd, *v = k + kvd;
        const int pos = row_pos[r];
        for (uint32_t h = 0; h < n_heads; ++h) { head_norm(q + (size_t)h * 2 * hd, q_norm_w, hd, eps); rope_partial(q + (size_t)h * 2 * hd, rope_dim, pos, inv_freq); }
        for (uint32_t h = 0; h < n_kv; ++h) { head_norm(k + (size_t)h * hd, k_norm_w, hd, eps); rope_partial(k + (size_t)h * hd, rope_dim, pos, inv_freq); }
        const size_t slot = (size_t)page_table[(size_t)row_seq[r] * pt_stride + pos / page_size] * page_size + pos % page_size;
        for (uint32_t i = 0; i < kvd; ++i) { k_cache[slot * kvd + i] = f32_to_f16(k[i]); v_cache[slot * kvd + i] = f32_to_f16(v[i]); }
    }
}

void orc_attention_paged_gated(const float *qkv, uint32_t rows, uint32_t row_stride, uint32_t n_heads, uint32_t n_kv,
                               uint32_t hd, const int32_t *row_seq, const int32_t *row_pos, const int32_t *page_table,
                               uint32_t pt_stride, uint32_t page_size, const uint16_t *k_cache,
                               const uint16_t *v_cache, float *out) {
#pragma omp parallel for schedule(dynamic)
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        const int32_t *pt = page_table + (size_t)row_seq[r] * pt_stride;
        attention_row(qkv + (size_t)r * row_stride, n_heads, n_kv, hd, (uint32_t)row_pos[r] + 1, k_cache, v_cache,
                      [&](uint32_t t) { return (uint32_t)pt[t / page_size] * page_size + t % page_size; },
                      out + (size_t)r * n_heads * hd);
    }
}

// T rows of one sequence; slots laid out as in qb_deltanet_rows.
void orc_deltanet_rows(const float *proj, uint32_t T, uint32_t proj_stride, const float *conv_w, const float *ssm_a,
                       const float *dt_bias, const float *norm_w, uint32_t nk, uint32_t nv, uint32_t hd, float eps,
                       float *state, float *conv, uint32_t n_slots, uint32_t slot_in, int write_all, float *core) {
    const DnShape d{nk, nv, hd, 4};
    const uint32_t C = d.qkv_dim(), vdim = nv * hd;
    const size_t ssz = (size_t)nv * hd * hd, csz = (size_t)C * 3;
    std::vector<float> S(state + slot_in * ssz, state + (slot_in + 1) * ssz), Cv(conv + slot_in * csz, conv + (slot_in + 1) * csz);
    for (uint32_t t = 0; t < T; ++t) {
        const float *row = proj + (size_t)t * proj_stride;
        deltanet_row(d, row, row + C, row + C + vdim, row + C + vdim + nv, conv_w, ssm_a, dt_bias, norm_w, eps,
                     S.data(), Cv.data(), core + (size_t)t * vdim);
        if (write_all && t < n_slots) { memcpy(state + t * ssz, S.data(), ssz * 4); memcpy(conv + t * csz, Cv.data(), csz * 4); }
    }
    if (!write_all) { memcpy(state, S.data(), ssz * 4); memcpy(conv, Cv.data(), csz * 4); }
}


// ---- sampling-mode acceptance ---------------------------------------------------------------
// sampling_distribution (src/qwen_native_backend.cpp:282-370): softmax(logits / temp) with the denominator summed in
// double, then top-k, min-p and nucleus truncation, each keeping a prefix of the descending order, renormalised over the
// kept set.  The reference isolates a growing window with nth_element; sorting the whole row gives the same kept set.
// Equal logits are ordered lowest index first here (the reference leaves their order to nth_element / sort).
static void sampling_distribution(const float *logits, int n, float temp, float top_p, int top_k, float min_p,
                                  std::vector<float> &out) {
    out.assign((size_t)n, 0.0f);
    const float inv_t = 1.0f / (temp > 0.0f ? temp : 1.0f);
    float maxv = logits[0];
    for (int i = 1; i < n; ++i) if (logits[i] > maxv) maxv = logits[i];
    double sum = 0.0;
    for (int i = 0; i < n; ++i) sum += std::exp((logits[i] - maxv) * inv_t);
    const float norm = (float)(1.0 / (sum > 0.0 ? sum : 1.0));
    auto prob_of = [&](int i) -> float { return std::exp((logits[i] - maxv) * inv_t) * norm; };
    const bool need_sort = (top_k > 0 && top_k < n) || (top_p < 1.0f && top_p > 0.0f) || (min_p > 0.0f);
    if (!need_sort) { for (int i = 0; i < n; ++i) out[i] = prob_of(i); return; }
    std::vector<int> idx((size_t)n);
    for (int i = 0; i < n; ++i) idx[i] = i;
    std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return logits[a] > logits[b]; });
    size_t keep = (size_t)n;
    if (top_k > 0 && (size_t)top_k < keep) keep = (size_t)top_k;
    if (min_p > 0.0f && keep > 0) {
        const float cutoff = prob_of(idx[0]) * min_p;
        size_t k = 0;
        while (k < keep && prob_of(idx[k]) >= cutoff) ++k;
        keep = k;
    }
    if (top_p < 1.0f && top_p > 0.0f) {
        double cum = 0.0;
        size_t k = keep;
        for (size_t i = 0; i < keep; ++i) { cum += prob_of(idx[i]); if (cum >= top_p) { k = i + 1; break; } }
        keep = k;
    }
    double kept_sum = 0.0;
    for (size_t i = 0; i < keep; ++i) kept_sum += prob_of(idx[i]);
    if (kept_sum <= 0.0) { out[idx[0]] = 1.0f; return; }
    const float kn = (float)(1.0 / kept_sum);
    for (size_t i = 0; i < keep; ++i) out[idx[i]] = prob_of(idx[i]) * kn;
}

// sample_from (:373-383) with the draw given: std::discrete_distribution over the nonzero entries in index order, i.e.
// weights divided by their sum, partial sums, the last forced to 1, first entry whose partial sum is >= u (libstdc++).
static int32_t sample_from_u(const std::vector<float> &probs, double u) {
    std::vector<double> w;
    std::vector<int> idx;
    for (int i = 0; i < (int)probs.size(); ++i) if (probs[i] > 0.0f) { w.push_back(probs[i]); idx.push_back(i); }
    if (w.empty()) return -1;
    if (w.size() < 2) return idx[0];
    double s = 0.0;
    for (double v : w) s += v;
    double c = 0.0;
    for (size_t j = 0; j < w.size(); ++j) {
        c += w[j] / s;
        if ((j + 1 == w.size() ? 1.0 : c) >= u) return idx[j];
    }
    return idx.back();
}

// One row of speculative_accept_pointmass (:399-467) without penalties: draft >= 0: accept with probability p[draft], on
// rejection draw from p with the draft removed (the draft itself if nothing is left); draft < 0: a plain draw from p.
void orc_sample_rows(const float *logits, uint32_t rows, uint32_t V, uint32_t stride, const int32_t *draft, const double *u_acc,
                     const double *u_res, float temp, float top_p, int32_t top_k, float min_p, int32_t *token,
                     int32_t *accepted, float *p_draft) {
#pragma omp parallel for schedule(dynamic)
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        std::vector<float> p;
        sampling_distribution(logits + (size_t)r * stride, (int)V, temp, top_p, top_k, min_p, p);
        const int d = draft ? draft[r] : -1;
        int acc = 0;
        float pd = 0.0f;
        int32_t tok = d;
        if (d >= 0 && (uint32_t)d < V) {
            pd = p[d];
            acc = u_acc[r] < (double)pd ? 1 : 0;
        }
        if (!acc) {
            if (d >= 0 && (uint32_t)d < V) p[d] = 0.0f;
            const int32_t s = sample_from_u(p, u_res[r]);
            tok = s >= 0 ? s : d;
        }
        token[r] = tok;
        if (accepted) accepted[r] = acc;
        if (p_draft) p_draft[r] = pd;
    }
}

// The distribution itself (one row), for the tests that pin it against the reference's function.
void orc_sampling_distribution(const float *logits, uint32_t V, float temp, float top_p, int32_t top_k, float min_p, float *out) {
    std::vector<float> p;
    sampling_distribution(logits, (int)V, temp, top_p, top_k, min_p, p);
    memcpy(out, p.data(), (size_t)V * sizeof(float));
}

void orc_argmax_rows(const float *x, uint32_t M, uint32_t n, uint32_t stride, int32_t *out) {
    for (uint32_t m = 0; m < M; ++m) out[m] = argmax(x + (size_t)m * stride, n);
}

// ---- model-level ---------------------------------------------------------------------------

void *orc_model_create(const qb_model_config *cfg, uint64_t seed, int32_t max_layers) {
    Model *m = new Model();
    m->cfg = *cfg;
    if (max_layers >= 0 && (uint32_t)max_layers < m->cfg.n_layers) m->cfg.n_layers = (uint32_t)max_layers;
    const auto &c = m->cfg;
    m->ones.assign(std::max({c.n_embd, c.head_dim, c.ssm_head_dim}), 1.0f);
    make_inv_freq(c.rope_dim, c.rope_theta, m->inv_freq);
    m->layers.resize(c.n_layers + (c.mtp_layers ? 1 : 0));
    for (uint32_t il = 0; il < c.n_layers; ++il) build_layer(*m, m->layers[il], il, !m->is_attn(il), seed);
    if (c.mtp_layers) {
        // the MTP block keeps the layer index n_layers of the full model (blk.<n_layers>.nextn.*,
        // src/qwen_native.cpp:271-298)
        build_layer(*m, m->layers[c.n_layers], cfg->n_layers, false, seed);
        q8_synth(seed, tid(cfg->n_layers, T_EH_PROJ), c.n_embd, 2 * c.n_embd, c.weight_sigma, m->eh_proj);
    }
    q8_synth(seed, tid(0xFFFF, T_TOKEN_EMBD), c.vocab_size, c.n_embd, c.weight_sigma, m->token_embd);
    q8_synth(seed, tid(0xFFFF, T_OUTPUT), c.vocab_size, c.n_embd, c.weight_sigma, m->output);
    for (Layer &L : m->layers) {
        L.attn_norm.assign(c.n_embd, 1.0f); L.ffn_norm.assign(c.n_embd, 1.0f);
        L.q_norm.assign(c.head_dim, 1.0f); L.k_norm.assign(c.head_dim, 1.0f); L.ssm_norm.assign(c.ssm_head_dim, 1.0f);
    }
    m->output_norm.assign(c.n_embd, 1.0f); m->enorm = m->hnorm = m->shared_head_norm = m->output_norm;
    return m;
}

// A model from named host tensors (the GGUF tensor set the reference binds, src/qwen_native.cpp:147-190 and
// :271-298; same descriptor as the product's qb_model_create).  Returns null when a tensor is missing or mis-shaped.
void *orc_model_create_tensors(const qb_model_config *cfg, const qb_tensor_desc *t, size_t n) {
    auto find = [&](const std::string &name) -> const qb_tensor_desc * {
        for (size_t i = 0; i < n; ++i) if (name == t[i].name) return &t[i];
        return nullptr;
    };
    bool ok = true;
    auto q8 = [&](const std::string &name, uint32_t rows, uint32_t cols, Q8 &w) {
        const qb_tensor_desc *d = find(name);
        if (!d || d->type != QB_TENSOR_Q8_0 || d->rows != rows || d->cols != cols) { fprintf(stderr, "oracle: bad tensor %s\n", name.c_str()); ok = false; return; }
        q8_from_blocks((const uint8_t *)d->data, rows, cols, w);
    };
    auto f32 = [&](const std::string &name, size_t count, std::vector<float> &v, const std::string &alt = "") {
        const qb_tensor_desc *d = find(name);
        if (!d && !alt.empty()) d = find(alt);
        if (!d || d->type != QB_TENSOR_F32 || d->rows * d->cols != count) { fprintf(stderr, "oracle: bad tensor %s\n", name.c_str()); ok = false; return; }
        v.assign((const float *)d->data, (const float *)d->data + count);
    };
    Model *m = new Model();
    m->cfg = *cfg;
    const auto &c = m->cfg;
    const uint32_t H = c.n_embd, V = c.vocab_size;
    m->ones.assign(std::max({c.n_embd, c.head_dim, c.ssm_head_dim}), 1.0f);
    make_inv_freq(c.rope_dim, c.rope_theta, m->inv_freq);
    m->layers.resize(c.n_layers + (c.mtp_layers ? 1 : 0));
    auto bind = [&](Layer &L, uint32_t il, bool recurrent) {
        const std::string b = "blk." + std::to_string(il) + ".";
        L.recurrent = recurrent;
        f32(b + "attn_norm.weight", H, L.attn_norm);
        f32(b + "ffn_norm.weight", H, L.ffn_norm, b + "post_attention_norm.weight");
        if (!recurrent) {
            const uint32_t inner = c.n_heads * c.head_dim, kvd = c.n_kv_heads * c.head_dim;
            q8(b + "attn_q.weight", 2 * inner, H, L.attn_q); q8(b + "attn_k.weight", kvd, H, L.attn_k);
            q8(b + "attn_v.weight", kvd, H, L.attn_v); q8(b + "attn_output.weight", H, inner, L.attn_out);
            f32(b + "attn_q_norm.weight", c.head_dim, L.q_norm); f32(b + "attn_k_norm.weight", c.head_dim, L.k_norm);
        } else {
            const DnShape d = m->dn();
            const uint32_t vdim = d.nv * d.hd;
            q8(b + "attn_qkv.weight", d.qkv_dim(), H, L.ssm_qkv); q8(b + "attn_gate.weight", vdim, H, L.ssm_z);
            q8(b + "ssm_alpha.weight", d.nv, H, L.ssm_alpha); q8(b + "ssm_beta.weight", d.nv, H, L.ssm_beta);
            q8(b + "ssm_out.weight", H, vdim, L.ssm_out);
            f32(b + "ssm_conv1d.weight", (size_t)d.qkv_dim() * d.conv_k, L.conv_w);
            f32(b + "ssm_a", d.nv, L.ssm_a); f32(b + "ssm_dt.bias", d.nv, L.dt_bias); f32(b + "ssm_norm.weight", d.hd, L.ssm_norm);
        }
        q8(b + "ffn_gate.weight", c.n_ff, H, L.ffn_gate); q8(b + "ffn_up.weight", c.n_ff, H, L.ffn_up);
        q8(b + "ffn_down.weight", H, c.n_ff, L.ffn_down);
    };
    for (uint32_t il = 0; il < c.n_layers; ++il) bind(m->layers[il], il, find("blk." + std::to_string(il) + ".attn_q.weight") == nullptr);
    q8("token_embd.weight", V, H, m->token_embd);
    if (find("output.weight")) q8("output.weight", V, H, m->output); else m->output = m->token_embd;
    f32("output_norm.weight", H, m->output_norm);
    m->enorm = m->hnorm = m->ones; m->enorm.resize(H); m->hnorm.resize(H);
    m->shared_head_norm = m->output_norm;
    if (c.mtp_layers) {
        const uint32_t il = c.n_layers;
        const std::string b = "blk." + std::to_string(il) + ".nextn.";
        bind(m->layers[il], il, false);
        q8(b + "eh_proj.weight", H, 2 * H, m->eh_proj);
        f32(b + "enorm.weight", H, m->enorm); f32(b + "hnorm.weight", H, m->hnorm);
        if (find(b + "shared_head_norm.weight")) f32(b + "shared_head_norm.weight", H, m->shared_head_norm);
        if (find(b + "embed_tokens.weight")) q8(b + "embed_tokens.weight", V, H, m->mtp_embd);
        if (find(b + "shared_head_head.weight")) q8(b + "shared_head_head.weight", V, H, m->mtp_head);
    }
    if (!ok) { delete m; return nullptr; }
    return m;
}
void orc_model_destroy(void *mp) { delete (Model *)mp; }
// Moves every gain of one layer's attn_norm by `ulps` units in the last place: the smallest change an equally valid
// fp32 implementation could make.  The tests measure how far the logits move under it (the int8 re-quantisation of
// the activations before every projection turns it into rounding flips), i.e. the noise floor of the model itself.
void orc_model_nudge_attn_norm(void *mp, uint32_t layer, int32_t ulps) {
    Model *m = (Model *)mp;
    if (layer >= m->layers.size()) return;
    for (float &g : m->layers[layer].attn_norm)
        for (int32_t i = 0; i < (ulps < 0 ? -ulps : ulps); ++i) g = std::nextafterf(g, ulps > 0 ? 2.0f * g + 1.0f : -1.0f);
}

void *orc_seq_create(void *mp, uint32_t max_ctx) {
    const Model *m = (const Model *)mp;
    Seq *s = new Seq();
    s->m = m; s->max_ctx = max_ctx;
    const uint32_t L = m->cfg.n_layers;
    s->kc.resize(L); s->vc.resize(L); s->state.resize(L); s->conv.resize(L);
    const DnShape d = m->dn();
    for (uint32_t il = 0; il < L; ++il)
        if (m->layers[il].recurrent) {
            s->state[il].assign((size_t)d.nv * d.hd * d.hd, 0.0f);
            s->conv[il].assign((size_t)d.qkv_dim() * (d.conv_k - 1), 0.0f);
        }
    s->h_prev.assign(m->cfg.n_embd, 0.0f);
    return s;
}
void orc_seq_destroy(void *sp) { delete (Seq *)sp; }
int orc_seq_position(void *sp) { return ((Seq *)sp)->pos; }
int orc_seq_cur_token(void *sp) { return ((Seq *)sp)->cur_tok; }
void orc_seq_set_cur_token(void *sp, int tok) { ((Seq *)sp)->cur_tok = tok; }

// Prompt ingestion (generate_mtp prefill loop src/qwen_native_backend.cpp:12772-12821 +
// prime_mtp_prefix src/qwen_executor.cpp:22543-22815): chunked target forward, MTP K/V for
// position p from (token_p, hidden_{p-1}) with a zero hidden before position 0; next token =
// argmax of the last row.
void orc_prefill(void *sp, const int32_t *tokens, uint32_t n, uint32_t chunk) {
    Seq &s = *(Seq *)sp;
    const Model &m = *s.m;
    const uint32_t H = m.cfg.n_embd;
    if (chunk == 0) chunk = n;
    for (uint32_t off = 0; off < n; off += chunk) {
        const uint32_t M = std::min(chunk, n - off);
        const bool last = off + M == n;
        std::vector<float> hidden, logits;
        target_forward(s, tokens + off, M, s.pos, hidden, last ? &logits : nullptr, M - 1, nullptr);
        if (m.cfg.mtp_layers) {
            std::vector<float> hp((size_t)M * H);
            memcpy(hp.data(), s.h_prev.data(), H * 4);
            if (M > 1) memcpy(hp.data() + H, hidden.data(), (size_t)(M - 1) * H * 4);
            mtp_rows(s, tokens + off, hp.data(), M, s.pos, true, nullptr, nullptr);
        }
        memcpy(s.h_prev.data(), &hidden[(size_t)(M - 1) * H], H * 4);
        s.pos += (int)M;
        if (last) { s.cur_tok = argmax(logits.data(), m.cfg.vocab_size); s.last_logits = logits; s.last_rows = 1; }
    }
}

// generate_plain step (forward_one_token, src/qwen_executor.cpp:5446-5816): forward the current
// token, next token = argmax.  Returns the emitted token.
int orc_greedy_step(void *sp) {
    Seq &s = *(Seq *)sp;
    std::vector<float> hidden, logits;
    const int tok = s.cur_tok;
    target_forward(s, &tok, 1, s.pos, hidden, &logits, 0, nullptr);
    s.h_prev = hidden;
    s.pos += 1;
    s.cur_tok = argmax(logits.data(), s.m->cfg.vocab_size);
    s.last_logits = logits; s.last_rows = 1;
    return s.cur_tok;
}

// One speculative step (src/qwen_native_backend.cpp:15770-16177):
//   draft chain (src/qwen_executor.cpp:6942-7023), verify rows [cur, d1..dk], accept the longest
//   prefix with argmax(row_i) == d_{i+1}, emit accepted drafts + argmax(row_accepted), restore the
//   checkpoint of row `accepted`, rebuild MTP K/V for the committed positions.
// forced_drafts (k ints) replaces the MTP drafts when non-null.  out_tokens gets n_out <= k+1 ids.
int orc_mtp_step(void *sp, uint32_t k, const int32_t *forced_drafts, int32_t *out_tokens, int32_t *drafts_out,
                 int32_t *row_argmax_out) {
    Seq &s = *(Seq *)sp;
    const Model &m = *s.m;
    const uint32_t H = m.cfg.n_embd, V = m.cfg.vocab_size;
    const int base = s.pos;
    std::vector<int> toks(k + 1);
    toks[0] = s.cur_tok;
    {   // draft chain: step i feeds (i==0 ? cur : draft_i, i==0 ? h_prev : mtp_h) at position base+i
        std::vector<float> hin = s.h_prev, mtp_h, logits;
        int tok = s.cur_tok;
        for (uint32_t i = 0; i < k; ++i) {
            mtp_rows(s, &tok, hin.data(), 1, base + (int)i, false, &mtp_h, &logits);
            tok = argmax(logits.data(), V);
            toks[i + 1] = tok;
            hin = mtp_h;
        }
    }
    if (forced_drafts) for (uint32_t i = 0; i < k; ++i) toks[i + 1] = forced_drafts[i];
    if (drafts_out) for (uint32_t i = 0; i < k; ++i) drafts_out[i] = toks[i + 1];

    // verify
    std::vector<std::vector<float>> st0 = s.state, cv0 = s.conv;
    std::vector<float> hidden, logits;
    RowCheckpoints ck;
    target_forward(s, toks.data(), k + 1, base, hidden, &logits, 0, &ck);
    std::vector<int> am(k + 1);
    for (uint32_t r = 0; r <= k; ++r) am[r] = argmax(&logits[(size_t)r * V], V);
    if (row_argmax_out) for (uint32_t r = 0; r <= k; ++r) row_argmax_out[r] = am[r];
    uint32_t a = 0;
    while (a < k && am[a] == toks[a + 1]) ++a;
    for (uint32_t i = 0; i < a; ++i) out_tokens[i] = toks[i + 1];
    out_tokens[a] = am[a];
    // commit / rollback: state after row a (restore_state_checkpoint, src/qwen_executor.cpp:22304-22428)
    for (uint32_t il = 0; il < m.cfg.n_layers; ++il)
        if (m.layers[il].recurrent) { s.state[il] = ck.state[il][a]; s.conv[il] = ck.conv[il][a]; }
    // MTP K/V of positions base+1..base+a from (d_i, hidden row i-1); position base was written by draft 0
    if (a > 0) mtp_rows(s, toks.data() + 1, hidden.data(), a, base + 1, true, nullptr, nullptr);
    memcpy(s.h_prev.data(), &hidden[(size_t)a * H], H * 4);
    s.pos = base + (int)a + 1;
    s.cur_tok = am[a];
    s.last_logits = logits; s.last_rows = k + 1;
    s.last_hidden = hidden;
    return (int)a + 1;
}

uint32_t orc_last_logits(void *sp, float *out, uint32_t max_rows) {
    Seq &s = *(Seq *)sp;
    const uint32_t r = std::min(max_rows, s.last_rows);
    memcpy(out, s.last_logits.data(), (size_t)r * s.m->cfg.vocab_size * 4);
    return r;
}

// Teacher-forced target forward of M rows without committing anything except K/V and state of
// those rows (used to time and to compare logits on given tokens).
void orc_forward_rows(void *sp, const int32_t *tokens, uint32_t M, float *logits_out, float *hidden_out) {
    Seq &s = *(Seq *)sp;
    std::vector<float> hidden, logits;
    target_forward(s, tokens, M, s.pos, hidden, logits_out ? &logits : nullptr, 0, nullptr);
    if (logits_out) memcpy(logits_out, logits.data(), logits.size() * 4);
    if (hidden_out) memcpy(hidden_out, hidden.data(), hidden.size() * 4);
    memcpy(s.h_prev.data(), &hidden[(size_t)(M - 1) * s.m->cfg.n_embd], s.m->cfg.n_embd * 4);
    s.pos += (int)M;
}

// Seeded prompt: uniform token ids in [0, vocab).
void orc_synth_prompt(uint64_t seed, uint32_t vocab, uint32_t n, int32_t *out) {
    for (uint32_t i = 0; i < n; ++i) out[i] = (int32_t)(qs_rand_u32(seed, 0x7011u, i) % vocab);
}

// Raw draws of the seeded generator (stream = tensor id): lets the test-side checkpoint writer rebuild the small fp32
// tensors of the seeded model (ssm_a, dt_bias, conv1d) with the recipe of build_layer.
void orc_rand_u32(uint64_t seed, uint32_t stream, uint64_t i0, uint64_t n, uint32_t *out) {
    for (uint64_t i = 0; i < n; ++i) out[i] = qs_rand_u32(seed, stream, i0 + i);
}

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
