// Host-side executor of the qwen35 MTP speculative-decode step.
//
// Mirrors the part of QwenExecutor / QwenNativeBackend that drives this path in the reference:
//   forward_n_tokens                      src/qwen_executor.cpp:6003-6836  (prefill + verify rows)
//   forward_one_token                     src/qwen_executor.cpp:5446-5816  (plain greedy step)
//   forward_mtp_draft_chain_with_prefix_device / forward_mtp_draft_from   :6942-7255
//   prime_mtp_prefix_from_last_batch_at   :22543-22815
//   restore_state_checkpoint              :22304-22428
//   the speculative loop and acceptance   src/qwen_native_backend.cpp:15770-16177
// All per-step control values (positions, selected state slot, current token, drafts) live in
// device memory and are updated by kernels, so a step needs no host decision and no mid-step
// synchronisation; the host reads back one small record per step.
#include "qb_internal.h"
#include "page_pool.h"

#include <string>

namespace {

enum TensorKind : uint32_t {
    T_ATTN_Q = 1, T_ATTN_K, T_ATTN_V, T_ATTN_OUT, T_FFN_GATE, T_FFN_UP, T_FFN_DOWN,
    T_SSM_QKV, T_SSM_Z, T_SSM_ALPHA, T_SSM_BETA, T_SSM_OUT, T_SSM_CONV, T_SSM_A, T_SSM_DT,
    T_EH_PROJ, T_TOKEN_EMBD, T_OUTPUT
};
inline uint32_t tensor_id(uint32_t layer, uint32_t kind) { return layer * 32u + kind; }
inline double urand(uint64_t seed, uint32_t stream, uint64_t i) {
    return (double)(qs_rand_u32(seed, stream, i) >> 8) / 16777216.0;
}

struct LayerW {
    bool recurrent = false;
    qb_weight *w_in = nullptr;       // attention: [q(+gate) ; k ; v]   DeltaNet: [qkv ; z ; alpha ; beta]
    qb_weight *w_out = nullptr;      // attn_output / ssm_out
    qb_weight *w_gate_up = nullptr;  // [gate ; up]
    qb_weight *w_down = nullptr;
    qb_weight w_kv;                  // view of the k and v rows of w_in (attention layers)
    float *conv_w = nullptr, *ssm_a = nullptr, *dt_bias = nullptr;
    // RMSNorm gains (attn_norm, ffn_norm / post_attention_norm, attn_q_norm, attn_k_norm, ssm_norm)
    const float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr, *ssm_norm = nullptr;
};

}  // namespace

struct qb_model {
    qb_model_config cfg;
    std::vector<LayerW> layers;      // n_layers (+ the MTP layer last)
    qb_weight *token_embd = nullptr, *output = nullptr, *eh_proj = nullptr;
    // MTP head: embedding table and LM head (nextn.embed_tokens / nextn.shared_head_head, else the target's)
    qb_weight *mtp_embd = nullptr, *mtp_head = nullptr;
    bool output_tied = false;        // no output.weight: the LM head is token_embd
    uint32_t tp_rank = 0, tp_world = 1;   // FFN weights are shard tp_rank of tp_world (tensor-parallel form), else whole
    float *ones = nullptr;           // every RMSNorm gain of the seeded model is 1.0
    const float *output_norm = nullptr, *enorm = nullptr, *hnorm = nullptr, *shared_head_norm = nullptr;
    std::vector<float *> owned_f32;  // fp32 tensors uploaded for this model
    float *inv_freq = nullptr;
    size_t weight_bytes = 0;
    uint32_t inner() const { return cfg.n_heads * cfg.head_dim; }
    uint32_t kvd() const { return cfg.n_kv_heads * cfg.head_dim; }
    uint32_t attn_in() const { return 2 * inner() + 2 * kvd(); }
    uint32_t qkv_dim() const { return (2 * cfg.ssm_num_k_heads + cfg.ssm_num_v_heads) * cfg.ssm_head_dim; }
    uint32_t vdim() const { return cfg.ssm_num_v_heads * cfg.ssm_head_dim; }
    uint32_t dn_in() const { return qkv_dim() + vdim() + 2 * cfg.ssm_num_v_heads; }
    bool is_attn(uint32_t i) const { return cfg.full_attention_interval && ((i + 1) % cfg.full_attention_interval) == 0; }
};

static size_t weight_bytes_of(const qb_weight *w) { return (size_t)w->rows * w->cols / 32 * 34; }

static int upload_f32(qb_ctx *ctx, const std::vector<float> &v, float **out) {
    QB_CUDA(cudaMalloc(out, v.size() * sizeof(float)));
    QB_CUDA(cudaMemcpyAsync(*out, v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    return QB_OK;
}

static int build_layer(qb_ctx *ctx, qb_model *m, LayerW &L, uint32_t il, bool recurrent, uint64_t seed) {
    const qb_model_config &c = m->cfg;
    const float sg = c.weight_sigma;
    L.recurrent = recurrent;
    if (!recurrent) {
        const uint32_t inner = m->inner(), kvd = m->kvd();
        QB_TRY(qb_weight_alloc(ctx, m->attn_in(), c.n_embd, &L.w_in));
        QB_TRY(qb_weight_fill_synth(ctx, L.w_in, 0, 2 * inner, seed, tensor_id(il, T_ATTN_Q), sg));
        QB_TRY(qb_weight_fill_synth(ctx, L.w_in, 2 * inner, kvd, seed, tensor_id(il, T_ATTN_K), sg));
        QB_TRY(qb_weight_fill_synth(ctx, L.w_in, 2 * inner + kvd, kvd, seed, tensor_id(il, T_ATTN_V), sg));
        QB_REQUIRE((2 * inner) % 128 == 0, "attention q rows %u not a multiple of 128", 2 * inner);
        QB_TRY(qb_weight_view(ctx, L.w_in, 2 * inner, 2 * kvd, &L.w_kv));
        QB_TRY(qb_weight_alloc(ctx, c.n_embd, inner, &L.w_out));
        QB_TRY(qb_weight_fill_synth(ctx, L.w_out, 0, c.n_embd, seed, tensor_id(il, T_ATTN_OUT), sg));
    } else {
        const uint32_t C = m->qkv_dim(), vdim = m->vdim(), nv = c.ssm_num_v_heads;
        QB_TRY(qb_weight_alloc(ctx, m->dn_in(), c.n_embd, &L.w_in));
        QB_TRY(qb_weight_fill_synth(ctx, L.w_in, 0, C, seed, tensor_id(il, T_SSM_QKV), sg));
        QB_TRY(qb_weight_fill_synth(ctx, L.w_in, C, vdim, seed, tensor_id(il, T_SSM_Z), sg));
        QB_TRY(qb_weight_fill_synth(ctx, L.w_in, C + vdim, nv, seed, tensor_id(il, T_SSM_ALPHA), sg));
        QB_TRY(qb_weight_fill_synth(ctx, L.w_in, C + vdim + nv, nv, seed, tensor_id(il, T_SSM_BETA), sg));
        QB_TRY(qb_weight_alloc(ctx, c.n_embd, vdim, &L.w_out));
        QB_TRY(qb_weight_fill_synth(ctx, L.w_out, 0, c.n_embd, seed, tensor_id(il, T_SSM_OUT), sg));
        // fp32 DeltaNet tensors: ssm_a = -exp(U(0, log 16)), dt_bias ~ U(-4,-1), conv1d ~ U(-0.5,0.5)
        std::vector<float> conv((size_t)C * c.ssm_conv_kernel), sa(nv), dt(nv);
        for (size_t i = 0; i < conv.size(); ++i) conv[i] = (float)((urand(seed, tensor_id(il, T_SSM_CONV), i) * 2.0 - 1.0) * 0.5);
        for (uint32_t v = 0; v < nv; ++v) {
            sa[v] = (float)(-std::exp(urand(seed, tensor_id(il, T_SSM_A), v) * std::log(16.0)));
            dt[v] = (float)(-4.0 + 3.0 * urand(seed, tensor_id(il, T_SSM_DT), v));
        }
        QB_TRY(upload_f32(ctx, conv, &L.conv_w));
        QB_TRY(upload_f32(ctx, sa, &L.ssm_a));
        QB_TRY(upload_f32(ctx, dt, &L.dt_bias));
    }
    // gate and up interleaved in groups of 64 rows: a 128-row tile holds both halves of 64 hidden indices.  In the
    // tensor-parallel form this rank holds FFN indices [lo, lo + f): those rows of gate and up, those columns of down.
    QB_REQUIRE(c.n_ff % (64 * m->tp_world) == 0 && (c.n_ff / m->tp_world) % 128 == 0, "model: FFN dimension %u does not split into %u shards of whole tiles",
               c.n_ff, m->tp_world);
    const uint32_t f = c.n_ff / m->tp_world, lo = m->tp_rank * f;
    QB_TRY(qb_weight_alloc(ctx, 2 * f, c.n_embd, &L.w_gate_up));
    QB_TRY(qb_weight_fill_synth_window(ctx, L.w_gate_up, 0, f, seed, tensor_id(il, T_FFN_GATE), sg, 64, lo, c.n_embd / 32, 0));
    QB_TRY(qb_weight_fill_synth_window(ctx, L.w_gate_up, 64, f, seed, tensor_id(il, T_FFN_UP), sg, 64, lo, c.n_embd / 32, 0));
    QB_TRY(qb_weight_alloc(ctx, c.n_embd, f, &L.w_down));
    QB_TRY(qb_weight_fill_synth_window(ctx, L.w_down, 0, c.n_embd, seed, tensor_id(il, T_FFN_DOWN), sg, 0, 0, c.n_ff / 32, lo / 32));
    m->weight_bytes += weight_bytes_of(L.w_in) + weight_bytes_of(L.w_out) + weight_bytes_of(L.w_gate_up) + weight_bytes_of(L.w_down);
    return QB_OK;
}

extern "C" void qb_model_destroy(qb_ctx *ctx, qb_model *m);

// Shape checks shared by every model constructor, the all-ones gain vector and the RoPE frequencies.
static int model_begin(qb_ctx *ctx, const qb_model_config &c, qb_model **out) {
    QB_REQUIRE(c.n_layers > 0 && c.n_embd % 128 == 0 && c.n_ff % 128 == 0, "n_embd and n_ff must be multiples of 128");
    QB_REQUIRE(c.head_dim == 64 || c.head_dim == 128 || c.head_dim == 256, "head_dim must be 64, 128 or 256");
    QB_REQUIRE(c.ssm_head_dim == 64 || c.ssm_head_dim == 128, "ssm_head_dim must be 64 or 128");
    QB_REQUIRE(c.ssm_conv_kernel == 4, "ssm_conv_kernel must be 4");
    QB_REQUIRE(c.n_kv_heads > 0 && c.n_heads % c.n_kv_heads == 0 && c.n_heads / c.n_kv_heads <= 8, "GQA group must divide and be <= 8");
    QB_REQUIRE((c.n_heads * c.head_dim) % 128 == 0 && (c.ssm_num_v_heads * c.ssm_head_dim) % 128 == 0, "inner dims must be multiples of 128");
    QB_REQUIRE(c.mtp_layers <= 1, "at most one MTP layer");
    QB_REQUIRE(c.rope_dim >= 2 && c.rope_dim % 2 == 0 && c.rope_dim <= c.head_dim, "rope_dim must be even and <= head_dim");
    QB_REQUIRE(c.vocab_size > 0, "vocab_size must be positive");
    QB_CUDA(cudaSetDevice(ctx->device));
    qb_model *m = new qb_model();
    m->cfg = c;
    *out = m;
    std::vector<float> ones(std::max({c.n_embd, c.head_dim, c.ssm_head_dim}), 1.0f);
    QB_TRY(upload_f32(ctx, ones, &m->ones));
    std::vector<float> invf(c.rope_dim / 2);
    for (uint32_t i = 0; i < c.rope_dim / 2; ++i) invf[i] = (float)std::pow((double)c.rope_theta, -2.0 * (double)i / (double)c.rope_dim);
    QB_TRY(upload_f32(ctx, invf, &m->inv_freq));
    m->layers.resize(c.n_layers + (c.mtp_layers ? 1 : 0));
    return QB_OK;
}

static int model_create_synth(qb_ctx *ctx, const qb_model_config *cfg, uint64_t seed, uint32_t tp_rank, uint32_t tp_world, qb_model **out);

extern "C" int qb_model_create_synth(qb_ctx *ctx, const qb_model_config *cfg, uint64_t seed, qb_model **out) {
    return model_create_synth(ctx, cfg, seed, 0, 1, out);
}

// The seeded model with its FFN pairs tensor-sharded: rank `rank` of `world` holds gate/up rows and down columns
// [rank * n_ff / world, (rank + 1) * n_ff / world) of every layer (and of the MTP layer); everything else is replicated.
// The shards are windows of the same seeded tensors, so the ranks together hold exactly the model of qb_model_create_synth.
extern "C" int qb_model_create_synth_tp(qb_ctx *ctx, const qb_model_config *cfg, uint64_t seed, uint32_t rank, uint32_t world, qb_model **out) {
    QB_REQUIRE(world >= 1 && world <= 8 && rank < world, "qb_model_create_synth_tp: rank %u of %u (at most 8)", rank, world);
    return model_create_synth(ctx, cfg, seed, rank, world, out);
}

static int model_create_synth(qb_ctx *ctx, const qb_model_config *cfg, uint64_t seed, uint32_t tp_rank, uint32_t tp_world, qb_model **out) {
    QB_REQUIRE(ctx && cfg && out, "qb_model_create_synth: null argument");
    const qb_model_config &c = *cfg;
    qb_model *m = nullptr;
    int st = model_begin(ctx, c, &m);
    if (st != QB_OK) { qb_model_destroy(ctx, m); return st; }
    m->tp_rank = tp_rank; m->tp_world = tp_world;
    auto body = [&]() -> int {
        for (uint32_t il = 0; il < c.n_layers; ++il) QB_TRY(build_layer(ctx, m, m->layers[il], il, !m->is_attn(il), seed));
        if (c.mtp_layers) {
            QB_TRY(build_layer(ctx, m, m->layers[c.n_layers], c.n_layers, false, seed));
            QB_TRY(qb_weight_q8_0_synth(ctx, seed, tensor_id(c.n_layers, T_EH_PROJ), c.n_embd, 2 * c.n_embd, c.weight_sigma, &m->eh_proj));
            m->weight_bytes += weight_bytes_of(m->eh_proj);
        }
        QB_TRY(qb_weight_q8_0_synth(ctx, seed, tensor_id(0xFFFF, T_TOKEN_EMBD), c.vocab_size, c.n_embd, c.weight_sigma, &m->token_embd));
        QB_TRY(qb_weight_q8_0_synth(ctx, seed, tensor_id(0xFFFF, T_OUTPUT), c.vocab_size, c.n_embd, c.weight_sigma, &m->output));
        m->weight_bytes += weight_bytes_of(m->token_embd) + weight_bytes_of(m->output);
        // every RMSNorm gain of the seeded model is 1.0; the MTP head shares the target's embedding and LM head
        for (LayerW &L : m->layers) L.attn_norm = L.ffn_norm = L.q_norm = L.k_norm = L.ssm_norm = m->ones;
        m->output_norm = m->enorm = m->hnorm = m->shared_head_norm = m->ones;
        m->mtp_embd = m->token_embd;
        m->mtp_head = m->output;
        QB_CUDA(cudaStreamSynchronize(ctx->stream));
        return QB_OK;
    };
    st = body();
    if (st != QB_OK) { qb_model_destroy(ctx, m); return st; }
    *out = m;
    return QB_OK;
}

// ---- a model from the caller's tensors (the GGUF tensor set of src/qwen_native.cpp:147-190, 271-298) ----
namespace {
struct TensorTable {
    const qb_tensor_desc *t; size_t n;
    const qb_tensor_desc *find(const std::string &name) const {
        for (size_t i = 0; i < n; ++i) if (t[i].name && name == t[i].name) return &t[i];
        return nullptr;
    }
};
std::string blk(uint32_t il, const char *name) { return "blk." + std::to_string(il) + "." + name; }
}  // namespace

static int need_q8(const TensorTable &tt, const std::string &name, uint32_t rows, uint32_t cols, const qb_tensor_desc **out) {
    const qb_tensor_desc *d = tt.find(name);
    if (!d) return qb_fail(QB_ERR_INVALID, "model: tensor %s is missing", name.c_str());
    if (d->type != QB_TENSOR_Q8_0)
        return qb_fail(QB_ERR_UNSUPPORTED, "model: tensor %s has type %u; this path takes Q8_0 (type 8) matrices only", name.c_str(), d->type);
    if (d->rows != rows || d->cols != cols || !d->data)
        return qb_fail(QB_ERR_INVALID, "model: tensor %s is %llu x %llu, expected %u x %u", name.c_str(), (unsigned long long)d->rows,
                       (unsigned long long)d->cols, rows, cols);
    *out = d;
    return QB_OK;
}
static int need_f32(qb_ctx *ctx, qb_model *m, const TensorTable &tt, const std::string &name, const std::string &alt, uint64_t count,
                    const float **out) {
    const qb_tensor_desc *d = tt.find(name);
    if (!d && !alt.empty()) d = tt.find(alt);
    if (!d) return qb_fail(QB_ERR_INVALID, "model: tensor %s is missing", name.c_str());
    if (d->type != QB_TENSOR_F32 || !d->data) return qb_fail(QB_ERR_UNSUPPORTED, "model: tensor %s must be F32 (type 0)", name.c_str());
    if (d->rows * d->cols != count)
        return qb_fail(QB_ERR_INVALID, "model: tensor %s has %llu elements, expected %llu", name.c_str(),
                       (unsigned long long)(d->rows * d->cols), (unsigned long long)count);
    float *dev = nullptr;
    QB_CUDA(cudaMalloc(&dev, count * sizeof(float)));
    m->owned_f32.push_back(dev);
    QB_CUDA(cudaMemcpyAsync(dev, d->data, count * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    *out = dev;
    return QB_OK;
}

static int bind_layer(qb_ctx *ctx, qb_model *m, const TensorTable &tt, LayerW &L, uint32_t il, bool recurrent) {
    const qb_model_config &c = m->cfg;
    const uint32_t H = c.n_embd;
    const qb_tensor_desc *d = nullptr;
    L.recurrent = recurrent;
    QB_TRY(need_f32(ctx, m, tt, blk(il, "attn_norm.weight"), "", H, &L.attn_norm));
    QB_TRY(need_f32(ctx, m, tt, blk(il, "ffn_norm.weight"), blk(il, "post_attention_norm.weight"), H, &L.ffn_norm));
    if (!recurrent) {
        const uint32_t inner = m->inner(), kvd = m->kvd();
        QB_REQUIRE((2 * inner) % 128 == 0, "attention q rows %u not a multiple of 128", 2 * inner);
        QB_TRY(qb_weight_alloc(ctx, m->attn_in(), H, &L.w_in));
        QB_TRY(need_q8(tt, blk(il, "attn_q.weight"), 2 * inner, H, &d));
        QB_TRY(qb_weight_fill_upload(ctx, L.w_in, 0, 2 * inner, d->data));
        QB_TRY(need_q8(tt, blk(il, "attn_k.weight"), kvd, H, &d));
        QB_TRY(qb_weight_fill_upload(ctx, L.w_in, 2 * inner, kvd, d->data));
        QB_TRY(need_q8(tt, blk(il, "attn_v.weight"), kvd, H, &d));
        QB_TRY(qb_weight_fill_upload(ctx, L.w_in, 2 * inner + kvd, kvd, d->data));
        QB_TRY(qb_weight_view(ctx, L.w_in, 2 * inner, 2 * kvd, &L.w_kv));
        QB_TRY(need_q8(tt, blk(il, "attn_output.weight"), H, inner, &d));
        QB_TRY(qb_weight_q8_0(ctx, d->data, H, inner, &L.w_out));
        QB_TRY(need_f32(ctx, m, tt, blk(il, "attn_q_norm.weight"), "", c.head_dim, &L.q_norm));
        QB_TRY(need_f32(ctx, m, tt, blk(il, "attn_k_norm.weight"), "", c.head_dim, &L.k_norm));
    } else {
        const uint32_t C = m->qkv_dim(), vdim = m->vdim(), nv = c.ssm_num_v_heads;
        QB_TRY(qb_weight_alloc(ctx, m->dn_in(), H, &L.w_in));
        QB_TRY(need_q8(tt, blk(il, "attn_qkv.weight"), C, H, &d));
        QB_TRY(qb_weight_fill_upload(ctx, L.w_in, 0, C, d->data));
        QB_TRY(need_q8(tt, blk(il, "attn_gate.weight"), vdim, H, &d));
        QB_TRY(qb_weight_fill_upload(ctx, L.w_in, C, vdim, d->data));
        QB_TRY(need_q8(tt, blk(il, "ssm_alpha.weight"), nv, H, &d));
        QB_TRY(qb_weight_fill_upload(ctx, L.w_in, C + vdim, nv, d->data));
        QB_TRY(need_q8(tt, blk(il, "ssm_beta.weight"), nv, H, &d));
        QB_TRY(qb_weight_fill_upload(ctx, L.w_in, C + vdim + nv, nv, d->data));
        QB_TRY(need_q8(tt, blk(il, "ssm_out.weight"), H, vdim, &d));
        QB_TRY(qb_weight_q8_0(ctx, d->data, H, vdim, &L.w_out));
        const float *p = nullptr;
        QB_TRY(need_f32(ctx, m, tt, blk(il, "ssm_conv1d.weight"), "", (uint64_t)C * c.ssm_conv_kernel, &p)); L.conv_w = const_cast<float *>(p);
        QB_TRY(need_f32(ctx, m, tt, blk(il, "ssm_a"), "", nv, &p)); L.ssm_a = const_cast<float *>(p);
        QB_TRY(need_f32(ctx, m, tt, blk(il, "ssm_dt.bias"), "", nv, &p)); L.dt_bias = const_cast<float *>(p);
        QB_TRY(need_f32(ctx, m, tt, blk(il, "ssm_norm.weight"), "", c.ssm_head_dim, &L.ssm_norm));
    }
    const qb_tensor_desc *g = nullptr, *u = nullptr;
    QB_REQUIRE(c.n_ff % 64 == 0, "model: FFN dimension %u is not a multiple of 64", c.n_ff);
    QB_TRY(need_q8(tt, blk(il, "ffn_gate.weight"), c.n_ff, H, &g));
    QB_TRY(need_q8(tt, blk(il, "ffn_up.weight"), c.n_ff, H, &u));
    QB_TRY(qb_weight_q8_0_gate_up(ctx, g->data, u->data, c.n_ff, H, &L.w_gate_up));
    QB_TRY(need_q8(tt, blk(il, "ffn_down.weight"), H, c.n_ff, &d));
    QB_TRY(qb_weight_q8_0(ctx, d->data, H, c.n_ff, &L.w_down));
    m->weight_bytes += weight_bytes_of(L.w_in) + weight_bytes_of(L.w_out) + weight_bytes_of(L.w_gate_up) + weight_bytes_of(L.w_down);
    return QB_OK;
}

// QwenNativeModel's tensor binding (src/qwen_native.cpp:147-190; MTP block :271-298) and QwenWeights' upload
// (src/qwen_weights.cpp:170-208) from the caller's host tensors.  A layer is full attention when its attn_q.weight
// exists (the reference's rule), which must agree with full_attention_interval.  output.weight falls back to
// token_embd.weight; the MTP head's embedding, LM head and final norm fall back to the target's.
extern "C" int qb_model_create(qb_ctx *ctx, const qb_model_config *cfg, const qb_tensor_desc *tensors, size_t n_tensors, qb_model **out) {
    QB_REQUIRE(ctx && cfg && tensors && out, "qb_model_create: null argument");
    const qb_model_config &c = *cfg;
    qb_model *m = nullptr;
    int st = model_begin(ctx, c, &m);
    if (st != QB_OK) { qb_model_destroy(ctx, m); return st; }
    const TensorTable tt{tensors, n_tensors};
    auto body = [&]() -> int {
        const uint32_t H = c.n_embd, V = c.vocab_size;
        const qb_tensor_desc *d = nullptr;
        for (uint32_t il = 0; il < c.n_layers; ++il) {
            const bool has_q = tt.find(blk(il, "attn_q.weight")) != nullptr;
            QB_REQUIRE(has_q == m->is_attn(il), "model: layer %u %s attn_q.weight but full_attention_interval = %u says otherwise", il,
                       has_q ? "has" : "lacks", c.full_attention_interval);
            QB_TRY(bind_layer(ctx, m, tt, m->layers[il], il, !has_q));
        }
        QB_TRY(need_q8(tt, "token_embd.weight", V, H, &d));
        QB_TRY(qb_weight_q8_0(ctx, d->data, V, H, &m->token_embd));
        m->weight_bytes += weight_bytes_of(m->token_embd);
        if (tt.find("output.weight")) {
            QB_TRY(need_q8(tt, "output.weight", V, H, &d));
            QB_TRY(qb_weight_q8_0(ctx, d->data, V, H, &m->output));
            m->weight_bytes += weight_bytes_of(m->output);
        } else {
            m->output = m->token_embd;
            m->output_tied = true;
        }
        QB_TRY(need_f32(ctx, m, tt, "output_norm.weight", "", H, &m->output_norm));
        m->mtp_embd = m->token_embd; m->mtp_head = m->output; m->shared_head_norm = m->output_norm;
        m->enorm = m->hnorm = m->ones;
        if (c.mtp_layers) {
            const uint32_t il = c.n_layers;
            QB_TRY(bind_layer(ctx, m, tt, m->layers[il], il, false));
            QB_TRY(need_q8(tt, blk(il, "nextn.eh_proj.weight"), H, 2 * H, &d));
            QB_TRY(qb_weight_q8_0(ctx, d->data, H, 2 * H, &m->eh_proj));
            m->weight_bytes += weight_bytes_of(m->eh_proj);
            QB_TRY(need_f32(ctx, m, tt, blk(il, "nextn.enorm.weight"), "", H, &m->enorm));
            QB_TRY(need_f32(ctx, m, tt, blk(il, "nextn.hnorm.weight"), "", H, &m->hnorm));
            if (tt.find(blk(il, "nextn.shared_head_norm.weight")))
                QB_TRY(need_f32(ctx, m, tt, blk(il, "nextn.shared_head_norm.weight"), "", H, &m->shared_head_norm));
            if (tt.find(blk(il, "nextn.embed_tokens.weight"))) {
                QB_TRY(need_q8(tt, blk(il, "nextn.embed_tokens.weight"), V, H, &d));
                QB_TRY(qb_weight_q8_0(ctx, d->data, V, H, &m->mtp_embd));
                m->weight_bytes += weight_bytes_of(m->mtp_embd);
            }
            if (tt.find(blk(il, "nextn.shared_head_head.weight"))) {
                QB_TRY(need_q8(tt, blk(il, "nextn.shared_head_head.weight"), V, H, &d));
                QB_TRY(qb_weight_q8_0(ctx, d->data, V, H, &m->mtp_head));
                m->weight_bytes += weight_bytes_of(m->mtp_head);
            }
        }
        QB_CUDA(cudaStreamSynchronize(ctx->stream));     // the caller's host tensors may go away after the call
        return QB_OK;
    };
    st = body();
    if (st != QB_OK) { qb_model_destroy(ctx, m); return st; }
    *out = m;
    return QB_OK;
}

extern "C" const qb_model_config *qb_model_get_config(const qb_model *m) { return m ? &m->cfg : nullptr; }

extern "C" void qb_model_destroy(qb_ctx *ctx, qb_model *m) {
    if (!m) return;
    cudaStreamSynchronize(ctx->stream);
    std::vector<const float *> owned(m->owned_f32.begin(), m->owned_f32.end());
    auto is_owned = [&](const float *p) { return std::find(owned.begin(), owned.end(), p) != owned.end(); };
    for (LayerW &L : m->layers) {
        qb_weight_free(ctx, L.w_in); qb_weight_free(ctx, L.w_out); qb_weight_free(ctx, L.w_gate_up); qb_weight_free(ctx, L.w_down);
        // the seeded constructor allocates these three itself; qb_model_create keeps them in owned_f32
        if (L.conv_w && !is_owned(L.conv_w)) cudaFree(L.conv_w);
        if (L.ssm_a && !is_owned(L.ssm_a)) cudaFree(L.ssm_a);
        if (L.dt_bias && !is_owned(L.dt_bias)) cudaFree(L.dt_bias);
    }
    if (m->mtp_embd && m->mtp_embd != m->token_embd) qb_weight_free(ctx, m->mtp_embd);
    if (m->mtp_head && m->mtp_head != m->output) qb_weight_free(ctx, m->mtp_head);
    if (!m->output_tied) qb_weight_free(ctx, m->output);
    qb_weight_free(ctx, m->token_embd); qb_weight_free(ctx, m->eh_proj);
    for (float *p : m->owned_f32) cudaFree(p);
    if (m->ones) cudaFree(m->ones);
    if (m->inv_freq) cudaFree(m->inv_freq);
    delete m;
}
extern "C" size_t qb_model_weight_bytes(const qb_model *m) { return m->weight_bytes; }

// ================================================================================================
// sequences
// ================================================================================================
struct QBuf {   // quantised activation buffer for one K
    int8_t *q = nullptr; float *d = nullptr; uint32_t K = 0;
};

struct qb_batch {
    qb_model *m = nullptr;
    uint32_t n_seqs = 0, max_ctx = 0, k = 0, page_size = 0, pages_per_seq = 0, rows_cap = 0, chunk = 0, logit_rows = 0;
    bool attn_tc = false;                  // decode / verify attention on the tensor-memory kernel: decided once, from n_seqs * max_ctx
    uint32_t attn_split = 0;               // keys per attention split of this batch (absolute boundaries): decided once with attn_tc
    uint32_t n_active = 0;                 // the decode steps run sequences [0, n_active); the rest keep their state untouched
    std::vector<__half *> kc, vc;          // per layer (attention layers only), + MTP layer at index n_layers
    std::vector<float *> state, conv;      // per layer (recurrent layers only): [n_seqs][k+1][...]
    std::vector<float *> conv_alt;         // second conv-state buffer: a forward reads one and writes the other
    int conv_par = 0;                      // which of the two holds the valid conv state (the same for all sequences)
    int32_t *page_table = nullptr;         // [n_seqs][pages_per_seq]
    // pooled form (qb_batch_create_pooled): the caches hold pool->total() pages shared by all sequences; a sequence's
    // page-table row grows as its position grows and goes back to the pool at qb_seq_reset
    QbPagePool *pool = nullptr;
    std::vector<std::vector<int32_t>> seq_pages;   // host mirror of the page-table rows (pooled form)
    std::vector<int32_t> chunk_end_pos;            // position after the sequence's last qb_prefill_chunk, -1 once anything else moved it
    // device control block (all int32)
    int32_t *ctl = nullptr;
    int32_t *pos = nullptr, *sel = nullptr, *cur = nullptr, *drafts = nullptr, *zero_sel = nullptr;
    int32_t *tok_buf = nullptr, *seqpos_buf = nullptr, *prefix_pos = nullptr, *prefix_tok = nullptr;
    int32_t *out_rec = nullptr;            // [n_out (n_seqs) | tokens (n_seqs*(k+1)) | pos (n_seqs)]
    int32_t *map_prevh = nullptr, *map_prefix = nullptr, *map_chunk = nullptr, *map_last = nullptr;
    long long *stats = nullptr;            // [QB_STATS]: steps, drafted, accepted, emitted, rejecting steps, -, -, -, then steps by accepted length
    int32_t *out_rec_host = nullptr;       // pinned mirror of out_rec
    // activations
    float *hid = nullptr;                  // [rows_cap + n_seqs][H]; rows rows_cap+s hold prev hidden of seq s
    float *mtp_h = nullptr, *embd = nullptr, *act = nullptr, *parts = nullptr;
    float *logits = nullptr, *am_val = nullptr, *att_acc = nullptr, *att_ml = nullptr;
    int32_t *am_idx = nullptr;
    QBuf xq_h, xq_attn, xq_dn, xq_ffn, xq_cat;
    size_t parts_floats = 0;
    std::vector<int32_t> host_pos;         // upper bound of pos per sequence
    uint32_t last_logit_rows = 0;
    int gemm_impl = 0;
    double *samp_u = nullptr;              // [2][logit_rows]: acceptance draws, then residual draws (sampling mode)
    uint32_t *seen = nullptr;              // [n_seqs][seen_words] bitmap of prompt + emitted tokens (token penalties), or null
    uint32_t seen_words = 0;
    float pen_presence = 0.0f, pen_repetition = 1.0f;
    qb_tp_group *tp = nullptr;             // tensor-parallel FFN group of the batch's model shard, or null
    float *normed = nullptr, *tp_y = nullptr;   // [rows_cap][H]: fp32 FFN input / all-reduced FFN output of the tensor-parallel form
    int32_t *tok_stage = nullptr;          // pinned staging of the prompt tokens being ingested
    int32_t *tok_all = nullptr;            // the same on the device: one copy per call, the chunks index into it
    cudaEvent_t tok_ev = nullptr;          // that copy has landed (the staging area may be rewritten)
    uint32_t tok_stage_cap = 0;
    double *first_draw_stage = nullptr;    // pinned: the first-token draw of a sampled request per sequence
    int32_t *limit = nullptr;              // [n_seqs] device: draft depth of the next step per sequence (<= k)
    int32_t *limit_host = nullptr;         // pinned staging of the same
    int32_t eos_token = -1;                // a draft equal to it ends the chain (-1: none)
    void *swap_tmp = nullptr;              // one sequence's largest per-layer state block (qb_seq_swap)
    size_t swap_bytes = 0;
    // sampled steps: pinned staging ring of the step's draws (a slot is reused when its copy of four steps ago has landed)
    static constexpr int SAMP_RING = 4;
    double *samp_stage = nullptr;
    cudaEvent_t samp_ev[SAMP_RING] = {};
    uint32_t samp_slot = 0;
    // position probe: keeps host_pos near the device's positions when nobody reads the step records (see probe_tick)
    int32_t *probe_host = nullptr;         // pinned [n_seqs]
    cudaEvent_t probe_ev = nullptr;
    bool probe_pending = false;
    int32_t probe_adv = 0;                 // positions enqueued since the probe's copy
    uint32_t steps_since_probe = 0;
};

static size_t ctl_count(const qb_batch *b);
static constexpr size_t QB_STATS = 16;

static int alloc_qbuf(QBuf &b, uint32_t rows, uint32_t K) {
    b.K = K;
    QB_CUDA(cudaMalloc(&b.q, (size_t)rows * K));
    QB_CUDA(cudaMalloc(&b.d, (size_t)(K / 32) * qb_act_ld(rows) * sizeof(float)));
    return QB_OK;
}

static uint32_t env_u32(const char *name, uint32_t dflt) {
    const char *v = getenv(name);
    return (v && *v) ? (uint32_t)strtoul(v, nullptr, 10) : dflt;
}

static int batch_create(qb_ctx *ctx, qb_model *m, uint32_t n_seqs, uint32_t max_ctx, uint32_t draft_k,
                        uint32_t page_size, int page_order, uint32_t pool_pages, qb_batch **out) {
    QB_REQUIRE(ctx && m && out && n_seqs > 0 && max_ctx > 0 && page_size > 0, "qb_batch_create: bad arguments");
    QB_REQUIRE(draft_k <= 7, "draft depth %u unsupported (<= 7)", draft_k);
    QB_REQUIRE(draft_k == 0 || m->cfg.mtp_layers == 1, "draft depth > 0 needs the MTP layer");
    QB_CUDA(cudaSetDevice(ctx->device));
    const qb_model_config &c = m->cfg;
    qb_batch *b = new qb_batch();
    b->m = m; b->n_seqs = n_seqs; b->n_active = n_seqs; b->max_ctx = max_ctx; b->k = draft_k; b->page_size = page_size;
    b->pages_per_seq = (max_ctx + draft_k + 1 + page_size - 1) / page_size;
    b->chunk = std::max(1u, env_u32("QW3B200_PREFILL_CHUNK", 512));
    // The tensor-memory attention kernel wins once a call has enough keys to fill the GPU (one long context, or many
    // sequences) and costs a few microseconds per call below that; the two kernels differ in the last bits, so the choice
    // is a property of the batch (the keys it can hold), the same for every row the batch ever computes.
    b->attn_tc = (uint64_t)n_seqs * max_ctx >= env_u32("QW3B200_ATTN_TC_MIN_KEYS", 16384);
    // Splits of 256 keys where the tensor-memory kernel runs (its tile pair); 128 keys otherwise: a short context then
    // spreads over twice the SMs, each streaming half the K/V bytes (7.87 against 8.01 ms per step at 2 K context).
    {
        const bool tc_shape = (c.head_dim == 256 || c.head_dim == 128) && page_size == 16 && c.n_heads / std::max(1u, c.n_kv_heads) <= 8;
        b->attn_split = b->attn_tc && tc_shape ? 256 : env_u32("QW3B200_ATTN_SPLIT_SMALL", 128);
        if (b->attn_split < 64 || b->attn_split % 64) b->attn_split = 128;
    }
    b->logit_rows = n_seqs * (draft_k + 1);
    b->rows_cap = std::max(b->chunk, b->logit_rows);
    b->gemm_impl = (int)env_u32("QW3B200_GEMM_IMPL", 0);
    const uint32_t H = c.n_embd, K1 = draft_k + 1, L = c.n_layers, rows = b->rows_cap;
    const size_t slots = (size_t)(pool_pages ? pool_pages : n_seqs * b->pages_per_seq) * page_size;
    const uint32_t kvd = m->kvd();
    b->kc.assign(L + 1, nullptr); b->vc.assign(L + 1, nullptr); b->state.assign(L, nullptr); b->conv.assign(L, nullptr); b->conv_alt.assign(L, nullptr);
    for (uint32_t il = 0; il <= L; ++il) {
        const bool attn = il == L ? c.mtp_layers == 1 : m->is_attn(il);
        if (attn) {
            QB_CUDA(cudaMalloc(&b->kc[il], slots * kvd * sizeof(__half)));
            QB_CUDA(cudaMalloc(&b->vc[il], slots * kvd * sizeof(__half)));
            QB_CUDA(cudaMemsetAsync(b->kc[il], 0, slots * kvd * sizeof(__half), ctx->stream));
            QB_CUDA(cudaMemsetAsync(b->vc[il], 0, slots * kvd * sizeof(__half), ctx->stream));
        } else if (il < L) {
            const size_t ssz = (size_t)n_seqs * K1 * c.ssm_num_v_heads * c.ssm_head_dim * c.ssm_head_dim;
            const size_t csz = (size_t)n_seqs * K1 * m->qkv_dim() * 3;
            QB_CUDA(cudaMalloc(&b->state[il], ssz * sizeof(float)));
            QB_CUDA(cudaMalloc(&b->conv[il], csz * sizeof(float)));
            QB_CUDA(cudaMemsetAsync(b->state[il], 0, ssz * sizeof(float), ctx->stream));
            QB_CUDA(cudaMemsetAsync(b->conv[il], 0, csz * sizeof(float), ctx->stream));
            QB_CUDA(cudaMalloc(&b->conv_alt[il], csz * sizeof(float)));
            QB_CUDA(cudaMemsetAsync(b->conv_alt[il], 0, csz * sizeof(float), ctx->stream));
        }
    }
    // page table: identity / reverse / seeded shuffle over the whole pool
    {
        const size_t total = (size_t)n_seqs * b->pages_per_seq;
        std::vector<int32_t> pt(total);
        for (size_t i = 0; i < total; ++i) pt[i] = (int32_t)i;
        if (page_order == 1) std::reverse(pt.begin(), pt.end());
        if (page_order == 2)
            for (size_t i = total - 1; i > 0; --i) std::swap(pt[i], pt[qs_rand_u32(0x9a6e5, 7, i) % (i + 1)]);
        if (pool_pages) {
            // no page is assigned yet: -1 everywhere (the append kernel refuses a negative page and records it)
            std::fill(pt.begin(), pt.end(), -1);
            b->pool = new QbPagePool(pool_pages);
            b->seq_pages.assign(n_seqs, {});
        }
        QB_CUDA(cudaMalloc(&b->page_table, total * sizeof(int32_t)));
        QB_CUDA(cudaMemcpyAsync(b->page_table, pt.data(), total * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
        QB_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    // control block
    {
        b->rows_cap = rows;
        const size_t n = ctl_count(b);
        QB_CUDA(cudaMalloc(&b->ctl, n * sizeof(int32_t)));
        QB_CUDA(cudaMemsetAsync(b->ctl, 0, n * sizeof(int32_t), ctx->stream));
        int32_t *p = b->ctl;
        auto take = [&](size_t cnt) { int32_t *r = p; p += cnt; return r; };
        b->pos = take(n_seqs); b->sel = take(n_seqs); b->cur = take(n_seqs); b->zero_sel = take(n_seqs);
        b->drafts = take((size_t)n_seqs * std::max(1u, draft_k));
        b->tok_buf = take(rows); b->seqpos_buf = take(n_seqs); b->prefix_pos = take(n_seqs);
        b->prefix_tok = take((size_t)n_seqs * std::max(1u, draft_k));
        b->out_rec = take((size_t)n_seqs * (K1 + 2));
        b->map_prevh = take(n_seqs); b->map_prefix = take((size_t)n_seqs * K1); b->map_chunk = take(rows); b->map_last = take(n_seqs);
        b->limit = take(n_seqs);
        std::vector<int32_t> prevh(n_seqs), mp((size_t)n_seqs * std::max(1u, draft_k));
        for (uint32_t s = 0; s < n_seqs; ++s) prevh[s] = (int32_t)(rows + s);
        for (uint32_t s = 0; s < n_seqs; ++s)
            for (uint32_t i = 0; i < draft_k; ++i) mp[(size_t)s * draft_k + i] = (int32_t)(s * K1 + i);
        QB_CUDA(cudaMemcpyAsync(b->map_prevh, prevh.data(), n_seqs * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
        if (draft_k)
            QB_CUDA(cudaMemcpyAsync(b->map_prefix, mp.data(), mp.size() * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
        QB_CUDA(cudaStreamSynchronize(ctx->stream));
        QB_CUDA(cudaMalloc(&b->stats, QB_STATS * sizeof(long long)));
        QB_CUDA(cudaMemsetAsync(b->stats, 0, QB_STATS * sizeof(long long), ctx->stream));
        QB_CUDA(cudaHostAlloc(&b->out_rec_host, (size_t)n_seqs * (K1 + 2) * sizeof(int32_t), cudaHostAllocDefault));
        QB_CUDA(cudaHostAlloc(&b->limit_host, (size_t)n_seqs * sizeof(int32_t), cudaHostAllocDefault));
        for (uint32_t s = 0; s < n_seqs; ++s) b->limit_host[s] = (int32_t)draft_k;
        QB_CUDA(cudaMemcpyAsync(b->limit, b->limit_host, n_seqs * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
        QB_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    // activations
    const uint32_t inner = m->inner(), vdim = m->vdim(), F = c.n_ff, V = c.vocab_size;
    const uint32_t act_cols = std::max({m->attn_in(), m->dn_in(), 2 * F});
    QB_CUDA(cudaMalloc(&b->hid, (size_t)(rows + n_seqs) * H * sizeof(float)));
    QB_CUDA(cudaMemsetAsync(b->hid, 0, (size_t)(rows + n_seqs) * H * sizeof(float), ctx->stream));
    QB_CUDA(cudaMalloc(&b->mtp_h, (size_t)rows * H * sizeof(float)));
    QB_CUDA(cudaMalloc(&b->embd, (size_t)rows * H * sizeof(float)));
    QB_CUDA(cudaMalloc(&b->act, (size_t)rows * act_cols * sizeof(float)));
    QB_CUDA(cudaMalloc(&b->logits, (size_t)b->logit_rows * V * sizeof(float)));
    QB_CUDA(cudaMalloc(&b->am_val, (size_t)b->logit_rows * QB_ARGMAX_BLOCKS * sizeof(float)));
    QB_CUDA(cudaMalloc(&b->am_idx, (size_t)b->logit_rows * QB_ARGMAX_BLOCKS * sizeof(int32_t)));
    {
        size_t per_row = 0;   // floats of split partials any GEMM of the model can need per row
        auto consider = [&](uint32_t N, uint32_t K, bool always) {
            const uint32_t S = qb_ksplit(N, K);
            if (S > 1 || always) per_row = std::max(per_row, (size_t)S * N);
        };
        consider(m->attn_in(), H, true); consider(m->dn_in(), H, true); consider(2 * F, H, false); consider(V, H, false);
        consider(H, inner, true); consider(H, vdim, true); consider(H, F, true); consider(H, 2 * H, true);
        b->parts_floats = std::max<size_t>(per_row, 1) * rows;
        QB_CUDA(cudaMalloc(&b->parts, b->parts_floats * sizeof(float)));
    }
    {
        size_t ml = 0;
        const size_t acc = qb_attention_scratch_floats(rows, c.n_heads, c.head_dim, max_ctx + draft_k + 1, &ml, b->attn_split);
        QB_CUDA(cudaMalloc(&b->att_acc, acc * sizeof(float)));
        QB_CUDA(cudaMalloc(&b->att_ml, ml * sizeof(float)));
    }
    QB_TRY(alloc_qbuf(b->xq_h, rows, H));
    QB_TRY(alloc_qbuf(b->xq_attn, rows, inner));
    QB_TRY(alloc_qbuf(b->xq_dn, rows, vdim));
    QB_TRY(alloc_qbuf(b->xq_ffn, rows, F));
    QB_TRY(alloc_qbuf(b->xq_cat, rows, 2 * H));
    b->host_pos.assign(n_seqs, 0);
    b->chunk_end_pos.assign(n_seqs, -1);
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    *out = b;
    return QB_OK;
}

extern "C" int qb_batch_create(qb_ctx *ctx, qb_model *m, uint32_t n_seqs, uint32_t max_ctx, uint32_t draft_k,
                               uint32_t page_size, int page_order, qb_batch **out) {
    return batch_create(ctx, m, n_seqs, max_ctx, draft_k, page_size, page_order, 0, out);
}

// The pooled form: the K/V caches of every attention layer and of the MTP layer hold pool_pages pages in all (one pool,
// one page table per sequence shared by all layers: allocate_continuous_kv_cache / _mtp_kv_cache,
// src/qwen_native_backend.cpp:6603-6709), handed to sequences page by page as their positions grow.
extern "C" int qb_batch_create_pooled(qb_ctx *ctx, qb_model *m, uint32_t n_seqs, uint32_t max_ctx, uint32_t draft_k,
                                      uint32_t page_size, uint32_t pool_pages, qb_batch **out) {
    QB_REQUIRE(pool_pages > 0, "qb_batch_create_pooled: needs a pool size");
    return batch_create(ctx, m, n_seqs, max_ctx, draft_k, page_size, 0, pool_pages, out);
}

extern "C" void qb_batch_destroy(qb_ctx *ctx, qb_batch *b) {
    if (!b) return;
    cudaStreamSynchronize(ctx->stream);
    delete b->pool;
    for (auto p : b->kc) if (p) cudaFree(p);
    for (auto p : b->vc) if (p) cudaFree(p);
    for (auto p : b->state) if (p) cudaFree(p);
    for (auto p : b->conv) if (p) cudaFree(p);
    for (auto p : b->conv_alt) if (p) cudaFree(p);
    void *ptrs[] = {b->page_table, b->ctl, b->stats, b->hid, b->mtp_h, b->embd, b->act, b->parts,
                    b->logits, b->am_val, b->am_idx, b->att_acc, b->att_ml, b->xq_h.q, b->xq_h.d, b->xq_attn.q,
                    b->xq_attn.d, b->xq_dn.q, b->xq_dn.d, b->xq_ffn.q, b->xq_ffn.d, b->xq_cat.q, b->xq_cat.d, b->samp_u, b->seen, b->swap_tmp,
                    b->normed, b->tp_y};
    for (void *p : ptrs) if (p) cudaFree(p);
    if (b->out_rec_host) cudaFreeHost(b->out_rec_host);
    if (b->limit_host) cudaFreeHost(b->limit_host);
    if (b->tok_stage) cudaFreeHost(b->tok_stage);
    if (b->tok_all) cudaFree(b->tok_all);
    if (b->tok_ev) cudaEventDestroy(b->tok_ev);
    if (b->first_draw_stage) cudaFreeHost(b->first_draw_stage);
    if (b->samp_stage) cudaFreeHost(b->samp_stage);
    for (cudaEvent_t e : b->samp_ev) if (e) cudaEventDestroy(e);
    if (b->probe_host) cudaFreeHost(b->probe_host);
    if (b->probe_ev) cudaEventDestroy(b->probe_ev);
    delete b;
}

// ================================================================================================
// small control kernels
// ================================================================================================
namespace {

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// Argmax of a row from its per-block partial results, by one warp (all lanes return it): largest value, lowest
// index among equals (argmax_kernel src/kernels_cuda.cu:1765-1771).
__device__ int final_argmax(const float *pval, const int32_t *pidx, uint32_t row) {
    const uint32_t lane = threadIdx.x & 31;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (uint32_t j = lane; j < QB_ARGMAX_BLOCKS; j += 32) {
        const float v = pval[(size_t)row * QB_ARGMAX_BLOCKS + j];
        const int i = pidx[(size_t)row * QB_ARGMAX_BLOCKS + j];
        if (better(v, i, bv, bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, bv, o);
        const int i = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(v, i, bv, bi)) { bv = v; bi = i; }
    }
    return bi;
}

// tokens / positions of draft step i: token = i ? drafts[s][i-1] : cur[s], position = pos[s] + i
__global__ void prep_draft_kernel(const int32_t *cur, const int32_t *drafts, const int32_t *pos, uint32_t n_seqs, uint32_t k,
                                  uint32_t i, int32_t *tok, int32_t *seqpos) {
    QB_PDL_ENTER();
    const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_seqs) return;
    tok[s] = i == 0 ? cur[s] : drafts[(size_t)s * k + i - 1];
    seqpos[s] = pos[s] + (int)i;
}

// one warp per sequence
__global__ void store_draft_kernel(const float *pval, const int32_t *pidx, uint32_t n_seqs, uint32_t k, uint32_t i, int32_t *drafts) {
    QB_PDL_ENTER();
    const uint32_t s = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (s >= n_seqs) return;
    const int tok = final_argmax(pval, pidx, s);
    if ((threadIdx.x & 31) == 0) drafts[(size_t)s * k + i] = tok;
}

__global__ void prep_verify_kernel(const int32_t *cur, const int32_t *drafts, uint32_t n_seqs, uint32_t k, int32_t *tok) {
    QB_PDL_ENTER();
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_seqs * (k + 1)) return;
    const uint32_t s = idx / (k + 1), j = idx % (k + 1);
    tok[idx] = j == 0 ? cur[s] : drafts[(size_t)s * k + j - 1];
}

// Forced drafts: draft i of sequence s is the caller's guess for absolute position pos+1+i.
__global__ void force_drafts_kernel(int32_t *drafts, const int32_t *pos, uint32_t n_seqs, uint32_t k, const int32_t *forced,
                                    uint32_t stride) {
    QB_PDL_ENTER();
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_seqs * k) return;
    const uint32_t s = idx / k, i = idx % k;
    const uint32_t p = (uint32_t)pos[s] + 1 + i;
    drafts[idx] = p < stride ? forced[(size_t)s * stride + p] : 0;
}

// Greedy acceptance + commit, one CTA per sequence (src/qwen_native_backend.cpp:15948-16154,
// src/qwen_executor.cpp:22304-22428): accepted = longest prefix with argmax(row i) == draft i+1;
// emit the accepted drafts and argmax(row accepted); select checkpoint slot `accepted`; advance the
// position; keep the hidden row `accepted` as the next step's MTP input.
__global__ void accept_commit_kernel(const float *pval, const int32_t *pidx, uint32_t k, uint32_t rows_cap, uint32_t H,
                                     int32_t *pos, int32_t *sel, int32_t *cur, const int32_t *drafts, int32_t *prefix_pos,
                                     int32_t *prefix_tok, int32_t *out_rec, uint32_t n_seqs, float *hid,
                                     unsigned long long *stats, const int32_t *limit, int32_t eos) {
    QB_PDL_ENTER();
    __shared__ int s_acc;
    __shared__ int am[8];
    const uint32_t s = blockIdx.x;
    const uint32_t K1 = k + 1;
    if (threadIdx.x / 32 < K1) {                                    // warp r takes verify row r
        const int t = final_argmax(pval, pidx, s * K1 + threadIdx.x / 32);
        if ((threadIdx.x & 31) == 0) am[threadIdx.x / 32] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // chain length of this step: the caller's depth limit (min(k, tokens still wanted), MtpAdaptivePolicy::draft_limit,
        // src/qwen_native_backend.cpp:1625-1628) cut before the first draft equal to the end-of-sequence token
        // (:15817-15821); a chain of length 0 is one plain step (:15829-15848)
        uint32_t kk = min(k, (uint32_t)max(limit[s], 0));
        if (eos >= 0)
            for (uint32_t i = 0; i < kk; ++i)
                if (drafts[(size_t)s * k + i] == eos) { kk = i; break; }
        uint32_t a = 0;
        while (a < kk && am[a] == drafts[(size_t)s * k + a]) ++a;
        int32_t *n_out = out_rec, *toks = out_rec + n_seqs, *opos = out_rec + n_seqs + (size_t)n_seqs * K1;
        for (uint32_t i = 0; i < a; ++i) toks[(size_t)s * K1 + i] = drafts[(size_t)s * k + i];
        toks[(size_t)s * K1 + a] = am[a];
        n_out[s] = (int)a + 1;
        const int old = pos[s];
        prefix_pos[s] = old + 1;
        for (uint32_t i = 0; i < k; ++i) prefix_tok[(size_t)s * k + i] = drafts[(size_t)s * k + i];
        pos[s] = old + (int)a + 1;
        opos[s] = pos[s];
        sel[s] = (int)a;
        cur[s] = am[a];
        s_acc = (int)a;
        atomicAdd(&stats[0], 1ull);
        atomicAdd(&stats[1], (unsigned long long)kk);
        atomicAdd(&stats[2], (unsigned long long)a);
        atomicAdd(&stats[3], (unsigned long long)(a + 1));
        if (a < kk) atomicAdd(&stats[4], 1ull);                      // a step that rejected a draft (mtp_spec_rejected)
        atomicAdd(&stats[8 + min(a, 7u)], 1ull);                     // mtp_accept_len_hist
    }
    __syncthreads();
    const uint32_t a = (uint32_t)s_acc;
    const float *src = hid + (size_t)(s * K1 + a) * H;
    float *dst = hid + (size_t)(rows_cap + s) * H;
    for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
}

// Greedy step / end of prefill: next token = argmax of the row; position advances by `adv`.
__global__ void greedy_commit_kernel(const float *pval, const int32_t *pidx, uint32_t logit_row0, uint32_t hid_row0,
                                     uint32_t hid_row_stride, uint32_t seq0, uint32_t n, uint32_t K1, uint32_t rows_cap, uint32_t H,
                                     int32_t *pos, int32_t *sel, int32_t *cur, int32_t adv, int32_t *out_rec, uint32_t n_seqs,
                                     float *hid, unsigned long long *stats) {
    QB_PDL_ENTER();
    const uint32_t j = blockIdx.x, s = seq0 + j;
    if (j >= n) return;
    int tok = 0;
    if (threadIdx.x < 32) tok = final_argmax(pval, pidx, logit_row0 + j);
    if (threadIdx.x == 0) {
        int32_t *n_out = out_rec, *toks = out_rec + n_seqs, *opos = out_rec + n_seqs + (size_t)n_seqs * K1;
        toks[(size_t)s * K1] = tok;
        n_out[s] = 1;
        pos[s] += adv;
        opos[s] = pos[s];
        sel[s] = 0;
        cur[s] = tok;
        atomicAdd(&stats[3], 1ull);
    }
    const float *src = hid + (size_t)(hid_row0 + j * hid_row_stride) * H;
    float *dst = hid + (size_t)(rows_cap + s) * H;
    for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
}

// Token-penalty bookkeeping (the `seen` map of the reference's generate loops, src/qwen_native_backend.cpp:15396, 15712):
// bits of the prompt tokens of a chunk, and of the tokens the last commit emitted.
__global__ void mark_seen_tokens_kernel(const int32_t *toks, uint32_t n, uint32_t *seen_row, uint32_t V) {
    QB_PDL_ENTER();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && (uint32_t)toks[i] < V) atomicOr(seen_row + ((uint32_t)toks[i] >> 5), 1u << (toks[i] & 31));
}
__global__ void mark_seen_record_kernel(const int32_t *out_rec, uint32_t n_seqs, uint32_t K1, uint32_t seq0, uint32_t ns, uint32_t *seen,
                                        uint32_t words, uint32_t V) {
    QB_PDL_ENTER();
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= ns * K1) return;
    const uint32_t s = seq0 + idx / K1, i = idx % K1;
    const int32_t *n_out = out_rec, *toks = out_rec + n_seqs;
    if ((int)i < n_out[s]) {
        const uint32_t t = (uint32_t)toks[(size_t)s * K1 + i];
        if (t < V) atomicOr(seen + (size_t)s * words + (t >> 5), 1u << (t & 31));
    }
}

__global__ void swap_ctl_kernel(int32_t *pos, int32_t *sel, int32_t *cur, int32_t *prefix_pos, int32_t *out_rec, int32_t *limit, uint32_t n_seqs,
                                uint32_t K1, uint32_t a, uint32_t b) {
    QB_PDL_ENTER();
    if (threadIdx.x == 0) {
        int32_t *n_out = out_rec, *toks = out_rec + n_seqs, *opos = out_rec + n_seqs + (size_t)n_seqs * K1;
        int32_t *arr[7] = {pos, sel, cur, prefix_pos, n_out, opos, limit};      // the step record follows its sequence
        for (int i = 0; i < 7; ++i) { const int32_t t = arr[i][a]; arr[i][a] = arr[i][b]; arr[i][b] = t; }
        for (uint32_t i = 0; i < K1; ++i) { const int32_t t = toks[(size_t)a * K1 + i]; toks[(size_t)a * K1 + i] = toks[(size_t)b * K1 + i]; toks[(size_t)b * K1 + i] = t; }
    }
}

// map[0] = the row that holds the previous chunk's last hidden, map[r] = r - 1 (prefill: hidden row feeding MTP row r)
__global__ void chunk_map_kernel(int32_t *map, uint32_t M, int32_t prev_row) {
    QB_PDL_ENTER();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < M) map[r] = r == 0 ? prev_row : (int32_t)r - 1;
}

// (every kernel that moves pos[s] also writes the position field of the sequence's step record: the host refreshes its
// position bound of ALL sequences from those fields, also of sequences that took no part in the last step)
__global__ void advance_kernel(int32_t *pos, int32_t *sel, uint32_t s, int32_t adv, uint32_t rows_cap, uint32_t H, uint32_t last_row, float *hid,
                               int32_t *opos) {
    QB_PDL_ENTER();
    if (threadIdx.x == 0) { pos[s] += adv; sel[s] = 0; opos[s] = pos[s]; }
    const float *src = hid + (size_t)last_row * H;
    float *dst = hid + (size_t)(rows_cap + s) * H;
    for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
}

}  // namespace

// ================================================================================================
// forward passes
// ================================================================================================

// y[rows][N] = W x, written to dst (row stride N).
static int gemm_to(qb_ctx *ctx, qb_batch *b, const qb_weight *w, const QBuf &x, uint32_t rows, float *dst, uint32_t S_override = 0) {
    const uint32_t S = S_override ? S_override : qb_ksplit(w->rows, w->cols);
    if (S == 1) return qb_launch_gemm(ctx, w, x.q, x.d, rows, dst, 1, b->gemm_impl);
    QB_REQUIRE((size_t)S * rows * w->rows <= b->parts_floats, "split scratch too small");
    QB_TRY(qb_launch_gemm(ctx, w, x.q, x.d, rows, b->parts, S, b->gemm_impl));
    return qb_launch_reduce_parts(ctx, b->parts, S, rows, w->rows, dst, w->rows);
}

// parts = split partials of W x (left in b->parts); returns S.
static int gemm_parts(qb_ctx *ctx, qb_batch *b, const qb_weight *w, const QBuf &x, uint32_t rows, uint32_t *S_out) {
    const uint32_t S = qb_ksplit(w->rows, w->cols);
    QB_REQUIRE((size_t)S * rows * w->rows <= b->parts_floats || S == 1, "split scratch too small");
    QB_REQUIRE((size_t)rows * w->rows <= b->parts_floats, "split scratch too small");
    *S_out = S;
    return qb_launch_gemm(ctx, w, x.q, x.d, rows, b->parts, S, b->gemm_impl);
}

// h += parts ; xq = quant(rmsnorm(h) * w)
static int residual_norm_quant(qb_ctx *ctx, qb_batch *b, float *h, uint32_t rows, uint32_t S, const float *norm_w, const QBuf &dst,
                               uint32_t q_col_off = 0, bool add_x = true, const float *parts = nullptr, float *normed_out = nullptr) {
    const qb_model_config &c = b->m->cfg;
    NormQuantArgs a;
    a.x = add_x ? h : nullptr; a.x_stride = c.n_embd;
    a.parts = parts ? parts : b->parts; a.S = S; a.part_ld = c.n_embd;
    a.normed_out = normed_out;
    a.h_out = h; a.h_stride = c.n_embd;
    a.w = norm_w; a.eps = c.rms_eps; a.n = c.n_embd; a.M = rows;
    a.q = dst.q; a.q_pitch = dst.K; a.q_col_off = q_col_off; a.d = dst.d; a.d_ld = qb_act_ld(rows); a.d_kb_off = q_col_off / 32;
    return qb_launch_norm_quant(ctx, a);
}

static int plain_norm_quant(qb_ctx *ctx, qb_batch *b, const float *x, const int32_t *row_map, uint32_t rows, const float *norm_w,
                            const QBuf &dst, uint32_t q_col_off = 0) {
    const qb_model_config &c = b->m->cfg;
    NormQuantArgs a;
    a.x = x; a.x_stride = c.n_embd; a.row_map = row_map;
    a.w = norm_w; a.eps = c.rms_eps; a.n = c.n_embd; a.M = rows;
    a.q = dst.q; a.q_pitch = dst.K; a.q_col_off = q_col_off; a.d = dst.d; a.d_ld = qb_act_ld(rows); a.d_kb_off = q_col_off / 32;
    return qb_launch_norm_quant(ctx, a);
}

struct RowSet {
    uint32_t seq0 = 0, ns = 0, R = 0;      // sequences [seq0, seq0+ns), R rows each
    const int32_t *seq_pos = nullptr;      // device [ns]: position of each sequence's first row
    uint32_t max_pos = 0;                  // host upper bound of any row position
    bool ingest = false;                   // rows of a prompt chunk (not of a decode / verify step)
    uint32_t rows() const { return ns * R; }
};

// One attention block on h (xq_h already holds quant(rmsnorm(h))).  kv_only: K/V append only.
static int attention_block(qb_ctx *ctx, qb_batch *b, const LayerW &L, uint32_t cache_idx, float *h, const RowSet &rs, bool kv_only,
                           const float *next_norm_w) {
    qb_model *m = b->m;
    const qb_model_config &c = m->cfg;
    const uint32_t rows = rs.rows();
    AttnArgs a;
    a.rows = rows; a.n_heads = c.n_heads; a.n_kv = c.n_kv_heads; a.hd = c.head_dim; a.rope_dim = c.rope_dim; a.eps = c.rms_eps;
    a.q_norm_w = L.q_norm; a.k_norm_w = L.k_norm; a.inv_freq = m->inv_freq;
    a.page_table = b->page_table + (size_t)rs.seq0 * b->pages_per_seq; a.pt_stride = b->pages_per_seq; a.page_size = b->page_size;
    a.err_flag = ctx->err_flag_dev;
    a.ingest = rs.ingest;
    a.prefer_tc = b->attn_tc;
    a.split_keys = b->attn_split;
    a.k_cache = b->kc[cache_idx]; a.v_cache = b->vc[cache_idx];
    a.max_pos = rs.max_pos; a.part_acc = b->att_acc; a.part_ml = b->att_ml; a.kv_only = kv_only;
    if (kv_only) {
        // only the k and v rows of the fused projection, with the split count of the fused weight so the
        // values are bit-identical to the full projection; compact [k | v] rows, no q heads
        const uint32_t S = qb_ksplit(L.w_in->rows, L.w_in->cols);
        QB_TRY(gemm_to(ctx, b, &L.w_kv, b->xq_h, rows, b->act, S));
        a.qkv = b->act; a.row_stride = 2 * m->kvd(); a.n_heads = 0;
        return qb_attn_prepare(ctx, a, rs.seq_pos, rs.ns);
    }
    // the consumers of the fused projection add its split partials themselves
    uint32_t S_in = 1;
    QB_TRY(gemm_parts(ctx, b, L.w_in, b->xq_h, rows, &S_in));
    a.qkv = b->parts; a.row_stride = m->attn_in(); a.in_S = S_in; a.in_pstride = (size_t)rows * m->attn_in();
    QB_TRY(qb_attn_prepare(ctx, a, rs.seq_pos, rs.ns));
    QB_TRY(qb_attn_run(ctx, a, rs.seq_pos, rs.ns, nullptr, b->xq_attn.q, b->xq_attn.K, b->xq_attn.d, qb_act_ld(rows)));
    uint32_t S = 1;
    QB_TRY(gemm_parts(ctx, b, L.w_out, b->xq_attn, rows, &S));
    return residual_norm_quant(ctx, b, h, rows, S, next_norm_w, b->xq_h, 0, true, nullptr, b->tp ? b->normed : nullptr);
}

static int ffn_block(qb_ctx *ctx, qb_batch *b, const LayerW &L, float *h, uint32_t rows, const float *next_norm_w) {
    const qb_model_config &c = b->m->cfg;
    if (b->tp) {
        // tensor-parallel form: this rank's shard of gate/up and down on the fp32 normalised rows, the all-reduce fused
        // into the down GEMM; every rank gets the same [rows][H] sum, added to the residual stream like one K segment
        QB_TRY(qb_tp_ffn(ctx, b->tp, L.w_gate_up, L.w_down, b->normed, rows, b->tp_y, c.n_embd));
        return residual_norm_quant(ctx, b, h, rows, 1, next_norm_w, b->xq_h, 0, true, b->tp_y);
    }
    QB_TRY(qb_ffn_gate_up_swiglu(ctx, L.w_gate_up, b->xq_h.q, b->xq_h.d, rows, b->act, b->parts, b->parts_floats, b->xq_ffn.q, b->xq_ffn.K,
                                 b->xq_ffn.d, qb_act_ld(rows), b->gemm_impl, 0));
    uint32_t S = 1;
    QB_TRY(gemm_parts(ctx, b, L.w_down, b->xq_ffn, rows, &S));
    return residual_norm_quant(ctx, b, h, rows, S, next_norm_w, b->xq_h);
}

static int deltanet_block(qb_ctx *ctx, qb_batch *b, const LayerW &L, uint32_t il, float *h, const RowSet &rs, bool checkpoints,
                          const float *next_norm_w) {
    qb_model *m = b->m;
    const qb_model_config &c = m->cfg;
    const uint32_t rows = rs.rows(), K1 = b->k + 1;
    uint32_t S_in = 1;
    QB_TRY(gemm_parts(ctx, b, L.w_in, b->xq_h, rows, &S_in));
    DnArgs d;
    d.proj = b->parts; d.proj_stride = m->dn_in(); d.proj_S = S_in; d.proj_pstride = (size_t)rows * m->dn_in();
    d.n_seqs = rs.ns; d.rows_per_seq = rs.R;
    d.conv_w = L.conv_w; d.ssm_a = L.ssm_a; d.dt_bias = L.dt_bias; d.norm_w = L.ssm_norm;
    d.nk = c.ssm_num_k_heads; d.nv = c.ssm_num_v_heads; d.hd = c.ssm_head_dim; d.eps = c.rms_eps;
    d.state = b->state[il] + (size_t)rs.seq0 * K1 * c.ssm_num_v_heads * c.ssm_head_dim * c.ssm_head_dim;
    const size_t conv_off = (size_t)rs.seq0 * K1 * m->qkv_dim() * 3;
    d.conv = (b->conv_par ? b->conv_alt[il] : b->conv[il]) + conv_off;
    d.conv_out = (b->conv_par ? b->conv[il] : b->conv_alt[il]) + conv_off;
    d.n_slots = K1; d.slot_in = b->sel + rs.seq0; d.write_all = checkpoints ? 1 : 0;
    d.q8 = b->xq_dn.q; d.q_pitch = b->xq_dn.K; d.d = b->xq_dn.d; d.d_ld = qb_act_ld(rows);
    QB_TRY(qb_launch_deltanet(ctx, d));
    uint32_t S = 1;
    QB_TRY(gemm_parts(ctx, b, L.w_out, b->xq_dn, rows, &S));
    return residual_norm_quant(ctx, b, h, rows, S, next_norm_w, b->xq_h, 0, true, nullptr, b->tp ? b->normed : nullptr);
}

// Target model on a row set.  tokens on the device ([rows]).  Leaves the pre-output-norm hidden rows
// in b->hid[0 .. rows).  logits: 0 none, 1 every row, 2 last row of each sequence.
static int target_forward(qb_ctx *ctx, qb_batch *b, const int32_t *tokens_dev, const RowSet &rs, bool checkpoints, int logits) {
    qb_model *m = b->m;
    const qb_model_config &c = m->cfg;
    const uint32_t rows = rs.rows();
    QB_REQUIRE(rows <= b->rows_cap, "forward: %u rows exceed capacity %u", rows, b->rows_cap);
    float *h = b->hid;
    QB_TRY(qb_launch_get_rows(ctx, m->token_embd, tokens_dev, rows, h, c.n_embd));
    QB_TRY(plain_norm_quant(ctx, b, h, nullptr, rows, m->layers[0].attn_norm, b->xq_h));
    for (uint32_t il = 0; il < c.n_layers; ++il) {
        const LayerW &L = m->layers[il];
        if (L.recurrent) QB_TRY(deltanet_block(ctx, b, L, il, h, rs, checkpoints, L.ffn_norm));
        else QB_TRY(attention_block(ctx, b, L, il, h, rs, false, L.ffn_norm));
        // the norm fused behind the FFN is the next layer's attn_norm, or output_norm after the last layer
        QB_TRY(ffn_block(ctx, b, L, h, rows, il + 1 < c.n_layers ? m->layers[il + 1].attn_norm : m->output_norm));
    }
    // the DeltaNet layers read the conv windows from one buffer and wrote the new ones to the other: a forward over
    // every sequence just swaps the two; one over a subset copies its windows back so all sequences stay in one
    if (rs.seq0 == 0 && rs.ns == b->n_seqs) {
        b->conv_par ^= 1;
    } else {
        const size_t per_seq = (size_t)(b->k + 1) * m->qkv_dim() * 3;
        for (uint32_t il = 0; il < c.n_layers; ++il) {
            if (!m->layers[il].recurrent) continue;
            float *rd = b->conv_par ? b->conv_alt[il] : b->conv[il], *wr = b->conv_par ? b->conv[il] : b->conv_alt[il];
            QB_CUDA(cudaMemcpyAsync(rd + rs.seq0 * per_seq, wr + rs.seq0 * per_seq, rs.ns * per_seq * sizeof(float),
                                    cudaMemcpyDeviceToDevice, ctx->stream));
        }
    }
    b->last_logit_rows = 0;
    if (logits == 1) {
        QB_REQUIRE(rows <= b->logit_rows, "logits for %u rows exceed capacity %u", rows, b->logit_rows);
        QB_TRY(gemm_to(ctx, b, m->output, b->xq_h, rows, b->logits));
        QB_TRY(qb_launch_argmax_partial(ctx, b->logits, rows, c.vocab_size, c.vocab_size, b->am_val, b->am_idx, QB_ARGMAX_BLOCKS));
        b->last_logit_rows = rows;
    } else if (logits == 2) {
        // last row of each sequence: quantise those rows again as a compact batch
        std::vector<int32_t> map(rs.ns);
        for (uint32_t s = 0; s < rs.ns; ++s) map[s] = (int32_t)(s * rs.R + rs.R - 1);
        QB_CUDA(cudaMemcpyAsync(b->map_last, map.data(), rs.ns * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
        QB_TRY(plain_norm_quant(ctx, b, h, b->map_last, rs.ns, m->output_norm, b->xq_h));
        QB_TRY(gemm_to(ctx, b, m->output, b->xq_h, rs.ns, b->logits));
        QB_TRY(qb_launch_argmax_partial(ctx, b->logits, rs.ns, c.vocab_size, c.vocab_size, b->am_val, b->am_idx, QB_ARGMAX_BLOCKS));
        b->last_logit_rows = rs.ns;
    }
    return QB_OK;
}

// MTP head on a row set (forward_mtp_draft_from, src/qwen_executor.cpp:7025-7255).  Row r uses token
// tokens_dev[r] and the hidden row hsrc[hmap[r]] as h_prev.  kv_only stops after the K/V append.
// Full mode leaves the post-layer hidden in b->mtp_h and the argmax partials of the logits.
static int mtp_forward(qb_ctx *ctx, qb_batch *b, const int32_t *tokens_dev, const float *hsrc, const int32_t *hmap, const RowSet &rs,
                       bool kv_only) {
    qb_model *m = b->m;
    const qb_model_config &c = m->cfg;
    const uint32_t rows = rs.rows(), H = c.n_embd;
    const LayerW &L = m->layers[c.n_layers];
    QB_TRY(qb_launch_get_rows(ctx, m->mtp_embd, tokens_dev, rows, b->embd, H));
    QB_TRY(plain_norm_quant(ctx, b, b->embd, nullptr, rows, m->enorm, b->xq_cat, 0));     // enorm
    QB_TRY(plain_norm_quant(ctx, b, hsrc, hmap, rows, m->hnorm, b->xq_cat, H));            // hnorm
    uint32_t S = 1;
    QB_TRY(gemm_parts(ctx, b, m->eh_proj, b->xq_cat, rows, &S));
    QB_TRY(residual_norm_quant(ctx, b, b->mtp_h, rows, S, L.attn_norm, b->xq_h, 0, /*add_x=*/false));
    QB_TRY(attention_block(ctx, b, L, c.n_layers, b->mtp_h, rs, kv_only, L.ffn_norm));
    if (kv_only) return QB_OK;
    QB_TRY(ffn_block(ctx, b, L, b->mtp_h, rows, m->shared_head_norm));
    QB_REQUIRE(rows <= b->logit_rows, "MTP logits rows exceed capacity");
    QB_TRY(gemm_to(ctx, b, m->mtp_head, b->xq_h, rows, b->logits));
    QB_TRY(qb_launch_argmax_partial(ctx, b->logits, rows, c.vocab_size, c.vocab_size, b->am_val, b->am_idx, QB_ARGMAX_BLOCKS));
    b->last_logit_rows = rows;
    return QB_OK;
}

static uint32_t max_host_pos(const qb_batch *b) {
    int32_t mx = 0;
    for (uint32_t s = 0; s < b->n_active; ++s) mx = std::max(mx, b->host_pos[s]);
    return (uint32_t)mx;
}
static void advance_host_pos(qb_batch *b, int32_t by) {
    for (uint32_t s = 0; s < b->n_active; ++s) b->host_pos[s] += by;
    b->probe_adv += by;
}
// host_pos is an upper bound: a speculative step advances it by k + 1 although the device commits 1 .. k + 1 positions.
// A caller that reads the step records gets the exact positions back (qb_read_step_output); for one that does not, every
// PROBE_EVERY steps the device positions are copied to pinned memory behind the step, and once that copy has landed
// (cudaEventQuery: never a wait) the bound becomes copied position + positions enqueued since.  Anything else that
// rewrites host_pos (prefill, reset, swap, restore, a change of the active count) drops a probe in flight.
static constexpr uint32_t PROBE_EVERY = 8;
static void probe_cancel(qb_batch *b) { b->probe_pending = false; b->steps_since_probe = 0; }
static int probe_tick(qb_ctx *ctx, qb_batch *b) {
    if (b->probe_pending) {
        if (cudaEventQuery(b->probe_ev) == cudaSuccess) {
            for (uint32_t s = 0; s < b->n_active; ++s) b->host_pos[s] = std::min(b->host_pos[s], b->probe_host[s] + b->probe_adv);
            probe_cancel(b);
        }
        return QB_OK;
    }
    if (++b->steps_since_probe < PROBE_EVERY) return QB_OK;
    if (!b->probe_host) {
        QB_CUDA(cudaHostAlloc(&b->probe_host, (size_t)b->n_seqs * sizeof(int32_t), cudaHostAllocDefault));
        QB_CUDA(cudaEventCreateWithFlags(&b->probe_ev, cudaEventDisableTiming));
    }
    QB_CUDA(cudaMemcpyAsync(b->probe_host, b->pos, (size_t)b->n_active * sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    QB_CUDA(cudaEventRecord(b->probe_ev, ctx->stream));
    b->probe_pending = true;
    b->probe_adv = 0;
    return QB_OK;
}

static int mark_seen_record(qb_ctx *ctx, qb_batch *b, uint32_t seq0, uint32_t ns) {
    if (!b->seen) return QB_OK;
    const uint32_t K1 = b->k + 1;
    QB_CUDA(qb_launch_pdl(ctx->stream, mark_seen_record_kernel, dim3((ns * K1 + 127) / 128), dim3(128), (size_t)0, b->out_rec, b->n_seqs, K1, seq0, ns,
                          b->seen, b->seen_words, b->m->cfg.vocab_size));
    QB_LAUNCHED(ctx, "mark_seen_record_kernel");
    return QB_OK;
}

// Token penalties of sampling requests (presence_penalty / repetition_penalty of the reference's sampler): from this call on
// the batch records the prompt and emitted tokens of every sequence, and qb_mtp_sample_rows penalises their logits.  Call
// before the prefill of the requests it should cover.  presence = 0 and repetition = 1 switch the penalties off again.
extern "C" int qb_batch_set_penalties(qb_ctx *ctx, qb_batch *b, float presence, float repetition) {
    QB_REQUIRE(ctx && b, "qb_batch_set_penalties: null argument");
    QB_CUDA(cudaSetDevice(ctx->device));
    if (!b->seen) {
        b->seen_words = (b->m->cfg.vocab_size + 31) / 32;
        QB_CUDA(cudaMalloc(&b->seen, (size_t)b->n_seqs * b->seen_words * sizeof(uint32_t)));
        QB_CUDA(cudaMemsetAsync(b->seen, 0, (size_t)b->n_seqs * b->seen_words * sizeof(uint32_t), ctx->stream));
    }
    b->pen_presence = presence;
    b->pen_repetition = repetition;
    return QB_OK;
}

// Prompt ingestion of one sequence in chunks.  more_follows: the prompt continues in a later call, so the last row needs
// no logits, no token is committed, nothing is counted as emitted or seen beyond the prompt tokens themselves.  samp
// (temp > 0): the first token is drawn from the last row (pick_from_last_logits, src/qwen_native_backend.cpp:15399-15428:
// penalties against the prompt, then sample_token with the request's first draw) instead of its argmax.
// ---- pooled page tables ------------------------------------------------------------------------------------------
// New entries of one page-table row, passed by value (no staging buffer to keep alive).
struct PageRun { int32_t p[16]; };
__global__ void set_pages_kernel(int32_t *row, uint32_t first, uint32_t n, PageRun run) {
    QB_PDL_ENTER();
    if (threadIdx.x < n) row[first + threadIdx.x] = run.p[threadIdx.x];
}
static int upload_pages(qb_ctx *ctx, qb_batch *b, uint32_t seq, uint32_t first, uint32_t n) {
    const std::vector<int32_t> &pg = b->seq_pages[seq];
    for (uint32_t off = 0; off < n; off += 16) {
        PageRun run;
        const uint32_t m = std::min(16u, n - off);
        for (uint32_t i = 0; i < 16; ++i) run.p[i] = i < m ? pg[first + off + i] : -1;
        QB_CUDA(qb_launch_pdl(ctx->stream, set_pages_kernel, dim3(1), dim3(32), (size_t)0, b->page_table + (size_t)seq * b->pages_per_seq,
                              first + off, m, run));
        QB_LAUNCHED(ctx, "set_pages_kernel");
    }
    return QB_OK;
}
// Pages for positions [0, upto) of a sequence (pooled form; nothing to do otherwise).  Allocation follows the host's
// position bound, which is never below the device's position, so a page is there before a row is appended to it; the
// pool hands out its most recently freed page first.  An exhausted pool is reported before anything is launched.
static int ensure_pages(qb_ctx *ctx, qb_batch *b, uint32_t seq, uint32_t upto) {
    if (!b->pool) return QB_OK;
    std::vector<int32_t> &pg = b->seq_pages[seq];
    const uint32_t need = std::min(b->pages_per_seq, (upto + b->page_size - 1) / b->page_size);
    if (pg.size() >= need) return QB_OK;
    const uint32_t first = (uint32_t)pg.size();
    if (b->pool->free_count() < need - first)
        return qb_fail(QB_ERR_CAPACITY, "K/V page pool exhausted: sequence %u needs %u more pages, %u of %u free", seq, need - first,
                       b->pool->free_count(), b->pool->total());
    while (pg.size() < need) pg.push_back(b->pool->alloc());
    return upload_pages(ctx, b, seq, first, need - first);
}
static int ensure_step_pages(qb_ctx *ctx, qb_batch *b, uint32_t extra) {
    if (!b->pool) return QB_OK;
    for (uint32_t s = 0; s < b->n_active; ++s) QB_TRY(ensure_pages(ctx, b, s, (uint32_t)b->host_pos[s] + extra));
    return QB_OK;
}
static void release_pages(qb_batch *b, uint32_t seq) {
    if (!b->pool) return;
    // last allocated first, so that the pool's next page is this sequence's first one again
    for (auto it = b->seq_pages[seq].rbegin(); it != b->seq_pages[seq].rend(); ++it) b->pool->drop(*it);
    b->seq_pages[seq].clear();
}

extern "C" int qb_batch_pool_info(qb_ctx *ctx, qb_batch *b, uint32_t *free_pages, uint32_t *total_pages, uint32_t *page_size) {
    QB_REQUIRE(ctx && b, "qb_batch_pool_info: null argument");
    QB_REQUIRE(b->pool, "qb_batch_pool_info: the batch has no page pool (qb_batch_create_pooled)");
    if (free_pages) *free_pages = b->pool->free_count();
    if (total_pages) *total_pages = b->pool->total();
    if (page_size) *page_size = b->page_size;
    return QB_OK;
}
// The pages a sequence holds, in position order (pooled form).
extern "C" int qb_seq_pages(qb_ctx *ctx, qb_batch *b, uint32_t seq, int32_t *pages_out, uint32_t cap, uint32_t *n_out) {
    QB_REQUIRE(ctx && b && seq < b->n_seqs && n_out, "qb_seq_pages: bad arguments");
    QB_REQUIRE(b->pool, "qb_seq_pages: the batch has no page pool (qb_batch_create_pooled)");
    const std::vector<int32_t> &pg = b->seq_pages[seq];
    *n_out = (uint32_t)pg.size();
    for (uint32_t i = 0; i < pg.size() && i < cap && pages_out; ++i) pages_out[i] = pg[i];
    return QB_OK;
}

// ---- shared prompt prefixes (the prefix cache of the reference's server, src/qwen_native_backend.cpp:9785-10410:
// seed_from_shared_prefix on a hit, pages pinned while an entry lives) -------------------------------------------------
// An entry is taken from a sequence that has ingested a prefix with qb_prefill_chunk and nothing since: it holds the K/V
// pages of the prefix once more (target layers and MTP layer share the page ids), and copies of what is not paged: every
// DeltaNet layer's state and conv window at the prefix end, the last hidden row (the MTP pass of the next chunk pairs its
// first token with it), the prefix's tokens (seen-token record).  Attaching it to an empty sequence makes that sequence
// continue from the prefix end without ingesting it: same pages, copied state.  The prefix length must be a whole number
// of pages, so the sequences' own tokens go to pages of their own.
struct qb_prefix {
    qb_batch *owner = nullptr;
    uint32_t n_tokens = 0;
    std::vector<int32_t> pages;
    std::vector<float *> state, conv;     // per layer (recurrent layers only)
    float *hid = nullptr;
    int32_t *tokens_dev = nullptr;
};
__global__ void set_seq_ctl_kernel(int32_t *pos, int32_t *sel, int32_t *cur, int32_t *opos, uint32_t s, int32_t p) {
    QB_PDL_ENTER();
    if (threadIdx.x == 0) { pos[s] = p; sel[s] = 0; cur[s] = 0; opos[s] = p; }
}

extern "C" void qb_prefix_release(qb_ctx *ctx, qb_prefix *px) {
    if (!px) return;
    cudaStreamSynchronize(ctx->stream);
    for (auto it = px->pages.rbegin(); it != px->pages.rend(); ++it) px->owner->pool->drop(*it);
    for (float *p : px->state) if (p) cudaFree(p);
    for (float *p : px->conv) if (p) cudaFree(p);
    if (px->hid) cudaFree(px->hid);
    if (px->tokens_dev) cudaFree(px->tokens_dev);
    delete px;
}

extern "C" int qb_prefix_capture(qb_ctx *ctx, qb_batch *b, uint32_t seq, const int32_t *tokens_host, uint32_t n_tokens, qb_prefix **out) {
    QB_REQUIRE(ctx && b && out && seq < b->n_seqs, "qb_prefix_capture: bad arguments");
    QB_REQUIRE(b->pool, "qb_prefix_capture: the batch has no page pool (qb_batch_create_pooled)");
    const int32_t n = b->host_pos[seq];
    QB_REQUIRE(n > 0 && b->chunk_end_pos[seq] == n, "qb_prefix_capture: sequence %u is not at the end of a qb_prefill_chunk", seq);
    QB_REQUIRE((uint32_t)n % b->page_size == 0, "qb_prefix_capture: a prefix of %d tokens is not a whole number of %u-token pages", n, b->page_size);
    QB_REQUIRE(!tokens_host || n_tokens == (uint32_t)n, "qb_prefix_capture: %u tokens given for a prefix of %d", n_tokens, n);
    QB_REQUIRE(tokens_host || !b->seen, "qb_prefix_capture: a batch with token penalties needs the prefix's tokens");
    QB_CUDA(cudaSetDevice(ctx->device));
    const qb_model_config &c = b->m->cfg;
    const uint32_t K1 = b->k + 1;
    const size_t sfl = (size_t)c.ssm_num_v_heads * c.ssm_head_dim * c.ssm_head_dim, cfl = (size_t)b->m->qkv_dim() * 3;
    qb_prefix *px = new qb_prefix();
    px->owner = b; px->n_tokens = (uint32_t)n;
    px->state.assign(c.n_layers, nullptr); px->conv.assign(c.n_layers, nullptr);
    auto fail = [&](int st) { qb_prefix_release(ctx, px); return st; };
    for (uint32_t il = 0; il < c.n_layers; ++il) {
        if (!b->state[il]) continue;
        // a sequence at a chunk end has its state in slot 0 and its conv window in slot 0 of the valid buffer
        if (cudaMalloc(&px->state[il], sfl * sizeof(float)) != cudaSuccess || cudaMalloc(&px->conv[il], cfl * sizeof(float)) != cudaSuccess)
            return fail(qb_fail(QB_ERR_CUDA, "qb_prefix_capture: out of device memory"));
        const float *cv = b->conv_par ? b->conv_alt[il] : b->conv[il];
        QB_CUDA(cudaMemcpyAsync(px->state[il], b->state[il] + (size_t)seq * K1 * sfl, sfl * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        QB_CUDA(cudaMemcpyAsync(px->conv[il], cv + (size_t)seq * K1 * cfl, cfl * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    }
    QB_CUDA(cudaMalloc(&px->hid, (size_t)c.n_embd * sizeof(float)));
    QB_CUDA(cudaMemcpyAsync(px->hid, b->hid + (size_t)(b->rows_cap + seq) * c.n_embd, (size_t)c.n_embd * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    if (tokens_host) {
        QB_CUDA(cudaMalloc(&px->tokens_dev, (size_t)n * sizeof(int32_t)));
        QB_CUDA(cudaMemcpyAsync(px->tokens_dev, tokens_host, (size_t)n * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
        QB_CUDA(cudaStreamSynchronize(ctx->stream));          // the caller's array may go away
    }
    for (uint32_t i = 0; i < (uint32_t)n / b->page_size; ++i) {
        const int32_t pg = b->seq_pages[seq][i];
        if (!b->pool->share(pg)) return fail(qb_fail(QB_ERR_INVALID, "qb_prefix_capture: page %d of sequence %u is not in use", pg, seq));
        px->pages.push_back(pg);
    }
    *out = px;
    return QB_OK;
}

extern "C" int qb_prefix_attach(qb_ctx *ctx, qb_batch *b, uint32_t seq, const qb_prefix *px) {
    QB_REQUIRE(ctx && b && px && seq < b->n_seqs, "qb_prefix_attach: bad arguments");
    QB_REQUIRE(px->owner == b, "qb_prefix_attach: the prefix belongs to another batch (its pages are in that batch's pool)");
    QB_REQUIRE(b->host_pos[seq] == 0 && b->seq_pages[seq].empty(), "qb_prefix_attach: sequence %u is not empty (qb_seq_reset first)", seq);
    QB_REQUIRE(px->n_tokens < b->max_ctx, "qb_prefix_attach: the prefix fills the context");
    QB_REQUIRE(!b->seen || px->tokens_dev, "qb_prefix_attach: the batch has token penalties on and the prefix carries no tokens");
    QB_CUDA(cudaSetDevice(ctx->device));
    const qb_model_config &c = b->m->cfg;
    const uint32_t K1 = b->k + 1;
    const size_t sfl = (size_t)c.ssm_num_v_heads * c.ssm_head_dim * c.ssm_head_dim, cfl = (size_t)b->m->qkv_dim() * 3;
    for (int32_t pg : px->pages) {
        QB_REQUIRE(b->pool->share(pg), "qb_prefix_attach: page %d of the prefix is not in use", pg);
        b->seq_pages[seq].push_back(pg);
    }
    QB_TRY(upload_pages(ctx, b, seq, 0, (uint32_t)px->pages.size()));
    for (uint32_t il = 0; il < c.n_layers; ++il) {
        if (!b->state[il]) continue;
        float *cv = b->conv_par ? b->conv_alt[il] : b->conv[il];
        QB_CUDA(cudaMemcpyAsync(b->state[il] + (size_t)seq * K1 * sfl, px->state[il], sfl * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        QB_CUDA(cudaMemcpyAsync(cv + (size_t)seq * K1 * cfl, px->conv[il], cfl * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    }
    QB_CUDA(cudaMemcpyAsync(b->hid + (size_t)(b->rows_cap + seq) * c.n_embd, px->hid, (size_t)c.n_embd * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    QB_CUDA(qb_launch_pdl(ctx->stream, set_seq_ctl_kernel, dim3(1), dim3(32), (size_t)0, b->pos, b->sel, b->cur,
                          b->out_rec + b->n_seqs + (size_t)b->n_seqs * K1, seq, (int32_t)px->n_tokens));
    QB_LAUNCHED(ctx, "set_seq_ctl_kernel");
    if (b->seen) {
        QB_CUDA(qb_launch_pdl(ctx->stream, mark_seen_tokens_kernel, dim3((px->n_tokens + 127) / 128), dim3(128), (size_t)0, (const int32_t *)px->tokens_dev,
                              px->n_tokens, b->seen + (size_t)seq * b->seen_words, c.vocab_size));
        QB_LAUNCHED(ctx, "mark_seen_tokens_kernel");
    }
    b->host_pos[seq] = (int32_t)px->n_tokens;
    b->chunk_end_pos[seq] = (int32_t)px->n_tokens;
    probe_cancel(b);
    return QB_OK;
}
extern "C" uint32_t qb_prefix_tokens(const qb_prefix *px) { return px ? px->n_tokens : 0; }

static int prefill_impl(qb_ctx *ctx, qb_batch *b, uint32_t seq, const int32_t *tokens_host, uint32_t n, bool more_follows,
                        const qb_sampling *samp) {
    QB_REQUIRE(ctx && b && tokens_host && n > 0 && seq < b->n_seqs, "qb_prefill: bad arguments");
    QB_REQUIRE((uint32_t)b->host_pos[seq] + n <= b->max_ctx, "qb_prefill: %u tokens at position %d exceed max_ctx %u", n, b->host_pos[seq],
               b->max_ctx);
    QB_REQUIRE(!samp || samp->temp > 0.0f, "qb_prefill_sampled: temp must be > 0 (temp <= 0 is the greedy qb_prefill)");
    if (b->pool) {      // the whole call's pages must be there before its first chunk runs
        const uint32_t need = std::min(b->pages_per_seq, ((uint32_t)b->host_pos[seq] + n + b->page_size - 1) / b->page_size);
        const uint32_t have = (uint32_t)b->seq_pages[seq].size();
        if (need > have && b->pool->free_count() < need - have)
            return qb_fail(QB_ERR_CAPACITY, "K/V page pool exhausted: sequence %u needs %u more pages, %u of %u free", seq, need - have,
                           b->pool->free_count(), b->pool->total());
    }
    QB_CUDA(cudaSetDevice(ctx->device));
    qb_model *m = b->m;
    const qb_model_config &c = m->cfg;
    const uint32_t K1 = b->k + 1;
    // the call's tokens go to the device in one asynchronous copy through pinned staging (the caller's array may go away);
    // a later call waits for nothing but that copy of the call before it, which lies ahead of that call's kernels
    if (!b->tok_ev) QB_CUDA(cudaEventCreateWithFlags(&b->tok_ev, cudaEventDisableTiming));
    if (b->tok_stage_cap < n) {
        QB_CUDA(cudaStreamSynchronize(ctx->stream));
        if (b->tok_stage) { QB_CUDA(cudaFreeHost(b->tok_stage)); b->tok_stage = nullptr; }
        if (b->tok_all) { QB_CUDA(cudaFree(b->tok_all)); b->tok_all = nullptr; }
        QB_CUDA(cudaHostAlloc(&b->tok_stage, (size_t)n * sizeof(int32_t), cudaHostAllocDefault));
        QB_CUDA(cudaMalloc(&b->tok_all, (size_t)n * sizeof(int32_t)));
        b->tok_stage_cap = n;
    } else {
        QB_CUDA(cudaEventSynchronize(b->tok_ev));
    }
    memcpy(b->tok_stage, tokens_host, (size_t)n * sizeof(int32_t));
    QB_CUDA(cudaMemcpyAsync(b->tok_all, b->tok_stage, (size_t)n * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
    QB_CUDA(cudaEventRecord(b->tok_ev, ctx->stream));
    for (uint32_t off = 0; off < n; off += b->chunk) {
        const uint32_t M = std::min(b->chunk, n - off);
        const bool last = off + M == n && !more_follows;
        const uint32_t p0 = (uint32_t)b->host_pos[seq];
        QB_TRY(ensure_pages(ctx, b, seq, p0 + M));
        const int32_t *toks = b->tok_all + off;
        if (b->seen) {
            QB_CUDA(qb_launch_pdl(ctx->stream, mark_seen_tokens_kernel, dim3((M + 127) / 128), dim3(128), (size_t)0, toks, M,
                                  b->seen + (size_t)seq * b->seen_words, c.vocab_size));
            QB_LAUNCHED(ctx, "mark_seen_tokens_kernel");
        }
        RowSet rs;
        rs.seq0 = seq; rs.ns = 1; rs.R = M; rs.seq_pos = b->pos + seq; rs.max_pos = p0 + M; rs.ingest = true;
        QB_TRY(target_forward(ctx, b, toks, rs, false, last ? 2 : 0));
        if (c.mtp_layers && b->k > 0) {
            // MTP-layer K/V of the chunk: row r pairs token r with the target hidden of row r-1 (row 0: the previous chunk's
            // last hidden, kept behind the chunk rows)
            QB_CUDA(qb_launch_pdl(ctx->stream, chunk_map_kernel, dim3((M + 127) / 128), dim3(128), (size_t)0, b->map_chunk, M,
                                  (int32_t)(b->rows_cap + seq)));
            QB_LAUNCHED(ctx, "chunk_map_kernel");
            // the MTP pass overwrites the logits' argmax partials only in full mode; kv_only leaves them alone
            QB_TRY(mtp_forward(ctx, b, toks, b->hid, b->map_chunk, rs, true));
        }
        if (last) {
            if (samp) {
                if (!b->samp_u) QB_CUDA(cudaMalloc(&b->samp_u, 2 * (size_t)b->n_seqs * K1 * sizeof(double)));
                QB_CUDA(cudaMemcpyAsync(b->samp_u, &b->first_draw_stage[seq], sizeof(double), cudaMemcpyHostToDevice, ctx->stream));
                QB_TRY(qb_launch_sample_rows(ctx, b->logits, 1, c.vocab_size, c.vocab_size, nullptr, 0, b->samp_u, b->samp_u, samp->temp,
                                             samp->top_p, samp->top_k, samp->min_p, nullptr, nullptr, nullptr, b->am_val, b->am_idx,
                                             QB_ARGMAX_BLOCKS, b->pen_presence, b->pen_repetition,
                                             b->seen ? b->seen + (size_t)seq * b->seen_words : nullptr, b->seen_words));
            }
            QB_CUDA(qb_launch_pdl(ctx->stream, greedy_commit_kernel, dim3(1), dim3(256), (size_t)(0), b->am_val, b->am_idx, 0, M - 1, 0, seq, 1, K1, b->rows_cap, c.n_embd,
                                                           b->pos, b->sel, b->cur, (int32_t)M, b->out_rec, b->n_seqs, b->hid,
                                                           (unsigned long long *)b->stats));
            QB_LAUNCHED(ctx, "greedy_commit_kernel");
            QB_TRY(mark_seen_record(ctx, b, seq, 1));
        } else {
            QB_CUDA(qb_launch_pdl(ctx->stream, advance_kernel, dim3(1), dim3(256), (size_t)(0), b->pos, b->sel, seq, (int32_t)M, b->rows_cap, c.n_embd, M - 1, b->hid,
                                  b->out_rec + b->n_seqs + (size_t)b->n_seqs * K1));
            QB_LAUNCHED(ctx, "advance_kernel");
        }
        b->host_pos[seq] += (int32_t)M;
        probe_cancel(b);
    }
    b->chunk_end_pos[seq] = more_follows ? b->host_pos[seq] : -1;
    return QB_OK;
}

extern "C" int qb_prefill(qb_ctx *ctx, qb_batch *b, uint32_t seq, const int32_t *tokens_host, uint32_t n) {
    return prefill_impl(ctx, b, seq, tokens_host, n, false, nullptr);
}

// A part of a prompt that is not its end: K/V, recurrent state and the MTP prefix advance, no token is chosen.
extern "C" int qb_prefill_chunk(qb_ctx *ctx, qb_batch *b, uint32_t seq, const int32_t *tokens_host, uint32_t n) {
    return prefill_impl(ctx, b, seq, tokens_host, n, true, nullptr);
}

// The end of a sampled request's prompt: the first token is drawn with the request's first uniform draw u.
extern "C" int qb_prefill_sampled(qb_ctx *ctx, qb_batch *b, uint32_t seq, const int32_t *tokens_host, uint32_t n, const qb_sampling *samp,
                                  double u) {
    QB_REQUIRE(b && samp && seq < b->n_seqs, "qb_prefill_sampled: bad arguments");
    if (!b->first_draw_stage) QB_CUDA(cudaHostAlloc(&b->first_draw_stage, (size_t)b->n_seqs * sizeof(double), cudaHostAllocDefault));
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    b->first_draw_stage[seq] = u;
    return prefill_impl(ctx, b, seq, tokens_host, n, false, samp);
}

static int check_room(qb_batch *b, uint32_t need) {
    if (b->n_active == 0) return qb_fail(QB_ERR_INVALID, "no active sequence");
    for (uint32_t s = 0; s < b->n_active; ++s)
        if ((uint32_t)b->host_pos[s] + need > b->max_ctx + b->k + 1 || (uint32_t)b->host_pos[s] >= b->max_ctx)
            return qb_fail(QB_ERR_CAPACITY, "sequence %u at position %d has no room for %u more positions (max_ctx %u)", s,
                           b->host_pos[s], need, b->max_ctx);
    return QB_OK;
}

extern "C" int qb_decode_greedy_step(qb_ctx *ctx, qb_batch *b) {
    QB_REQUIRE(ctx && b, "qb_decode_greedy_step: null argument");
    QB_TRY(check_room(b, 1));
    QB_CUDA(cudaSetDevice(ctx->device));
    QB_TRY(ensure_step_pages(ctx, b, 1));
    const qb_model_config &c = b->m->cfg;
    RowSet rs;
    rs.seq0 = 0; rs.ns = b->n_active; rs.R = 1; rs.seq_pos = b->pos; rs.max_pos = max_host_pos(b) + 1;
    QB_TRY(target_forward(ctx, b, b->cur, rs, false, 1));
    QB_CUDA(qb_launch_pdl(ctx->stream, greedy_commit_kernel, dim3(b->n_active), dim3(256), (size_t)(0), b->am_val, b->am_idx, 0, 0, 1, 0, b->n_active, b->k + 1, b->rows_cap,
                                                           c.n_embd, b->pos, b->sel, b->cur, 1, b->out_rec, b->n_seqs, b->hid,
                                                           (unsigned long long *)b->stats));
    QB_LAUNCHED(ctx, "greedy_commit_kernel");
    QB_TRY(mark_seen_record(ctx, b, 0, b->n_active));
    advance_host_pos(b, 1);
    return probe_tick(ctx, b);
}

extern "C" int qb_mtp_draft(qb_ctx *ctx, qb_batch *b) {
    QB_REQUIRE(ctx && b && b->k > 0, "qb_mtp_draft: needs a batch with draft depth > 0");
    QB_TRY(check_room(b, b->k + 1));
    QB_CUDA(cudaSetDevice(ctx->device));
    QB_TRY(ensure_step_pages(ctx, b, b->k + 1));         // covers the drafts, the verify rows and the MTP prefix rows of the step
    const uint32_t ns = b->n_active, k = b->k;
    for (uint32_t i = 0; i < k; ++i) {
        QB_CUDA(qb_launch_pdl(ctx->stream, prep_draft_kernel, dim3((ns + 127) / 128), dim3(128), (size_t)(0), b->cur, b->drafts, b->pos, ns, k, i, b->tok_buf, b->seqpos_buf));
        QB_LAUNCHED(ctx, "prep_draft_kernel");
        RowSet rs;
        rs.seq0 = 0; rs.ns = ns; rs.R = 1; rs.seq_pos = b->seqpos_buf; rs.max_pos = max_host_pos(b) + i + 1;
        // step 0 reads the target hidden of the last committed position, later steps the MTP hidden
        if (i == 0) QB_TRY(mtp_forward(ctx, b, b->tok_buf, b->hid, b->map_prevh, rs, false));
        else QB_TRY(mtp_forward(ctx, b, b->tok_buf, b->mtp_h, nullptr, rs, false));
        QB_CUDA(qb_launch_pdl(ctx->stream, store_draft_kernel, dim3((ns + 3) / 4), dim3(128), (size_t)(0), b->am_val, b->am_idx, ns, k, i, b->drafts));
        QB_LAUNCHED(ctx, "store_draft_kernel");
    }
    return QB_OK;
}

extern "C" int qb_mtp_force_drafts(qb_ctx *ctx, qb_batch *b, const int32_t *forced_dev, uint32_t stride) {
    QB_REQUIRE(ctx && b && forced_dev && b->k > 0, "qb_mtp_force_drafts: bad arguments");
    const uint32_t n = b->n_active * b->k;
    QB_CUDA(qb_launch_pdl(ctx->stream, force_drafts_kernel, dim3((n + 127) / 128), dim3(128), (size_t)0, b->drafts, b->pos, b->n_active,
                          b->k, forced_dev, stride));
    QB_LAUNCHED(ctx, "force_drafts_kernel");
    return QB_OK;
}

extern "C" int qb_mtp_set_drafts(qb_ctx *ctx, qb_batch *b, const int32_t *drafts_host) {
    QB_REQUIRE(ctx && b && drafts_host && b->k > 0, "qb_mtp_set_drafts: bad arguments");
    QB_CUDA(cudaMemcpyAsync(b->drafts, drafts_host, (size_t)b->n_active * b->k * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
    return QB_OK;
}

extern "C" int qb_mtp_verify(qb_ctx *ctx, qb_batch *b) {
    QB_REQUIRE(ctx && b && b->k > 0, "qb_mtp_verify: needs a batch with draft depth > 0");
    QB_TRY(check_room(b, b->k + 1));
    QB_CUDA(cudaSetDevice(ctx->device));
    QB_TRY(ensure_step_pages(ctx, b, b->k + 1));
    const uint32_t ns = b->n_active, K1 = b->k + 1;
    QB_CUDA(qb_launch_pdl(ctx->stream, prep_verify_kernel, dim3((ns * K1 + 127) / 128), dim3(128), (size_t)(0), b->cur, b->drafts, ns, b->k, b->tok_buf));
    QB_LAUNCHED(ctx, "prep_verify_kernel");
    RowSet rs;
    rs.seq0 = 0; rs.ns = ns; rs.R = K1; rs.seq_pos = b->pos; rs.max_pos = max_host_pos(b) + K1;
    return target_forward(ctx, b, b->tok_buf, rs, true, 1);
}

extern "C" int qb_mtp_accept_commit(qb_ctx *ctx, qb_batch *b) {
    QB_REQUIRE(ctx && b && b->k > 0, "qb_mtp_accept_commit: needs a batch with draft depth > 0");
    QB_CUDA(cudaSetDevice(ctx->device));
    const qb_model_config &c = b->m->cfg;
    const uint32_t ns = b->n_active, k = b->k;
    QB_CUDA(qb_launch_pdl(ctx->stream, accept_commit_kernel, dim3(ns), dim3(256), (size_t)(0), b->am_val, b->am_idx, k, b->rows_cap, c.n_embd, b->pos, b->sel, b->cur, b->drafts,
                                                    b->prefix_pos, b->prefix_tok, b->out_rec, b->n_seqs, b->hid,
                                                    (unsigned long long *)b->stats, (const int32_t *)b->limit, b->eos_token));
    QB_LAUNCHED(ctx, "accept_commit_kernel");
    QB_TRY(mark_seen_record(ctx, b, 0, ns));
    // MTP-layer K/V of positions old_pos+1 .. old_pos+k from (draft_i, target hidden of row i-1); the
    // rows beyond the accepted prefix land past the committed length and are overwritten later.
    RowSet rs;
    rs.seq0 = 0; rs.ns = ns; rs.R = k; rs.seq_pos = b->prefix_pos; rs.max_pos = max_host_pos(b) + k + 1;
    QB_TRY(mtp_forward(ctx, b, b->prefix_tok, b->hid, b->map_prefix, rs, true));
    advance_host_pos(b, (int32_t)(k + 1));               // upper bound until the host reads the step record
    return probe_tick(ctx, b);
}

// Tensor-parallel form of a batch: its model is a shard (qb_model_create_synth_tp) and `group` the FFN group of the ranks
// (created for at least as many rows as the batch forwards at once: qb_batch_max_rows).  Every rank must then run the
// same calls on the same tokens; all of them get the same bits.  NULL goes back to the single-GPU form.
extern "C" int qb_batch_set_tp(qb_ctx *ctx, qb_batch *b, qb_tp_group *group) {
    QB_REQUIRE(ctx && b, "qb_batch_set_tp: null argument");
    QB_REQUIRE(!group || b->m->tp_world > 1 || b->m->tp_world == 1, "qb_batch_set_tp: bad model");
    if (group && !b->normed) {
        const size_t n = (size_t)b->rows_cap * b->m->cfg.n_embd * sizeof(float);
        QB_CUDA(cudaMalloc(&b->normed, n));
        QB_CUDA(cudaMalloc(&b->tp_y, n));
    }
    b->tp = group;
    qb_tp_group_set_ileave(group, 64);        // the model's gate/up shards are interleaved in groups of 64 rows
    return QB_OK;
}
extern "C" uint32_t qb_batch_max_rows(const qb_batch *b) { return b ? b->rows_cap : 0; }

// Chain policy of the speculative loop (src/qwen_native_backend.cpp:1625-1628, 15817-15848): limits_host[s] = draft depth of
// sequence s from the next step on (the reference passes min(k, tokens still wanted), at least 1; 0 here makes the step
// a plain one), eos_token = the token that ends a chain when drafted (-1: none, the reference's ignore_eos).  NULL limits
// restore depth k everywhere.  The verify forward still runs k+1 rows; the cut-off drafts are simply not compared.
extern "C" int qb_batch_set_draft_policy(qb_ctx *ctx, qb_batch *b, const int32_t *limits_host, int32_t eos_token) {
    QB_REQUIRE(ctx && b, "qb_batch_set_draft_policy: null argument");
    QB_CUDA(cudaStreamSynchronize(ctx->stream));        // the staging buffer may still be read by an earlier copy
    for (uint32_t s = 0; s < b->n_seqs; ++s) b->limit_host[s] = limits_host ? std::min<int32_t>(std::max<int32_t>(limits_host[s], 0), (int32_t)b->k) : (int32_t)b->k;
    QB_CUDA(cudaMemcpyAsync(b->limit, b->limit_host, b->n_seqs * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
    b->eos_token = eos_token;
    return QB_OK;
}

// Sampling-mode acceptance (speculative_accept_pointmass, src/qwen_native_backend.cpp:399-467): every verifier row takes
// its decision on the device from the logits the verify forward left, and hands the commit kernel the decided token in
// place of the row's argmax -- the draft itself when accepted, the residual draw when rejected, the bonus draw on the last
// row -- so the longest-matching-prefix commit that follows is the reference's accept loop.  u_host: double [n_seqs][k+1],
// the caller's uniform draws in the order its generator is consumed: row i accepts with u[i]; a rejection at row i draws
// its residual with u[i+1]; the bonus draw of a chain of depth d (k, or the sequence's draft limit, or the index of a
// drafted end-of-sequence token) is u[d].  A step that rejects after `a` acceptances consumes a + 2 of them (a + 1
// acceptance tests and the residual draw), a fully accepted chain of depth d consumes d + 1.
extern "C" int qb_mtp_sample_rows(qb_ctx *ctx, qb_batch *b, float temp, float top_p, int32_t top_k, float min_p, const double *u_host) {
    QB_REQUIRE(ctx && b && u_host && b->k > 0, "qb_mtp_sample_rows: needs draws and a batch with draft depth > 0");
    QB_CUDA(cudaSetDevice(ctx->device));
    const uint32_t ns = b->n_active, k = b->k, K1 = k + 1, rows = ns * K1;
    if (!b->samp_u) QB_CUDA(cudaMalloc(&b->samp_u, 2 * (size_t)b->n_seqs * K1 * sizeof(double)));
    const size_t slot_doubles = 2 * (size_t)b->n_seqs * K1;
    if (!b->samp_stage) {
        QB_CUDA(cudaHostAlloc(&b->samp_stage, qb_batch::SAMP_RING * slot_doubles * sizeof(double), cudaHostAllocDefault));
        for (cudaEvent_t &e : b->samp_ev) QB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    // no stream synchronisation: the draws go through a pinned ring; a slot waits only for its own copy of four steps ago
    const uint32_t slot = b->samp_slot++ % qb_batch::SAMP_RING;
    QB_CUDA(cudaEventSynchronize(b->samp_ev[slot]));
    double *u = b->samp_stage + slot * slot_doubles;
    for (uint32_t s = 0; s < ns; ++s)
        for (uint32_t i = 0; i < K1; ++i) {
            u[(size_t)s * K1 + i] = u_host[(size_t)s * K1 + i];                                  // acceptance draw of row i
            u[(size_t)rows + s * K1 + i] = u_host[(size_t)s * K1 + (i < k ? i + 1 : k)];          // residual / bonus draw
        }
    QB_CUDA(cudaMemcpyAsync(b->samp_u, u, 2 * (size_t)rows * sizeof(double), cudaMemcpyHostToDevice, ctx->stream));
    QB_CUDA(cudaEventRecord(b->samp_ev[slot], ctx->stream));
    const qb_model_config &c = b->m->cfg;
    return qb_launch_sample_rows(ctx, b->logits, rows, c.vocab_size, c.vocab_size, b->drafts, K1, b->samp_u, b->samp_u + rows, temp, top_p,
                                 top_k, min_p, nullptr, nullptr, nullptr, b->am_val, b->am_idx, QB_ARGMAX_BLOCKS, b->pen_presence, b->pen_repetition,
                                 b->seen, b->seen_words, b->limit, b->eos_token);
}

extern "C" int qb_mtp_step_sampled(qb_ctx *ctx, qb_batch *b, float temp, float top_p, int32_t top_k, float min_p, const double *u_host) {
    QB_TRY(qb_mtp_draft(ctx, b));
    QB_TRY(qb_mtp_verify(ctx, b));
    QB_TRY(qb_mtp_sample_rows(ctx, b, temp, top_p, top_k, min_p, u_host));
    return qb_mtp_accept_commit(ctx, b);
}

extern "C" int qb_mtp_step(qb_ctx *ctx, qb_batch *b) {
    QB_TRY(qb_mtp_draft(ctx, b));
    QB_TRY(qb_mtp_verify(ctx, b));
    return qb_mtp_accept_commit(ctx, b);
}

extern "C" int qb_read_step_output(qb_ctx *ctx, qb_batch *b, int32_t *n_out_host, int32_t *tokens_host) {
    QB_REQUIRE(ctx && b, "qb_read_step_output: null argument");
    const uint32_t ns = b->n_seqs, K1 = b->k + 1;
    const size_t n = (size_t)ns * (K1 + 2);
    QB_CUDA(cudaMemcpyAsync(b->out_rec_host, b->out_rec, n * sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    QB_TRY(qb_synchronize(ctx));
    if (n_out_host) memcpy(n_out_host, b->out_rec_host, ns * sizeof(int32_t));
    if (tokens_host) memcpy(tokens_host, b->out_rec_host + ns, (size_t)ns * K1 * sizeof(int32_t));
    for (uint32_t s = 0; s < ns; ++s) b->host_pos[s] = b->out_rec_host[ns + (size_t)ns * K1 + s];
    probe_cancel(b);
    return QB_OK;
}

// Counters of the speculative loop as the reference's summary lines report them (native mtp_spec_summary: /
// mtp_accept_hist:, src/qwen_native_backend.cpp:16313-16392): out[0] = steps that rejected a draft, out[1 + a] = steps that
// accepted exactly a drafts, a = 0 .. min(k, n - 2).
extern "C" int qb_batch_accept_hist(qb_ctx *ctx, qb_batch *b, int64_t *out, uint32_t n) {
    QB_REQUIRE(ctx && b && out && n >= 1, "qb_batch_accept_hist: bad arguments");
    long long h[QB_STATS];
    QB_CUDA(cudaMemcpyAsync(h, b->stats, sizeof(h), cudaMemcpyDeviceToHost, ctx->stream));
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    out[0] = h[4];
    for (uint32_t a = 0; a + 1 < n && a <= b->k && a < 8; ++a) out[1 + a] = h[8 + a];
    return QB_OK;
}

extern "C" int qb_batch_stats(qb_ctx *ctx, qb_batch *b, int64_t *out4) {
    QB_CUDA(cudaMemcpyAsync(out4, b->stats, 4 * sizeof(long long), cudaMemcpyDeviceToHost, ctx->stream));
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    return QB_OK;
}

extern "C" int qb_seq_position(qb_ctx *ctx, qb_batch *b, uint32_t seq, int32_t *pos) {
    QB_REQUIRE(seq < b->n_seqs, "qb_seq_position: sequence out of range");
    QB_CUDA(cudaMemcpyAsync(pos, b->pos + seq, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    return QB_OK;
}

// Slot recycling of the continuous-batching loop: the retired request's recurrent state, conv windows, position and
// previous hidden row go back to their initial values; the slot keeps its K/V pages (entries beyond the position are
// never read, so they need no clearing).
extern "C" int qb_seq_reset(qb_ctx *ctx, qb_batch *b, uint32_t seq) {
    QB_REQUIRE(ctx && b && seq < b->n_seqs, "qb_seq_reset: bad arguments");
    QB_CUDA(cudaSetDevice(ctx->device));
    const qb_model_config &c = b->m->cfg;
    const uint32_t K1 = b->k + 1;
    const size_t ssz = (size_t)K1 * c.ssm_num_v_heads * c.ssm_head_dim * c.ssm_head_dim, csz = (size_t)K1 * b->m->qkv_dim() * 3;
    for (uint32_t il = 0; il < c.n_layers; ++il) {
        if (!b->state[il]) continue;
        QB_CUDA(cudaMemsetAsync(b->state[il] + seq * ssz, 0, ssz * sizeof(float), ctx->stream));
        QB_CUDA(cudaMemsetAsync(b->conv[il] + seq * csz, 0, csz * sizeof(float), ctx->stream));
        QB_CUDA(cudaMemsetAsync(b->conv_alt[il] + seq * csz, 0, csz * sizeof(float), ctx->stream));
    }
    // the step record of the slot too: the host's position mirror is refreshed from it (qb_read_step_output)
    for (int32_t *p : {b->pos, b->sel, b->cur, b->prefix_pos, b->out_rec, b->out_rec + b->n_seqs + (size_t)b->n_seqs * K1})
        QB_CUDA(cudaMemsetAsync(p + seq, 0, sizeof(int32_t), ctx->stream));
    QB_CUDA(cudaMemsetAsync(b->hid + (size_t)(b->rows_cap + seq) * c.n_embd, 0, (size_t)c.n_embd * sizeof(float), ctx->stream));
    if (b->seen) QB_CUDA(cudaMemsetAsync(b->seen + (size_t)seq * b->seen_words, 0, (size_t)b->seen_words * sizeof(uint32_t), ctx->stream));
    b->host_pos[seq] = 0;
    probe_cancel(b);
    b->chunk_end_pos[seq] = -1;
    release_pages(b, seq);                                   // stream order keeps earlier readers of these pages ahead of their next writer
    return QB_OK;
}

// The decode steps run the sequences [0, n): a continuous-batching loop keeps its live requests in the first slots
// (qb_seq_swap moves one) so that empty slots and requests still being prefilled cost nothing.
extern "C" int qb_batch_set_active(qb_ctx *ctx, qb_batch *b, uint32_t n) {
    QB_REQUIRE(ctx && b && n <= b->n_seqs, "qb_batch_set_active: bad arguments");
    b->n_active = n;
    probe_cancel(b);
    return QB_OK;
}

// Exchange everything two sequence slots hold: K/V pages (their page-table rows), DeltaNet state and conv windows of
// every layer, position, selected checkpoint, current token, previous hidden row, seen-token record.
extern "C" int qb_seq_swap(qb_ctx *ctx, qb_batch *b, uint32_t s1, uint32_t s2) {
    QB_REQUIRE(ctx && b && s1 < b->n_seqs && s2 < b->n_seqs, "qb_seq_swap: bad arguments");
    if (s1 == s2) return QB_OK;
    QB_CUDA(cudaSetDevice(ctx->device));
    const qb_model_config &c = b->m->cfg;
    const uint32_t K1 = b->k + 1;
    const size_t ssz = (size_t)K1 * c.ssm_num_v_heads * c.ssm_head_dim * c.ssm_head_dim * sizeof(float);
    const size_t csz = (size_t)K1 * b->m->qkv_dim() * 3 * sizeof(float);
    const size_t need = std::max({ssz, csz, (size_t)c.n_embd * sizeof(float), (size_t)b->pages_per_seq * sizeof(int32_t),
                                  (size_t)b->seen_words * sizeof(uint32_t)});
    if (b->swap_bytes < need) {
        if (b->swap_tmp) { QB_CUDA(cudaStreamSynchronize(ctx->stream)); QB_CUDA(cudaFree(b->swap_tmp)); b->swap_tmp = nullptr; }
        QB_CUDA(cudaMalloc(&b->swap_tmp, need));
        b->swap_bytes = need;
    }
    auto swap_block = [&](void *base, size_t bytes) -> int {
        char *a = (char *)base + (size_t)s1 * bytes, *d = (char *)base + (size_t)s2 * bytes;
        QB_CUDA(cudaMemcpyAsync(b->swap_tmp, a, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        QB_CUDA(cudaMemcpyAsync(a, d, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        QB_CUDA(cudaMemcpyAsync(d, b->swap_tmp, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        return QB_OK;
    };
    for (uint32_t il = 0; il < c.n_layers; ++il) {
        if (!b->state[il]) continue;
        QB_TRY(swap_block(b->state[il], ssz));
        QB_TRY(swap_block(b->conv[il], csz));
        QB_TRY(swap_block(b->conv_alt[il], csz));
    }
    QB_TRY(swap_block(b->page_table, (size_t)b->pages_per_seq * sizeof(int32_t)));
    QB_TRY(swap_block(b->hid + (size_t)b->rows_cap * c.n_embd, (size_t)c.n_embd * sizeof(float)));
    if (b->seen) QB_TRY(swap_block(b->seen, (size_t)b->seen_words * sizeof(uint32_t)));
    QB_CUDA(qb_launch_pdl(ctx->stream, swap_ctl_kernel, dim3(1), dim3(32), (size_t)0, b->pos, b->sel, b->cur, b->prefix_pos, b->out_rec, b->limit, b->n_seqs, K1, s1, s2));
    QB_LAUNCHED(ctx, "swap_ctl_kernel");
    std::swap(b->host_pos[s1], b->host_pos[s2]);
    if (b->pool) std::swap(b->seq_pages[s1], b->seq_pages[s2]);
    std::swap(b->chunk_end_pos[s1], b->chunk_end_pos[s2]);
    probe_cancel(b);
    return QB_OK;
}

// ---- state snapshots (StateSnapshot / capture_state / restore_state, src/qwen_executor.cpp:7285-7411) ----------------
// Everything a later restore needs to continue every sequence from this point: the control block (positions, selected
// checkpoint slots, current tokens, step records), the previous hidden rows, every DeltaNet state slot and conv window,
// the seen-token record.  The K/V caches are not copied: entries at or beyond a sequence's position are never read, and
// entries below it are never rewritten.
struct qb_snapshot {
    std::vector<void *> bufs;
    QbPagePool::State pool;
    std::vector<std::vector<int32_t>> seq_pages;
    std::vector<int32_t> host_pos;
    int conv_par = 0;
    uint32_t n_active = 0;
    size_t ctl_ints = 0;
};

static size_t ctl_count(const qb_batch *b) {
    return (size_t)b->n_seqs * (17 + 4 * (b->k + 1)) + 4 * (size_t)b->rows_cap + 256;
}

template <typename F>
static int for_each_state_block(qb_batch *b, F f) {
    const qb_model_config &c = b->m->cfg;
    const uint32_t K1 = b->k + 1;
    const size_t ssz = (size_t)b->n_seqs * K1 * c.ssm_num_v_heads * c.ssm_head_dim * c.ssm_head_dim * sizeof(float);
    const size_t csz = (size_t)b->n_seqs * K1 * b->m->qkv_dim() * 3 * sizeof(float);
    QB_TRY(f((void *)b->ctl, ctl_count(b) * sizeof(int32_t)));
    QB_TRY(f((void *)(b->hid + (size_t)b->rows_cap * c.n_embd), (size_t)b->n_seqs * c.n_embd * sizeof(float)));
    QB_TRY(f((void *)b->stats, QB_STATS * sizeof(long long)));
    QB_TRY(f((void *)b->page_table, (size_t)b->n_seqs * b->pages_per_seq * sizeof(int32_t)));      // qb_seq_swap exchanges rows
    for (uint32_t il = 0; il < c.n_layers; ++il) {
        if (!b->state[il]) continue;
        QB_TRY(f((void *)b->state[il], ssz));
        QB_TRY(f((void *)b->conv[il], csz));
        QB_TRY(f((void *)b->conv_alt[il], csz));
    }
    if (b->seen) QB_TRY(f((void *)b->seen, (size_t)b->n_seqs * b->seen_words * sizeof(uint32_t)));
    return QB_OK;
}

extern "C" int qb_batch_snapshot(qb_ctx *ctx, qb_batch *b, qb_snapshot **out) {
    QB_REQUIRE(ctx && b && out, "qb_batch_snapshot: null argument");
    QB_CUDA(cudaSetDevice(ctx->device));
    qb_snapshot *sn = new qb_snapshot();
    int st = for_each_state_block(b, [&](void *src, size_t bytes) -> int {
        void *dst = nullptr;
        QB_CUDA(cudaMalloc(&dst, bytes));
        sn->bufs.push_back(dst);
        QB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        return QB_OK;
    });
    if (st != QB_OK) { for (void *p : sn->bufs) cudaFree(p); delete sn; return st; }
    sn->host_pos = b->host_pos; sn->conv_par = b->conv_par; sn->n_active = b->n_active; sn->ctl_ints = ctl_count(b);
    if (b->pool) { sn->pool = b->pool->save(); sn->seq_pages = b->seq_pages; }
    *out = sn;
    return QB_OK;
}

extern "C" int qb_batch_restore(qb_ctx *ctx, qb_batch *b, const qb_snapshot *sn) {
    QB_REQUIRE(ctx && b && sn && sn->ctl_ints == ctl_count(b) && sn->host_pos.size() == b->n_seqs, "qb_batch_restore: the snapshot is not of this batch");
    QB_CUDA(cudaSetDevice(ctx->device));
    size_t i = 0;
    QB_TRY(for_each_state_block(b, [&](void *dst, size_t bytes) -> int {
        QB_REQUIRE(i < sn->bufs.size(), "qb_batch_restore: the batch gained state since the snapshot");
        QB_CUDA(cudaMemcpyAsync(dst, sn->bufs[i++], bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        return QB_OK;
    }));
    b->host_pos = sn->host_pos; b->conv_par = sn->conv_par; b->n_active = sn->n_active;
    if (b->pool) { b->pool->load(sn->pool); b->seq_pages = sn->seq_pages; }
    probe_cancel(b);
    return QB_OK;
}

extern "C" void qb_snapshot_free(qb_ctx *ctx, qb_snapshot *sn) {
    if (!sn) return;
    cudaStreamSynchronize(ctx->stream);
    for (void *p : sn->bufs) cudaFree(p);
    delete sn;
}

extern "C" int qb_debug_last_logits(qb_ctx *ctx, qb_batch *b, float *host_out, uint32_t max_rows, uint32_t *rows_out) {
    const uint32_t r = std::min(max_rows, b->last_logit_rows);
    if (r) QB_CUDA(cudaMemcpyAsync(host_out, b->logits, (size_t)r * b->m->cfg.vocab_size * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (rows_out) *rows_out = r;
    return QB_OK;
}
extern "C" int qb_debug_last_drafts(qb_ctx *ctx, qb_batch *b, int32_t *host_out) {
    QB_REQUIRE(ctx && b && host_out && b->k > 0, "qb_debug_last_drafts: bad arguments");
    QB_CUDA(cudaMemcpyAsync(host_out, b->drafts, (size_t)b->n_seqs * b->k * sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    return QB_OK;
}
