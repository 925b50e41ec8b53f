// Op-level C entry points for the attention and DeltaNet kernels (used by the parity tests and by
// a DeviceBackend shim; the engine calls the launchers directly).
#include "qb_internal.h"

extern "C" int qb_qk_norm_rope_append(qb_ctx *ctx, float *qkv_dev, uint32_t rows, uint32_t row_stride, const float *q_norm_w,
                                      const float *k_norm_w, const float *inv_freq_dev, uint32_t n_heads, uint32_t n_kv_heads,
                                      uint32_t head_dim, uint32_t rope_dim, float eps, const int32_t *seq_pos_dev,
                                      uint32_t n_seqs, const int32_t *page_table_dev, uint32_t page_table_stride,
                                      uint32_t page_size, void *k_cache_dev, void *v_cache_dev) {
    QB_REQUIRE(ctx && qkv_dev && q_norm_w && k_norm_w && inv_freq_dev && seq_pos_dev && page_table_dev && k_cache_dev && v_cache_dev,
               "qb_qk_norm_rope_append: null argument");
    QB_REQUIRE(n_seqs > 0 && rows > 0 && page_size > 0, "qb_qk_norm_rope_append: empty launch");
    AttnArgs a;
    a.qkv = qkv_dev; a.rows = rows; a.row_stride = row_stride; a.n_heads = n_heads; a.n_kv = n_kv_heads; a.hd = head_dim;
    a.rope_dim = rope_dim; a.eps = eps; a.q_norm_w = q_norm_w; a.k_norm_w = k_norm_w; a.inv_freq = inv_freq_dev;
    a.page_table = page_table_dev; a.pt_stride = page_table_stride; a.page_size = page_size;
    a.k_cache = (__half *)k_cache_dev; a.v_cache = (__half *)v_cache_dev;
    return qb_attn_prepare(ctx, a, seq_pos_dev, n_seqs);
}

static int attention_paged(qb_ctx *ctx, const float *qkv_dev, uint32_t rows, uint32_t row_stride, uint32_t n_heads,
                           uint32_t n_kv_heads, uint32_t head_dim, const int32_t *seq_pos_dev, uint32_t n_seqs,
                           const int32_t *page_table_dev, uint32_t page_table_stride, uint32_t page_size,
                           const void *k_cache_dev, const void *v_cache_dev, uint32_t max_pos, float *out_dev, bool gated);

extern "C" int qb_attention_paged_gated(qb_ctx *ctx, const float *qkv_dev, uint32_t rows, uint32_t row_stride, uint32_t n_heads,
                                        uint32_t n_kv_heads, uint32_t head_dim, const int32_t *seq_pos_dev, uint32_t n_seqs,
                                        const int32_t *page_table_dev, uint32_t page_table_stride, uint32_t page_size,
                                        const void *k_cache_dev, const void *v_cache_dev, uint32_t max_pos, float *out_dev) {
    return attention_paged(ctx, qkv_dev, rows, row_stride, n_heads, n_kv_heads, head_dim, seq_pos_dev, n_seqs, page_table_dev, page_table_stride,
                           page_size, k_cache_dev, v_cache_dev, max_pos, out_dev, true);
}
// The same attention without the output gate (attention_decode, include/qw3/device_backend.hpp:2204-2217; the caller
// applies apply_attn_gate itself).
extern "C" int qb_attention_paged(qb_ctx *ctx, const float *qkv_dev, uint32_t rows, uint32_t row_stride, uint32_t n_heads,
                                  uint32_t n_kv_heads, uint32_t head_dim, const int32_t *seq_pos_dev, uint32_t n_seqs,
                                  const int32_t *page_table_dev, uint32_t page_table_stride, uint32_t page_size,
                                  const void *k_cache_dev, const void *v_cache_dev, uint32_t max_pos, float *out_dev) {
    return attention_paged(ctx, qkv_dev, rows, row_stride, n_heads, n_kv_heads, head_dim, seq_pos_dev, n_seqs, page_table_dev, page_table_stride,
                           page_size, k_cache_dev, v_cache_dev, max_pos, out_dev, false);
}

static int attention_paged(qb_ctx *ctx, const float *qkv_dev, uint32_t rows, uint32_t row_stride, uint32_t n_heads,
                           uint32_t n_kv_heads, uint32_t head_dim, const int32_t *seq_pos_dev, uint32_t n_seqs,
                           const int32_t *page_table_dev, uint32_t page_table_stride, uint32_t page_size,
                           const void *k_cache_dev, const void *v_cache_dev, uint32_t max_pos, float *out_dev, bool gated) {
    QB_REQUIRE(ctx && qkv_dev && seq_pos_dev && page_table_dev && k_cache_dev && v_cache_dev && out_dev,
               "qb_attention_paged_gated: null argument");
    QB_REQUIRE(n_seqs > 0 && rows > 0 && page_size > 0, "qb_attention_paged_gated: empty launch");
    AttnArgs a;
    a.qkv = const_cast<float *>(qkv_dev); a.rows = rows; a.row_stride = row_stride; a.n_heads = n_heads; a.n_kv = n_kv_heads;
    a.hd = head_dim; a.page_table = page_table_dev; a.pt_stride = page_table_stride; a.page_size = page_size;
    a.k_cache = (__half *)const_cast<void *>(k_cache_dev); a.v_cache = (__half *)const_cast<void *>(v_cache_dev);
    a.max_pos = max_pos;
    a.no_gate = !gated;
    size_t ml = 0;
    const size_t acc = qb_attention_scratch_floats(rows, n_heads, head_dim, max_pos, &ml);
    void *scr = nullptr;
    QB_TRY(qb_ctx_scratch(ctx, (acc + ml) * sizeof(float), &scr));
    a.part_acc = (float *)scr;
    a.part_ml = a.part_acc + acc;
    return qb_attn_run(ctx, a, seq_pos_dev, n_seqs, out_dev, nullptr, 0, nullptr, 0);
}

extern "C" int qb_deltanet_rows(qb_ctx *ctx, const float *proj_dev, uint32_t n_seqs, uint32_t rows_per_seq, uint32_t proj_stride,
                                const float *conv_w, const float *ssm_a, const float *dt_bias, const float *norm_w, uint32_t nk,
                                uint32_t nv, uint32_t hd, float eps, float *state_dev, float *conv_dev, uint32_t n_slots,
                                const int32_t *slot_in_dev, int write_all, float *core_dev) {
    QB_REQUIRE(ctx && proj_dev && conv_w && ssm_a && dt_bias && norm_w && state_dev && conv_dev && slot_in_dev && core_dev,
               "qb_deltanet_rows: null argument");
    const uint32_t rows = n_seqs * rows_per_seq, C = (2 * nk + nv) * hd, vdim = nv * hd;
    QB_REQUIRE(proj_stride >= C + vdim + 2 * nv, "qb_deltanet_rows: proj_stride %u too small", proj_stride);
    // the kernel reads the conv windows from one buffer and writes the new ones to another: the old ones are
    // copied to scratch first so the caller's buffer can be the output
    const size_t conv_floats = (size_t)n_seqs * n_slots * C * 3;
    void *scr = nullptr;
    QB_TRY(qb_ctx_scratch(ctx, conv_floats * sizeof(float), &scr));
    float *conv_old = (float *)scr;
    QB_CUDA(cudaMemcpyAsync(conv_old, conv_dev, conv_floats * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    DnArgs d;
    d.proj = proj_dev; d.proj_stride = proj_stride; d.n_seqs = n_seqs; d.rows_per_seq = rows_per_seq;
    d.conv_w = conv_w; d.ssm_a = ssm_a; d.dt_bias = dt_bias; d.norm_w = norm_w; d.nk = nk; d.nv = nv; d.hd = hd; d.eps = eps;
    d.state = state_dev; d.conv = conv_old; d.conv_out = conv_dev; d.n_slots = n_slots; d.slot_in = slot_in_dev; d.write_all = write_all;
    d.core_out = core_dev;
    return qb_launch_deltanet(ctx, d);
}

// q8_0_matmul_silu_mul (include/qw3/device_backend.hpp:300-539) for the fused [gate; up] weight, leaving the result
// as the quantised input of the down projection.
extern "C" int qb_q8_0_matmul_silu_mul_q8(qb_ctx *ctx, const qb_weight *gate_up, const float *x_dev, uint32_t M, uint32_t x_stride,
                                          int8_t *hq_dev, float *hd_dev, int mode) {
    QB_REQUIRE(ctx && gate_up && x_dev && hq_dev && hd_dev && M > 0, "qb_q8_0_matmul_silu_mul_q8: bad arguments");
    QB_REQUIRE(gate_up->rows % 128 == 0 && gate_up->cols % 128 == 0, "qb_q8_0_matmul_silu_mul_q8: weight must be whole 128 x 128 tiles");
    const uint32_t K = gate_up->cols, N = gate_up->rows, F = N / 2, ld = qb_act_ld(M), S = qb_ksplit(N, K);
    const size_t q_bytes = ((size_t)M * K + 255) & ~(size_t)255, d_bytes = ((size_t)(K / 32) * ld * 4 + 255) & ~(size_t)255;
    const size_t act_floats = (size_t)S * M * N;
    void *scr = nullptr;
    QB_TRY(qb_ctx_scratch(ctx, q_bytes + d_bytes + act_floats * sizeof(float), &scr));
    int8_t *xq = (int8_t *)scr;
    float *xd = (float *)((uint8_t *)scr + q_bytes), *act = (float *)((uint8_t *)scr + q_bytes + d_bytes);
    NormQuantArgs a;
    a.x = x_dev; a.x_stride = x_stride; a.n = K; a.M = M; a.q = xq; a.q_pitch = K; a.d = xd; a.d_ld = ld;
    QB_TRY(qb_launch_norm_quant(ctx, a));
    return qb_ffn_gate_up_swiglu(ctx, gate_up, xq, xd, M, act, act, act_floats, hq_dev, F, hd_dev, ld, 0, mode);
}

namespace {
// [proj | gate | alpha | beta] of the DeviceBackend interface (four tensors with their own row strides) -> the fused
// row layout of the DeltaNet kernel.
__global__ void pack_dn_rows_kernel(float *fused, uint32_t fstride, const float *proj, uint32_t ps, const float *gate, uint32_t gs,
                                    const float *alpha, uint32_t as, const float *beta, uint32_t bs, uint32_t C, uint32_t vdim, uint32_t nv) {
    QB_PDL_ENTER();
    const uint32_t row = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= fstride) return;
    float v;
    if (i < C) v = proj[(size_t)row * ps + i];
    else if (i < C + vdim) v = gate[(size_t)row * gs + (i - C)];
    else if (i < C + vdim + nv) v = alpha[(size_t)row * as + (i - C - vdim)];
    else v = beta[(size_t)row * bs + (i - C - vdim - nv)];
    fused[(size_t)row * fstride + i] = v;
}
}  // namespace

// DeviceBackend::recurrent_batch / recurrent_single_token with the interface's own tensors (include/qw3/device_backend.hpp:
// 665-800): `batch` consecutive tokens of ONE sequence.  state = float [nv][hd][hd] and conv_state = float [qkv_dim][3] are
// read and left at the values after the last token; with ckpt_count > 0 the state / conv window after token t < ckpt_count
// also go to state_ckpt[t] / conv_ckpt[t] (src/gated_delta_net.cu:165-176, src/kernels_cuda.cu:3682-3691).
// core = float [batch][core_stride] receives the gated, normalised output (nv*hd per row).
extern "C" int qb_recurrent_batch(qb_ctx *ctx, float *core, uint32_t core_stride, float *state, float *conv_state, const float *proj,
                                  uint32_t proj_stride, const float *gate, uint32_t gate_stride, const float *alpha, uint32_t alpha_stride,
                                  const float *beta, uint32_t beta_stride, const float *conv_w, const float *ssm_a, const float *dt_bias,
                                  const float *ssm_norm, uint32_t batch, uint32_t nk, uint32_t nv, uint32_t hd, float eps, float *state_ckpt,
                                  float *conv_ckpt, uint32_t ckpt_count) {
    QB_REQUIRE(ctx && core && state && conv_state && proj && gate && alpha && beta && conv_w && ssm_a && dt_bias && ssm_norm && batch > 0,
               "qb_recurrent_batch: bad arguments");
    QB_REQUIRE(ckpt_count == 0 || (state_ckpt && conv_ckpt && ckpt_count <= batch), "qb_recurrent_batch: checkpoint buffers missing or too many checkpoints");
    const uint32_t C = (2 * nk + nv) * hd, vdim = nv * hd, fstride = C + vdim + 2 * nv;
    QB_REQUIRE(core_stride >= vdim, "qb_recurrent_batch: core_stride %u below %u", core_stride, vdim);
    const uint32_t n_slots = ckpt_count ? batch : 1;
    const size_t sfl = (size_t)nv * hd * hd, cfl = (size_t)C * 3;
    auto al = [](size_t v) { return (v + 63) & ~(size_t)63; };
    const size_t o_fused = 0, o_state = o_fused + al((size_t)batch * fstride), o_conv = o_state + al(n_slots * sfl), o_conv2 = o_conv + al(n_slots * cfl),
                 o_core = o_conv2 + al(n_slots * cfl), o_zero = o_core + al((size_t)batch * vdim), total = o_zero + 64;
    void *scr = nullptr;
    QB_TRY(qb_ctx_scratch2(ctx, total * sizeof(float), &scr));
    float *f = (float *)scr;
    QB_CUDA(qb_launch_pdl(ctx->stream, pack_dn_rows_kernel, dim3((fstride + 255) / 256, batch), dim3(256), (size_t)0, f + o_fused, fstride, proj, proj_stride,
                          gate, gate_stride, alpha, alpha_stride, beta, beta_stride, C, vdim, nv));
    QB_LAUNCHED(ctx, "pack_dn_rows_kernel");
    QB_CUDA(cudaMemcpyAsync(f + o_state, state, sfl * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    QB_CUDA(cudaMemcpyAsync(f + o_conv, conv_state, cfl * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    QB_CUDA(cudaMemsetAsync(f + o_zero, 0, 64 * sizeof(float), ctx->stream));
    DnArgs d;
    d.proj = f + o_fused; d.proj_stride = fstride; d.n_seqs = 1; d.rows_per_seq = batch;
    d.conv_w = conv_w; d.ssm_a = ssm_a; d.dt_bias = dt_bias; d.norm_w = ssm_norm; d.nk = nk; d.nv = nv; d.hd = hd; d.eps = eps;
    d.state = f + o_state; d.conv = f + o_conv; d.conv_out = f + o_conv2; d.n_slots = n_slots; d.slot_in = (const int32_t *)(f + o_zero);
    d.write_all = ckpt_count ? 1 : 0;
    d.core_out = core_stride == vdim ? core : f + o_core;
    QB_TRY(qb_launch_deltanet(ctx, d));
    const uint32_t last = ckpt_count ? batch - 1 : 0;
    QB_CUDA(cudaMemcpyAsync(state, f + o_state + last * sfl, sfl * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    QB_CUDA(cudaMemcpyAsync(conv_state, f + o_conv2 + last * cfl, cfl * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    if (ckpt_count) {
        QB_CUDA(cudaMemcpyAsync(state_ckpt, f + o_state, (size_t)ckpt_count * sfl * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        QB_CUDA(cudaMemcpyAsync(conv_ckpt, f + o_conv2, (size_t)ckpt_count * cfl * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    }
    if (core_stride != vdim)
        QB_CUDA(cudaMemcpy2DAsync(core, (size_t)core_stride * sizeof(float), f + o_core, (size_t)vdim * sizeof(float), (size_t)vdim * sizeof(float), batch,
                                  cudaMemcpyDeviceToDevice, ctx->stream));
    return QB_OK;
}
