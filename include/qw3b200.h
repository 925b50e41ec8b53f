/* qw3b200 — C ABI of the B200 (sm_100a) MTP speculative-decode step for the qwen35 hybrid
 * model (Q8_0 weights, paged fp16 KV, gated DeltaNet + gated full attention).
 *
 * This is the drop-in boundary: plain pointers and sizes, no C++ or torch types.  Every
 * entry point names the reference interface it stands in for (path:line inside the
 * kvmem-qw3 tree).  Functions return 0 on success and a non-zero code on failure;
 * qb_last_error() returns the message of the last failure on the calling thread (the
 * same lifetime rule as the reference's DeviceStatus::message,
 * include/qw3/device_backend.hpp:24-27).  All device work is enqueued on the context's
 * single stream in call order (the reference backend's exec stream,
 * src/kernels_cuda.cu:9673-9695); nothing here falls back to the CPU.
 */
#ifndef QW3B200_H
#define QW3B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QB_OK 0
#define QB_ERR_INVALID 1
#define QB_ERR_CUDA 2
#define QB_ERR_UNSUPPORTED 3
#define QB_ERR_CAPACITY 4

typedef struct qb_ctx qb_ctx;
typedef struct qb_weight qb_weight;
typedef struct qb_model qb_model;
typedef struct qb_batch qb_batch;

/* Hyper-parameters of the qwen35 hybrid model; field meaning follows QwenConfig
 * (include/qw3/qwen_config.hpp:15-68).  Layer i is full attention iff
 * (i + 1) % full_attention_interval == 0. */
typedef struct qb_model_config {
    uint32_t n_layers;
    uint32_t n_embd;
    uint32_t n_ff;
    uint32_t n_heads;
    uint32_t n_kv_heads;
    uint32_t head_dim;
    uint32_t rope_dim;
    float    rope_theta;
    float    rms_eps;
    uint32_t ssm_conv_kernel;      /* 4 */
    uint32_t ssm_num_k_heads;      /* ssm_group_count */
    uint32_t ssm_num_v_heads;      /* ssm_time_step_rank */
    uint32_t ssm_head_dim;         /* ssm_state_size: head_k_dim == head_v_dim */
    uint32_t full_attention_interval;
    uint32_t vocab_size;
    uint32_t mtp_layers;           /* 0 or 1 (nextn_predict_layers) */
    float    weight_sigma;         /* std of the seeded random-init weights (0.02) */
} qb_model_config;

/* ---- context ---------------------------------------------------------------------- */

/* make_cuda_device_backend (include/qw3/device_backend.hpp:2744) + the backend ctor's
 * device/stream set-up (src/kernels_cuda.cu:9673-9695).  `device` is the CUDA ordinal. */
int  qb_create(int device, qb_ctx **out);
void qb_destroy(qb_ctx *ctx);
const char *qb_last_error(void);
/* DeviceBackend::synchronize / end (device_backend.hpp:93-95). */
int  qb_synchronize(qb_ctx *ctx);
/* Raw CUDA stream handle (cudaStream_t) of the context, for callers that time with events. */
void *qb_stream(qb_ctx *ctx);
int  qb_sm_count(qb_ctx *ctx);

/* DeviceBackend::tensor_f32/f16/i32, scratch_f32 (device_backend.hpp:124-213) reduced to
 * bytes; copy_to_host (:148), copy_i32_from_host (:2454), copy_d2d (:2514), zero_tensor. */
/* DeviceBackend::free_device_bytes / total_device_bytes (device_backend.hpp:97-103). */
int qb_mem_info(qb_ctx *ctx, size_t *free_bytes, size_t *total_bytes);
int qb_malloc(qb_ctx *ctx, size_t bytes, void **dev_ptr);
int qb_free(qb_ctx *ctx, void *dev_ptr);
int qb_memcpy_h2d(qb_ctx *ctx, void *dev_dst, const void *host_src, size_t bytes);
int qb_memcpy_d2h(qb_ctx *ctx, void *host_dst, const void *dev_src, size_t bytes);
int qb_memcpy_d2d(qb_ctx *ctx, void *dev_dst, const void *dev_src, size_t bytes);
int qb_memset(qb_ctx *ctx, void *dev_ptr, int value, size_t bytes);
/* Pinned host buffers for end-to-end timing (cudaHostAlloc). */
int qb_host_alloc(qb_ctx *ctx, size_t bytes, void **host_ptr);
int qb_host_free(qb_ctx *ctx, void *host_ptr);

/* CUDA-event timing on the context stream. */
int qb_event_create(qb_ctx *ctx, void **event);
int qb_event_record(qb_ctx *ctx, void *event);
int qb_event_elapsed_ms(qb_ctx *ctx, void *start, void *stop, float *ms);
int qb_event_destroy(qb_ctx *ctx, void *event);
/* Writes `bytes` of a private buffer (larger than L2) so the next timed call starts cold. */
int qb_flush_l2(qb_ctx *ctx);

/* ---- Q8_0 weights ----------------------------------------------------------------- */

/* DeviceBackend::weight_q8_0(data, rows, cols, label) (device_backend.hpp:215) and the
 * CudaWeight Q8_0 ctor's repack (src/kernels_cuda.cu:1566-1594).  `host_blocks` is the GGUF
 * layout: rows x (cols/32) blocks of 34 bytes [fp16 d | int8 q[32]].  The pointer is not
 * retained.  cols must be a multiple of 128. */
int qb_weight_q8_0(qb_ctx *ctx, const void *host_blocks, uint32_t rows, uint32_t cols, qb_weight **out);
/* Seeded random-init weight generated on the device, byte-identical to uploading the
 * blocks produced by qs_synth_q8_0_block (include/qw3b200_synth.h). */
int qb_weight_q8_0_synth(qb_ctx *ctx, uint64_t seed, uint32_t tensor_id, uint32_t rows, uint32_t cols,
                         float sigma, qb_weight **out);
/* Inverse repack back to GGUF 34-byte blocks (test aid). */
int qb_weight_q8_0_download(qb_ctx *ctx, const qb_weight *w, void *host_blocks);
void qb_weight_free(qb_ctx *ctx, qb_weight *w);
uint32_t qb_weight_rows(const qb_weight *w);
uint32_t qb_weight_cols(const qb_weight *w);

/* ---- activation quantisation ------------------------------------------------------ */

/* quantize_q8_1_kernel (src/mmvq_q8.cu:83-112): out = M x (K/32) blocks of 36 bytes
 * {half d, half sum, int8 q[32]}. */
int qb_quantize_q8_1(qb_ctx *ctx, const float *x_dev, uint32_t M, uint32_t K, uint32_t x_stride, void *out_dev);
/* quantize_mmq_q8_1_kernel (src/mmvq_q8.cu:669-722): out = (K/128) x M blocks of 144 bytes
 * {float d4[4], int8 q[128]}, block index sb * M + row. */
int qb_quantize_q8_1_mmq(qb_ctx *ctx, const float *x_dev, uint32_t M, uint32_t K, uint32_t x_stride, void *out_dev);
/* The engine's own planar form of the same arithmetic as q8_1_mmq: q_dev = int8 [M][K],
 * d_dev = float [K/32][ld] with ld = M rounded up to a multiple of 4 (scale of block kb of row m at kb*ld + m). */
int qb_quantize_act(qb_ctx *ctx, const float *x_dev, uint32_t M, uint32_t K, uint32_t x_stride,
                    int8_t *q_dev, float *d_dev);

/* ---- Q8_0 x Q8 products ----------------------------------------------------------- */

/* Number of K segments the engine uses for an [N x K] weight (a function of the shape only,
 * never of M, so a row's result does not depend on how many rows share the launch). */
uint32_t qb_ksplit_policy(uint32_t N, uint32_t K);

/* Exact int32 block dots: out_dev = int32 [M][N][K/32], the integer part shared by
 * mul_mat_vec_q8_0_kernel (src/mmvq_q8.cu:156-172) and the MMQ kernels (src/mmq_q8.cu:1738-1748). */
int qb_q8_block_dots(qb_ctx *ctx, const qb_weight *w, const int8_t *q_dev, uint32_t M, int32_t *out_dev);

/* DeviceBackend::q8_0_matmul / q8_0_matvec (device_backend.hpp:300-539):
 * y[m][n] = sum_kb d_w[n][kb] * d_x[m][kb] * int32dot, fp32 in / fp32 out.
 *   order = 0: engine order (K segments of qb_ksplit_policy or `ksplit` if non-zero; sequential
 *              fma per 32-block inside a segment as in src/mmq_q8.cu:1738-1748; segments summed ascending)
 *   impl  = 0: automatic, 1: CUDA-core dp4a streaming kernel, 2: tcgen05 INT8 tensor-core kernel.
 * Both implementations produce identical bits. */
int qb_q8_0_matmul(qb_ctx *ctx, const qb_weight *w, const float *x_dev, uint32_t M, uint32_t x_stride,
                   float *y_dev, uint32_t y_stride, uint32_t ksplit, int impl);
/* The same product as qb_q8_0_matmul (identical bits) for callers that must not allocate device memory:
 * a server whose own arena already owns the whole device, or a loop that cannot take the device-wide
 * synchronisation hidden in cudaMalloc / cudaFree.  It has no counterpart in the reference.  The work area
 * (int8 activations, scales, K-segment partial sums) is an 8 MiB array built into the library image, held by
 * every GPU that loads the library; shapes that need more are refused with QB_ERR_CAPACITY.  The first call on
 * a device looks the array's address up (make that call before any stream capture starts).  All calls share
 * the one array: calls that may overlap on the GPU (different streams or contexts of one device) race. */
int qb_q8_0_matmul_noalloc(qb_ctx *ctx, const qb_weight *w, const float *x_dev, uint32_t M, uint32_t x_stride,
                           float *y_dev, uint32_t y_stride, uint32_t ksplit);
/* Same product from already-quantised activations, leaving the per-segment partial sums:
 * part_dev = float [ksplit][M][N]. */
int qb_q8_gemm_partials(qb_ctx *ctx, const qb_weight *w, const int8_t *q_dev, const float *d_dev, uint32_t M,
                        float *part_dev, uint32_t ksplit, int impl);

/* The two FFN input tensors as ONE weight, rows interleaved in groups of 64 (tile t = gate rows [64t, 64t+64) then
 * up rows [64t, 64t+64)): what weight_q8_0 (include/qw3/device_backend.hpp:215) does for ffn_gate and ffn_up, in
 * the layout the fused kernel below needs. */
int qb_weight_q8_0_gate_up(qb_ctx *ctx, const void *gate_blocks, const void *up_blocks, uint32_t n_ff, uint32_t cols,
                           qb_weight **out);
/* q8_0_matmul_silu_mul (include/qw3/device_backend.hpp:300-539): h = silu(W_gate x) * (W_up x) for M rows, left as
 * the quantised input of the down projection: hq_dev = int8 [M][n_ff], hd_dev = float [n_ff/32][ld] (qb_quantize_act
 * layout).  With M <= 16 and a one-segment weight the GEMM's epilogue does it in one launch; otherwise GEMM + a
 * SwiGLU kernel.  mode: 0 = choose, 1 = always two launches, 2 = one launch or fail; all give the same bits. */
int qb_q8_0_matmul_silu_mul_q8(qb_ctx *ctx, const qb_weight *gate_up, const float *x_dev, uint32_t M, uint32_t x_stride,
                               int8_t *hq_dev, float *hd_dev, int mode);

/* ---- element-wise / norm / rope / embedding --------------------------------------- */

/* q8_get_rows_batch_kernel (src/kernels_cuda.cu:2075-2157): out[i][:] = dequant(row ids[i]). */
int qb_q8_0_get_rows(qb_ctx *ctx, const qb_weight *w, const int32_t *ids_dev, uint32_t n, float *out_dev,
                     uint32_t out_stride);
/* rms_norm_batch (src/kernels_cuda.cu:1948-2010, :14781). */
int qb_rms_norm(qb_ctx *ctx, const float *x_dev, const float *w_dev, uint32_t M, uint32_t n, uint32_t stride,
                float eps, float *out_dev);
/* Row grouping of the attention and DeltaNet entry points: sequence s owns rows
 * [s*R, (s+1)*R) with R = rows / n_seqs, at consecutive positions seq_pos_dev[s] .. seq_pos_dev[s]+R-1
 * (the (k+1) verify rows of a request, or one decode row).  seq_pos_dev is int32 [n_seqs] on the device. */

/* rmsnorm_per_head_batch + rope_partial_batch on q and k, then kv_append_batch_paged_device
 * (src/kernels_cuda.cu:4622-4645, 4697-4799, 8921-8969) in one launch.  qkv_dev rows are
 * [q: n_heads x (2*head_dim, second half = output gate) | k: n_kv x head_dim | v: n_kv x head_dim]; q is
 * normalised and rotated in place; k,v of a row at position pos go to physical slot
 * page_table[seq][pos/page_size]*page_size + pos%page_size as fp16 (cache = [slot][n_kv][head_dim]).
 * inv_freq_dev = float [rope_dim/2], theta^(-2i/rope_dim). */
int qb_qk_norm_rope_append(qb_ctx *ctx, float *qkv_dev, uint32_t rows, uint32_t row_stride,
                           const float *q_norm_w, const float *k_norm_w, const float *inv_freq_dev,
                           uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t rope_dim, float eps,
                           const int32_t *seq_pos_dev, uint32_t n_seqs,
                           const int32_t *page_table_dev, uint32_t page_table_stride, uint32_t page_size,
                           void *k_cache_dev, void *v_cache_dev);

/* attention_decode_batch_paged_gated_device / ..._ragged_device (src/kernels_cuda.cu:20187-20358,
 * device_backend.hpp:2204-2450): a row at position pos attends keys [0, pos] of its sequence's pages,
 * scale 1/sqrt(head_dim), GQA, fp16 K/V, fp32 softmax, output x sigmoid(gate).  max_pos is a host upper
 * bound of every row position.  out_dev = float [rows][n_heads*head_dim]. */
int qb_attention_paged_gated(qb_ctx *ctx, const float *qkv_dev, uint32_t rows, uint32_t row_stride,
                             uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                             const int32_t *seq_pos_dev, uint32_t n_seqs,
                             const int32_t *page_table_dev, uint32_t page_table_stride, uint32_t page_size,
                             const void *k_cache_dev, const void *v_cache_dev, uint32_t max_pos,
                             float *out_dev);

/* DeviceBackend::recurrent_batch / recurrent_batch_ragged with checkpoints (device_backend.hpp:665-933,
 * src/kernels_cuda.cu:15053-15972): conv1d(4)+SiLU, L2-norm q/k, gated delta rule, RMSNorm x SiLU(z).
 * proj_dev rows = [qkv (2*nk*hd + nv*hd) | z (nv*hd) | alpha (nv) | beta (nv)], row stride proj_stride,
 * rows_per_seq rows per sequence.  State slots: state_dev = float [n_seqs][n_slots][nv][hd][hd],
 * conv_dev = float [n_seqs][n_slots][qkv_dim][3].  Sequence s reads slot slot_in_dev[s]; with
 * write_all != 0 the state after row t goes to slot t (rows_per_seq <= n_slots), else only the final
 * state goes to slot 0.  core_dev = float [rows][nv*hd] (gated, normalised output). */
int qb_deltanet_rows(qb_ctx *ctx, const float *proj_dev, uint32_t n_seqs, uint32_t rows_per_seq, uint32_t proj_stride,
                     const float *conv_w, const float *ssm_a, const float *dt_bias, const float *norm_w,
                     uint32_t nk, uint32_t nv, uint32_t hd, float eps,
                     float *state_dev, float *conv_dev, uint32_t n_slots, const int32_t *slot_in_dev, int write_all,
                     float *core_dev);

/* recurrent_batch / recurrent_single_token with the interface's own tensors (device_backend.hpp:665-800): `batch`
 * consecutive tokens of one sequence; proj / gate / alpha / beta are separate row-major tensors with their own strides;
 * state = float [nv][hd][hd] and conv_state = float [qkv_dim][3] are updated to the values after the last token; with
 * ckpt_count > 0 the state and conv window after token t < ckpt_count also go to state_ckpt[t] / conv_ckpt[t]
 * (src/gated_delta_net.cu:165-176, src/kernels_cuda.cu:3682-3691).  core = float [batch][core_stride]. */
int qb_recurrent_batch(qb_ctx *ctx, float *core, uint32_t core_stride, float *state, float *conv_state, const float *proj,
                       uint32_t proj_stride, const float *gate, uint32_t gate_stride, const float *alpha, uint32_t alpha_stride,
                       const float *beta, uint32_t beta_stride, const float *conv_w, const float *ssm_a, const float *dt_bias,
                       const float *ssm_norm, uint32_t batch, uint32_t nk, uint32_t nv, uint32_t hd, float eps, float *state_ckpt,
                       float *conv_ckpt, uint32_t ckpt_count);

/* argmax_batch (src/kernels_cuda.cu:1765-1888, :20814): lowest index wins ties.  out_dev = int32 [M]. */
int qb_argmax_rows(qb_ctx *ctx, const float *x_dev, uint32_t M, uint32_t n, uint32_t stride, int32_t *out_dev);
/* argmax / argmax_to_buffer / copy_argmax_buffer_to_host (include/qw3/device_backend.hpp:2456-2497): token and logit
 * of row m go to tok_dev[out_offset + m] / val_dev[out_offset + m] (a DeviceArgmaxBuffer is the pair of arrays). */
int qb_argmax_rows_val(qb_ctx *ctx, const float *x_dev, uint32_t M, uint32_t n, uint32_t stride, int32_t *tok_dev, float *val_dev,
                       uint32_t out_offset);

/* ---- the operators the executor calls one by one -----------------------------------------------------------------
 * The fused step launches none of these (norms, RoPE, K/V append and gating live inside its attention / DeltaNet /
 * norm kernels); a DeviceBackend subclass over this library needs them to answer every virtual. */
/* add, add_n (include/qw3/device_backend.hpp:639-647), mul (:649), silu (:648), silu_mul / silu_mul_n (:650-664;
 * silu_mul_kernel src/kernels_cuda.cu:1894-1903).  out may alias an input. */
int qb_add(qb_ctx *ctx, float *out, const float *a, const float *b, uint64_t n);
int qb_mul(qb_ctx *ctx, float *out, const float *a, const float *b, uint64_t n);
int qb_silu(qb_ctx *ctx, float *out, const float *x, uint64_t n);
int qb_silu_mul(qb_ctx *ctx, float *out, const float *gate, const float *up, uint64_t n);
/* rmsnorm_per_head / rmsnorm_per_head_batch (device_backend.hpp:948-974; src/kernels_cuda.cu:4622-4645): in place,
 * unit u of row b at x + b*batch_stride + u*per_unit_stride, head_dim elements, one gain vector for all units. */
int qb_rmsnorm_per_head(qb_ctx *ctx, float *x, const float *w, uint32_t batch, uint32_t batch_stride, uint32_t n_units,
                        uint32_t per_unit_stride, uint32_t head_dim, float eps);
/* rope_partial / rope_partial_batch / rope_partial_batch_positions (device_backend.hpp:975-1044; src/kernels_cuda.cu:
 * 4697-4719, 4779-4799): rotates the first rope_dim elements of every unit, pairs (i, i + rope_dim/2); row b is at
 * position base_pos + b, or positions_dev[b] when that is given. */
int qb_rope_partial(qb_ctx *ctx, float *x, uint32_t batch, uint32_t batch_stride, uint32_t n_units, uint32_t per_unit_stride,
                    uint32_t rope_dim, uint32_t base_pos, const int32_t *positions_dev, float theta);
/* kv_append / kv_append_batch (device_backend.hpp:1047-1089; src/kernels_cuda.cu:8921-8949) when page_indices_dev is
 * NULL, kv_append_batch_paged_device (:1090-1119, :8950-8969) otherwise: row b (per_pos_size floats) goes as fp16 to
 * slot base_pos + b, or page_indices[pos / page_size] * page_size + pos % page_size. */
int qb_kv_append(qb_ctx *ctx, void *cache_f16, const float *src, uint32_t base_pos, uint32_t per_pos_size, uint32_t batch,
                 const int32_t *page_indices_dev, uint32_t n_pages, uint32_t page_size);
/* apply_attn_gate / apply_attn_gate_batch (device_backend.hpp:2218-2262; src/kernels_cuda.cu:9448-9465):
 * out[b][h][d] *= sigmoid(q[b*batch_stride_q + h*q_stride + head_dim + d]). */
int qb_apply_attn_gate(qb_ctx *ctx, float *out, const float *q, uint32_t q_stride, uint32_t batch, uint32_t batch_stride_q,
                       uint32_t batch_stride_out, uint32_t n_heads, uint32_t head_dim);
/* attention_decode (device_backend.hpp:2204-2217): qb_attention_paged_gated without the output gate. */
int qb_attention_paged(qb_ctx *ctx, const float *qkv_dev, uint32_t rows, uint32_t row_stride,
                       uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                       const int32_t *seq_pos_dev, uint32_t n_seqs,
                       const int32_t *page_table_dev, uint32_t page_table_stride, uint32_t page_size,
                       const void *k_cache_dev, const void *v_cache_dev, uint32_t max_pos,
                       float *out_dev);
/* pack_mtp_prefix_hinputs (device_backend.hpp:2646-2660): dst[0] = first_h, dst[1..batch-1] = h_batch[0..batch-2], rows of
 * h_stride floats.  pack_mtp_concat (:2662-2695): dst[row] = [left[row][0:width] | right[row][0:width]]. */
int qb_pack_mtp_prefix_hinputs(qb_ctx *ctx, float *dst, const float *first_h, const float *h_batch, uint32_t batch, uint32_t h_stride);
int qb_pack_mtp_concat(qb_ctx *ctx, float *dst, const float *left, const float *right, uint32_t batch, uint32_t left_stride,
                       uint32_t right_stride, uint32_t concat_stride, uint32_t width);

/* ---- model / sequences / the MTP step --------------------------------------------- */

/* QwenWeights ctor (src/qwen_weights.cpp:170-208) with seeded random-init tensors instead of a
 * GGUF file: every Q8_0 tensor ~ quantise(N(0, sigma^2)), norm gains 1, DeltaNet fp32 tensors from
 * the same seed (recipe in qw3b200_synth.h and the engine source). */
int  qb_model_create_synth(qb_ctx *ctx, const qb_model_config *cfg, uint64_t seed, qb_model **out);
/* One named tensor of a checkpoint on the host.  Names are the GGUF names the reference binds
 * (src/qwen_native.cpp:147-190, MTP block :271-298): token_embd.weight, output_norm.weight, output.weight,
 * blk.<i>.attn_norm.weight, blk.<i>.ffn_norm.weight (or post_attention_norm.weight), attention layers
 * attn_q / attn_k / attn_v / attn_output / attn_q_norm / attn_k_norm, DeltaNet layers attn_qkv / attn_gate /
 * ssm_alpha / ssm_beta / ssm_out (.weight), ssm_conv1d.weight, ssm_a, ssm_dt.bias, ssm_norm.weight, every layer
 * ffn_gate / ffn_up / ffn_down (.weight); the MTP layer is block n_layers with nextn.eh_proj / nextn.enorm /
 * nextn.hnorm and the optional nextn.embed_tokens / nextn.shared_head_head / nextn.shared_head_norm.
 * type is the GGUF tensor type: the two the reference maps from a GGUF file (src/model_source.cpp:120-121).
 * cols = dims[0] (input features), rows = product of the other dims (src/qwen_weights.cpp:12-22). */
#define QB_TENSOR_F32 0u     /* data = float [rows * cols] */
#define QB_TENSOR_Q8_0 8u    /* data = rows x (cols / 32) blocks of 34 bytes [fp16 d | int8 q[32]] */
typedef struct qb_tensor_desc {
    const char *name;
    uint32_t    type;
    uint64_t    rows, cols;
    const void *data;
} qb_tensor_desc;
/* QwenNativeModel tensor binding + QwenWeights upload (src/qwen_native.cpp:147-190, 271-298;
 * src/qwen_weights.cpp:170-208) from the caller's tensors: every projection Q8_0, every norm gain and the small
 * DeltaNet tensors F32.  The host pointers are not retained.  A missing or mis-shaped tensor fails with its name. */
int  qb_model_create(qb_ctx *ctx, const qb_model_config *cfg, const qb_tensor_desc *tensors, size_t n_tensors, qb_model **out);
/* GgufFile + QwenConfig + the binding above (src/gguf.cpp:216-278, src/qwen_config.cpp:53-108): maps a GGUF v3
 * file, reads the qwen35.* hyper-parameters (vocab_size = length of tokenizer.ggml.tokens) and uploads the tensors.
 * cfg_out (may be NULL) receives the configuration read. */
int  qb_model_load_gguf(qb_ctx *ctx, const char *path, qb_model **out, qb_model_config *cfg_out);
/* The parsing half alone (no device needed): configuration, number of F32 / Q8_0 tensors and their bytes. */
int  qb_gguf_read_config(const char *path, qb_model_config *cfg_out, uint64_t *n_tensors_out, uint64_t *tensor_bytes_out);
const qb_model_config *qb_model_get_config(const qb_model *m);
void qb_model_destroy(qb_ctx *ctx, qb_model *m);
size_t qb_model_weight_bytes(const qb_model *m);

/* ---- tokenizer (host only; no device) ----------------------------------------------------------------------------
 * qw3::QwenTokenizer (include/qw3/tokenizer.hpp:30-45, src/tokenizer.cpp): the byte-level BPE tokenizer of the
 * checkpoint, built from tokenizer.ggml.tokens / tokenizer.ggml.merges and the bos / eos / add_bos hints
 * (src/tokenizer.cpp:180-216).  The chat-template special tokens the vocabulary holds (<|im_start|>, <think>, ...,
 * :327-358) are matched whole; the text between them is cut by the Qwen split pattern (:376-514) and merged piece by
 * piece (:516-562).  Token ids are what qb_prefill takes. */
typedef struct qb_tokenizer qb_tokenizer;
/* QwenTokenizer(const GgufFile &) */
int  qb_tokenizer_load_gguf(const char *path, qb_tokenizer **out);
/* The same from the caller's own tables: n_tokens strings (id = index), n_merges lines "left right" (rank = index). */
int  qb_tokenizer_create(const char *const *tokens, const uint32_t *token_lens, uint32_t n_tokens, const char *const *merges,
                         const uint32_t *merge_lens, uint32_t n_merges, int32_t bos_id, int32_t eos_id, int add_bos,
                         qb_tokenizer **out);
void qb_tokenizer_destroy(qb_tokenizer *t);
/* vocab_size(), bos_id(), eos_id(), add_bos_default() (tokenizer.hpp:40-43) and the number of special tokens found;
 * any output may be NULL. */
int  qb_tokenizer_info(const qb_tokenizer *t, int32_t *vocab_size, int32_t *bos_id, int32_t *eos_id, int *add_bos_default,
                       uint32_t *n_special);
/* token_id() (tokenizer.hpp:47-50): the id of a literal vocabulary string, -1 if absent. */
int  qb_tokenizer_token_id(const qb_tokenizer *t, const char *token, uint32_t len);
/* encode() (src/tokenizer.cpp:574-717): BOS first when add_bos or the checkpoint's default asks for it.  *n_out is
 * the number of tokens even when cap is too small (the call then fails with the capacity error). */
int  qb_tokenizer_encode(const qb_tokenizer *t, const char *text, size_t len, int add_bos, int32_t *ids, size_t cap, size_t *n_out);
/* decode() (src/tokenizer.cpp:719-745): bytes, not necessarily whole UTF-8 sequences; ids outside the vocabulary are
 * skipped. */
int  qb_tokenizer_decode(const qb_tokenizer *t, const int32_t *ids, size_t n, char *text, size_t cap, size_t *len_out);
/* detail::qwen_pre_tokenize (src/tokenizer_internal.hpp): the piece boundaries of a text without special tokens,
 * piece_ends[i] = byte offset one past piece i. */
int  qb_tokenizer_split(const char *text, size_t len, uint32_t *piece_ends, size_t cap, size_t *n_out);

/* Per-request executor state of `n_seqs` sequences (QwenExecutor state, src/qwen_executor.hpp:763-819
 * KvPageTable; GlobalKvPagePool src/qwen_native_backend.cpp:1155-1265): paged fp16 K/V for the target
 * and the MTP layer, DeltaNet/conv state slots, positions.  page_order: 0 = identity, 1 = reverse,
 * 2 = seeded shuffle (the alloc modes of src/qwen_executor.cpp:1752-1774). */
int  qb_batch_create(qb_ctx *ctx, qb_model *m, uint32_t n_seqs, uint32_t max_ctx, uint32_t draft_k,
                     uint32_t page_size, int page_order, qb_batch **out);
/* The pooled form of the same (GlobalKvPagePool, src/qwen_native_backend.cpp:1155-1265; allocate_continuous_kv_cache /
 * _mtp_kv_cache, :6603-6709): the K/V caches hold pool_pages pages in all, shared by the n_seqs sequences; a sequence's
 * page-table row grows page by page as its position grows (most recently freed page first) and goes back to the pool at
 * qb_seq_reset.  A call that needs more pages than are free returns QB_ERR_CAPACITY before anything is launched. */
int  qb_batch_create_pooled(qb_ctx *ctx, qb_model *m, uint32_t n_seqs, uint32_t max_ctx, uint32_t draft_k,
                            uint32_t page_size, uint32_t pool_pages, qb_batch **out);
int  qb_batch_pool_info(qb_ctx *ctx, qb_batch *b, uint32_t *free_pages, uint32_t *total_pages, uint32_t *page_size);
/* The pages sequence `seq` holds, in position order (at most cap written; *n_out = how many it holds). */
int  qb_seq_pages(qb_ctx *ctx, qb_batch *b, uint32_t seq, int32_t *pages_out, uint32_t cap, uint32_t *n_out);
/* The allocator of the pooled batches on its own, for a caller that keeps its own page tables over the op-level entry
 * points (host side only, thread-safe): a LIFO free stack that hands out page 0 first; a page may have several holders
 * (qb_page_pool_share) and returns to the stack when the last one drops it.  alloc: page id or -1 when exhausted;
 * share: 1, or 0 for a page that is not in use; drop: holders left, or -1 for a page that is not in use. */
void    *qb_page_pool_create(uint32_t total_pages);
void     qb_page_pool_destroy(void *pool);
int32_t  qb_page_pool_alloc(void *pool);
int32_t  qb_page_pool_share(void *pool, int32_t page);
int32_t  qb_page_pool_drop(void *pool, int32_t page);
uint32_t qb_page_pool_free_count(void *pool);
/* Shared prompt prefixes (the server's prefix cache, src/qwen_native_backend.cpp:9785-10410: a hit seeds the request from
 * the cached entry, whose pages stay pinned while it lives).  qb_prefix_capture takes an entry from a sequence of a pooled
 * batch that has ingested exactly the prefix with qb_prefill_chunk (a whole number of pages): the entry holds the
 * prefix's K/V pages once more and copies of the DeltaNet state, conv windows and last hidden row at its end;
 * tokens_host (the prefix's tokens; may be NULL unless token penalties are on) feeds the seen-token record.
 * qb_prefix_attach makes an empty sequence (after qb_seq_reset) of the same batch continue from the prefix end: it shares
 * the pages and receives the copies; the caller goes on with qb_prefill / qb_prefill_chunk of the rest of its prompt.
 * qb_prefix_release drops the entry's hold on the pages (they return to the pool when no sequence uses them either); an
 * entry must be released before its batch is destroyed (the pool lives in the batch). */
typedef struct qb_prefix qb_prefix;
int  qb_prefix_capture(qb_ctx *ctx, qb_batch *b, uint32_t seq, const int32_t *tokens_host, uint32_t n_tokens, qb_prefix **out);
int  qb_prefix_attach(qb_ctx *ctx, qb_batch *b, uint32_t seq, const qb_prefix *prefix);
uint32_t qb_prefix_tokens(const qb_prefix *prefix);
void qb_prefix_release(qb_ctx *ctx, qb_prefix *prefix);
void qb_batch_destroy(qb_ctx *ctx, qb_batch *b);

/* forward_n_tokens prefill branch + prime_mtp_prefix (src/qwen_executor.cpp:6003-6836,
 * 22543-22815): ingest `n` prompt tokens of sequence `seq` (chunked), leave next token = argmax of
 * the last row. */
int qb_prefill(qb_ctx *ctx, qb_batch *b, uint32_t seq, const int32_t *tokens_host, uint32_t n);
/* A part of a prompt that is not its end (the chunked ingestion of a continuous-batching loop, ContinuousPrefillBatch,
 * src/qwen_native_backend.cpp:4482-4530): K/V, recurrent state and MTP prefix advance; no LM head, no token is chosen,
 * nothing is counted as emitted or recorded as seen beyond the prompt tokens.  Finish with qb_prefill(_sampled). */
int qb_prefill_chunk(qb_ctx *ctx, qb_batch *b, uint32_t seq, const int32_t *tokens_host, uint32_t n);
/* Sampling parameters of a request (GenerationOptions, include/qw3/qw3.hpp:222-230). */
typedef struct qb_sampling { float temp, top_p; int32_t top_k; float min_p; } qb_sampling;
/* The end of a sampled request's prompt: as qb_prefill, but the first token is drawn from the last row's logits with
 * the request's first uniform draw u (pick_from_last_logits, src/qwen_native_backend.cpp:15399-15428: token penalties
 * against the prompt when qb_batch_set_penalties is on, then sample_token). */
int qb_prefill_sampled(qb_ctx *ctx, qb_batch *b, uint32_t seq, const int32_t *tokens_host, uint32_t n, const qb_sampling *samp, double u);

/* forward_one_token + argmax (src/qwen_executor.cpp:5446-5816): one non-speculative greedy step
 * for every sequence.  Emits one token per sequence. */
int qb_decode_greedy_step(qb_ctx *ctx, qb_batch *b);

/* forward_mtp_draft_chain_with_prefix_device (src/qwen_executor.cpp:6942-7023): k chained MTP-head
 * forwards per sequence, argmax kept on the device. */
int qb_mtp_draft(qb_ctx *ctx, qb_batch *b);
/* Replace the drafts by forced ones before verification (the seeded-acceptance form of the benchmark):
 * draft i of sequence s becomes forced_dev[s*stride + pos + 1 + i], the caller's guess for the token at
 * absolute position pos+1+i (int32 [n_seqs][stride] on the device). */
int qb_mtp_force_drafts(qb_ctx *ctx, qb_batch *b, const int32_t *forced_dev, uint32_t stride);
/* Drafts supplied by the host (int32 [n_seqs][k], pinned memory for an asynchronous copy): the
 * host-driven form of the reference loop, where the host holds the chain it verifies
 * (src/qwen_native_backend.cpp:15903). */
int qb_mtp_set_drafts(qb_ctx *ctx, qb_batch *b, const int32_t *drafts_host);
/* forward_n_tokens verify branch (src/qwen_executor.cpp:6003-6836): (k+1)-row target forward per
 * sequence with per-row DeltaNet/conv state checkpoints and per-row argmax. */
int qb_mtp_verify(qb_ctx *ctx, qb_batch *b);
/* Acceptance + commit (src/qwen_native_backend.cpp:15948-16154; restore_state_checkpoint
 * src/qwen_executor.cpp:22304-22428; prime_mtp_prefix_from_last_batch_at :22543) on the device:
 * longest draft prefix equal to the row argmaxes, emit accepted+1 tokens, select the state
 * checkpoint, advance the position, rebuild the MTP-layer K/V of the committed positions. */
int qb_mtp_accept_commit(qb_ctx *ctx, qb_batch *b);
/* draft + verify + accept_commit. */
int qb_mtp_step(qb_ctx *ctx, qb_batch *b);
/* Chain policy of the speculative loop: limits_host[seq] = draft depth from the next step on, the reference's
 * min(chain, tokens still wanted) (MtpAdaptivePolicy::draft_limit, src/qwen_native_backend.cpp:1625-1628; 0 makes the
 * step a plain one, the empty-chain case of :15829-15848; NULL = depth k everywhere); eos_token = the token that ends a
 * chain when drafted (:15817-15821; -1 = none, the reference's ignore_eos).  The counters of qb_batch_stats count the
 * drafts of the cut chain, as the reference's mtp_spec_summary does. */
int qb_batch_set_draft_policy(qb_ctx *ctx, qb_batch *b, const int32_t *limits_host, int32_t eos_token);

/* Sampling-mode requests (temp > 0).  The reference copies the verifier's logits to the host and runs
 * sampling_distribution (src/qwen_native_backend.cpp:282-370: softmax(logits / temp), then top-k, min-p and nucleus
 * truncation, renormalised over the kept set) and speculative_accept_pointmass (:399-467: a greedy draft is accepted with
 * probability p[draft]; a rejection draws from p with the draft removed and stops; a fully accepted chain draws a bonus
 * token from the last row) there.  qb_sample_rows does the same per logits row on the device:
 *   draft_dev[row] >= 0: accepted_dev[row] = (u_acc_dev[row] < p[draft]); token = draft if accepted, else the residual draw
 *   with u_res_dev[row]; draft_dev == NULL or draft_dev[row] < 0: token = a draw from p with u_res_dev[row].
 * Draws walk the nonzero entries in index order (sample_from, :373-383, std::discrete_distribution).  top_k <= 0, top_p
 * outside (0,1) and min_p <= 0 switch the respective truncation off.  Ties at the truncation boundary are kept lowest index
 * first.  Token penalties are applied by the batch-level form below only.  p_draft_dev / accepted_dev may be NULL. */
int qb_sample_rows(qb_ctx *ctx, const float *logits_dev, uint32_t rows, uint32_t V, uint32_t stride, const int32_t *draft_dev,
                   const double *u_acc_dev, const double *u_res_dev, float temp, float top_p, int32_t top_k, float min_p,
                   int32_t *token_dev, int32_t *accepted_dev, float *p_draft_dev);
/* The same decision for the rows of the last qb_mtp_verify, left where qb_mtp_accept_commit reads the row tokens: call
 * between the two.  u_host: double [n_seqs][k+1], the caller's uniform draws in the order the reference consumes its
 * generator: row i accepts with u[i], a rejection at row i draws with u[i+1], the bonus draw of a chain of depth d is u[d]
 * (d = k, or less under qb_batch_set_draft_policy: the sequence's limit, or the index of a drafted end-of-sequence token);
 * a step that rejects after a acceptances uses the first a + 2 of them, a fully accepted chain d + 1.  One difference to
 * the reference's generator remains: std::discrete_distribution draws nothing when fewer than two tokens are left to
 * choose from, this function counts that draw as used; the sampled distribution is the same. */
int qb_mtp_sample_rows(qb_ctx *ctx, qb_batch *b, float temp, float top_p, int32_t top_k, float min_p, const double *u_host);
/* Token penalties of sampling requests (apply_token_penalties, src/qwen_native_backend.cpp:262-280: a seen token's logit is
 * divided by repetition when >= 0, multiplied when < 0, then lowered by presence): from this call on the batch records the
 * prompt and emitted tokens of every sequence, and qb_mtp_sample_rows penalises their logits and, on row i, those of the
 * step's drafts 0..i-1 (the running prefix of the accept loop, :432-447).  Call before the prefill of the requests it
 * should cover; qb_seq_reset clears a sequence's record.  presence = 0 and repetition = 1 switch the penalties off. */
int qb_batch_set_penalties(qb_ctx *ctx, qb_batch *b, float presence, float repetition);
/* draft + verify + sample_rows + accept_commit. */
int qb_mtp_step_sampled(qb_ctx *ctx, qb_batch *b, float temp, float top_p, int32_t top_k, float min_p, const double *u_host);

/* Host view of what the last step emitted: n_out[seq] tokens in tokens[seq*(k+1) ...]. Performs
 * the step's single device->host copy and a stream sync. */
int qb_read_step_output(qb_ctx *ctx, qb_batch *b, int32_t *n_out_host, int32_t *tokens_host);
/* Counters since creation: [steps, drafted, accepted, emitted] per batch. */
int qb_batch_stats(qb_ctx *ctx, qb_batch *b, int64_t *out4);
/* Counters behind the reference's `native mtp_spec_summary:` / `native mtp_accept_hist:` lines
 * (src/qwen_native_backend.cpp:16313-16392): out[0] = steps that rejected a draft (rejected = rollbacks there),
 * out[1 + a] = steps that accepted exactly a drafts (len<a>), for a = 0 .. min(k, n - 2). */
int qb_batch_accept_hist(qb_ctx *ctx, qb_batch *b, int64_t *out, uint32_t n);
/* Position (committed tokens) of a sequence; reads a device counter (syncs). */
int qb_seq_position(qb_ctx *ctx, qb_batch *b, uint32_t seq, int32_t *pos);
/* Slot recycling of the continuous-batching loop (request retirement and admission,
 * src/qwen_native_backend.cpp:6711-6866; page release of GlobalKvPagePool :1155-1265): sequence `seq` goes back to
 * position 0 with zero DeltaNet / conv state, ready for qb_prefill of the next request.  The slot keeps its K/V pages.
 * The other sequences of the batch are untouched. */
int qb_seq_reset(qb_ctx *ctx, qb_batch *b, uint32_t seq);
/* The decode steps (greedy, draft, verify, sample, accept) run the sequences [0, n); the others keep their state untouched
 * and may be prefilled meanwhile.  A continuous-batching loop keeps its live requests in the first slots: empty slots and
 * requests still being ingested then cost nothing (the reference's worker loop likewise decodes its `active` list only,
 * src/qwen_native_backend.cpp:6711-6866).  A new batch has n = n_seqs. */
int qb_batch_set_active(qb_ctx *ctx, qb_batch *b, uint32_t n);
/* Exchange the contents of two sequence slots (page-table rows, DeltaNet state and conv windows, position, current
 * token, previous hidden row, seen-token record). */
int qb_seq_swap(qb_ctx *ctx, qb_batch *b, uint32_t s1, uint32_t s2);
/* StateSnapshot / capture_state / restore_state (src/qwen_executor.cpp:7285-7411): a snapshot holds what a later restore
 * needs to continue every sequence of the batch from this point (positions, selected checkpoint slots, current tokens,
 * previous hidden rows, every DeltaNet state slot and conv window, the seen-token record); the K/V caches are not copied
 * (entries at or beyond a position are never read, entries below it never rewritten).  Restore into the same batch. */
typedef struct qb_snapshot qb_snapshot;
int  qb_batch_snapshot(qb_ctx *ctx, qb_batch *b, qb_snapshot **out);
int  qb_batch_restore(qb_ctx *ctx, qb_batch *b, const qb_snapshot *snap);
void qb_snapshot_free(qb_ctx *ctx, qb_snapshot *snap);
/* Test aids: logits of the last verify/greedy/prefill rows (float [rows][vocab]) and hidden rows. */
int qb_debug_last_logits(qb_ctx *ctx, qb_batch *b, float *host_out, uint32_t max_rows, uint32_t *rows_out);
/* Drafts of the last qb_mtp_draft / qb_mtp_force_drafts: int32 [n_seqs][k] (test aid, syncs). */
int qb_debug_last_drafts(qb_ctx *ctx, qb_batch *b, int32_t *host_out);
/* Per-launch CUDA-event timing of the Q8 GEMM kernels on the context stream (the reference's
 * per-op timing, src/qwen_executor.cpp:1788-1804, without its synchronise-per-op): enable, run,
 * then read the summed duration, the summed algorithmic bytes and the number of launches. */
int qb_prof_enable(qb_ctx *ctx, int on);
int qb_prof_summary(qb_ctx *ctx, double *total_ms, double *total_bytes, int64_t *launches);
/* Launch trace: while enabled an event is recorded after every kernel launch of the library; the
 * summary gives, per kernel name, the number of launches and the summed time between its event and
 * the preceding one, as "name<TAB>launches<TAB>microseconds" lines. */
int qb_trace_enable(qb_ctx *ctx, int on);
int qb_trace_summary(qb_ctx *ctx, char *buf, size_t buf_bytes);
/* ---- tensor-parallel FFN pair over NVLink peer memory ------------------------------------------------
 * The one sharded case of the path: the FFN dimension F is split over `world` GPUs (one process each).
 * Rank r holds gate/up rows [r*F/world, (r+1)*F/world) fused as [gate_r; up_r] (2*f_shard x n_in) and the
 * matching K slice of down (n_out x f_shard).  qb_tp_ffn = quantise x, gate/up GEMM, SwiGLU, down GEMM
 * whose epilogue stores its split partials into every rank's receive area and signals (from 32 rows on:
 * a rank adds its own segments first and pushes one slice), then a reduce that adds, in rank order, each
 * rank's sum over its segments: every rank ends with the same bits, sum_r (sum_s partial[r][s]), whatever
 * the row count.  Stands where the reference would place ncclAllReduce after a row-parallel
 * q8_0_matmul (the reference itself runs one GPU per model replica and has no such call).
 *
 * Receive areas: one allocation of qb_tp_recv_bytes() per GPU (qb_malloc), 256-byte aligned, passed as
 * recv_ptrs[world] with this rank's own at [rank] and the peers' as mapped by qb_ipc_open.  All ranks
 * must have created their group (which zeroes its own arrival counters) before any rank pushes, and
 * must call push/reduce with the same M in the same order.  A reduce whose peers never arrive gives up
 * after about a second; the next qb_synchronize reports it. */
typedef struct qb_tp_group qb_tp_group;
size_t qb_tp_recv_bytes(uint32_t world, uint32_t max_rows, uint32_t n_out, uint32_t k_shard);
int qb_tp_group_create(qb_ctx *ctx, uint32_t rank, uint32_t world, void *const *recv_ptrs, uint32_t max_rows,
                       uint32_t n_in, uint32_t f_shard, uint32_t n_out, qb_tp_group **out);
int qb_tp_group_destroy(qb_ctx *ctx, qb_tp_group *g);
int qb_tp_ffn_push(qb_ctx *ctx, qb_tp_group *g, const qb_weight *gate_up_shard, const qb_weight *down_shard,
                   const float *x_dev, uint32_t M);
int qb_tp_ffn_reduce(qb_ctx *ctx, qb_tp_group *g, uint32_t M, float *y_dev, uint32_t y_stride);
int qb_tp_ffn(qb_ctx *ctx, qb_tp_group *g, const qb_weight *gate_up_shard, const qb_weight *down_shard,
              const float *x_dev, uint32_t M, float *y_dev, uint32_t y_stride);
/* The sharded FFN inside the step (the latency configuration: one request served by `world` GPUs).
 * qb_model_create_synth_tp: the seeded model with every FFN pair sharded as above (rank's gate/up rows and down columns
 * are windows of the same seeded tensors, everything else replicated).  qb_batch_set_tp: the batch's forward passes run
 * their FFN blocks through `group` (sized for qb_batch_max_rows rows); every rank runs the same calls on the same tokens
 * and all get the same bits, so a speculative run still equals the greedy run of the same rank count exactly. */
int qb_model_create_synth_tp(qb_ctx *ctx, const qb_model_config *cfg, uint64_t seed, uint32_t rank, uint32_t world, qb_model **out);
int qb_batch_set_tp(qb_ctx *ctx, qb_batch *b, qb_tp_group *group);
uint32_t qb_batch_max_rows(const qb_batch *b);
/* CUDA IPC: export a qb_malloc'ed buffer as a 64-byte handle another process opens (peer access is
 * enabled on open). */
int qb_ipc_export(qb_ctx *ctx, const void *dev_ptr, void *handle64);
int qb_ipc_open(qb_ctx *ctx, const void *handle64, void **dev_ptr_out);
int qb_ipc_close(qb_ctx *ctx, void *dev_ptr);

/* Device timeline of the tensor-core GEMM launches: after qb_debug_timeline_enable(ctx, n) the next n such
 * launches record, per CTA, {entry, dependency wait passed, exit} in nanoseconds of the GPU's global timer
 * and the SM id (4 uint64 per CTA, 320 CTA slots per launch).  qb_debug_timeline_read copies the recorded
 * launches out: out = uint64 [n][320][4], grids[i] = CTAs of launch i, bytes[i] = its algorithmic bytes
 * (weight records + int8 activations and scales + fp32 partials).  enable(ctx, 0) frees the buffer. */
int qb_debug_timeline_enable(qb_ctx *ctx, uint32_t max_launches);
int qb_debug_timeline_read(qb_ctx *ctx, uint64_t *out, uint32_t *grids, double *bytes, uint32_t max_launches,
                           uint32_t *n_out);
/* Number of kernels this library launched on the context since creation. */
int64_t qb_launch_count(qb_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* QW3B200_H */
