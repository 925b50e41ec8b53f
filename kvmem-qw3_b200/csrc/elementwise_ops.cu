// Op-level entry points of the small element-wise / per-head operators of the DeviceBackend interface
// (include/qw3/device_backend.hpp:624-664, 948-1119, 2218-2262, 2456-2497, 2646-2695).  The fused step does not launch
// these (its norms, RoPE, K/V append and gating live inside the attention / DeltaNet / norm_quant kernels); they exist
// so that a DeviceBackend subclass over this library answers every virtual the reference's executor calls one by one.
// All are memory-bound streaming kernels over a few rows; grid = ceil(n / 256) or one CTA per (row, head).
#include "qb_internal.h"

namespace {

__global__ void add_kernel(float *out, const float *a, const float *b, uint64_t n) {
    QB_PDL_ENTER();
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}
__global__ void mul_kernel(float *out, const float *a, const float *b, uint64_t n) {
    QB_PDL_ENTER();
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] * b[i];
}
// silu_kernel / silu_mul_kernel (src/kernels_cuda.cu:1894-1903): x / (1 + exp(-x)) [* up]
__global__ void silu_kernel(float *out, const float *x, uint64_t n) {
    QB_PDL_ENTER();
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fdiv_rn(x[i], 1.0f + expf(-x[i]));
}
__global__ void silu_mul_kernel(float *out, const float *gate, const float *up, uint64_t n) {
    QB_PDL_ENTER();
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = qb_swiglu(gate[i], up[i]);
}

// rmsnorm_per_head_kernel (src/kernels_cuda.cu:4622-4645): one warp per (row, unit); y = x * rsqrt(mean(x^2) + eps) * w.
__global__ void rmsnorm_per_head_kernel(float *x, const float *w, uint32_t batch_stride, uint32_t n_units, uint32_t per_unit_stride,
                                        uint32_t head_dim, float eps) {
    QB_PDL_ENTER();
    const uint32_t b = blockIdx.x, unit = blockIdx.y * (blockDim.x / 32) + threadIdx.x / 32, lane = threadIdx.x & 31;
    if (unit >= n_units) return;
    float *p = x + (size_t)b * batch_stride + (size_t)unit * per_unit_stride;
    float ss = 0.0f;
    for (uint32_t i = lane; i < head_dim; i += 32) ss += p[i] * p[i];
    ss = warp_sum(ss);
    const float sc = rsqrtf(ss / (float)head_dim + eps);
    for (uint32_t i = lane; i < head_dim; i += 32) p[i] = p[i] * sc * w[i];
}

// rope_partial_kernel / rope_partial_positions_kernel (src/kernels_cuda.cu:4697-4719, 4779-4799): the first rope_dim
// elements of every unit, pairs (i, i + rope_dim/2), angle = pos * theta^(-2i/rope_dim).
__global__ void rope_partial_kernel(float *x, uint32_t n_units, uint32_t per_unit_stride, uint32_t rope_dim, uint32_t base_pos,
                                    const int32_t *positions, uint32_t batch_stride, float theta) {
    QB_PDL_ENTER();
    const uint32_t b = blockIdx.x, unit = blockIdx.y, i = threadIdx.x, half = rope_dim / 2;
    if (unit >= n_units || i >= half) return;
    float *base = x + (size_t)b * batch_stride + (size_t)unit * per_unit_stride;
    const float inv_freq = powf(theta, -2.0f * (float)i / (float)rope_dim);
    const float pos = positions ? (float)positions[b] : (float)(base_pos + b);
    float s, c;
    sincosf(pos * inv_freq, &s, &c);
    const float x0 = base[i], x1 = base[i + half];
    base[i] = x0 * c - x1 * s;
    base[i + half] = x0 * s + x1 * c;
}

// kv_append_batch_f16 / kv_append_batch_paged (src/kernels_cuda.cu:8921-8969): row b at position base_pos + b goes to
// slot pos (dense) or page_indices[pos / page_size] * page_size + pos % page_size, fp32 -> fp16.
__global__ void kv_append_kernel(__half *cache, const float *src, uint32_t base_pos, uint32_t per_pos_size, const int32_t *pages,
                                 uint32_t n_pages, uint32_t page_size, int *err_flag) {
    QB_PDL_ENTER();
    const uint32_t b = blockIdx.x, pos = base_pos + b;
    size_t slot = pos;
    if (pages) {
        const uint32_t pg = pos / page_size;
        if (pg >= n_pages) { if (threadIdx.x == 0) atomicExch(err_flag, 3001); return; }      // recorded, not dereferenced
        slot = (size_t)pages[pg] * page_size + pos % page_size;
    }
    for (uint32_t i = threadIdx.x; i < per_pos_size; i += blockDim.x)
        cache[slot * per_pos_size + i] = __float2half_rn(src[(size_t)b * per_pos_size + i]);
}

// apply_attn_gate_kernel (src/kernels_cuda.cu:9448-9465): out[b][h][d] *= sigmoid(q[b][h * q_stride + head_dim + d]).
__global__ void attn_gate_kernel(float *out, const float *q, uint32_t q_stride, uint32_t n_heads, uint32_t head_dim, uint32_t bsq,
                                 uint32_t bso) {
    QB_PDL_ENTER();
    const uint32_t b = blockIdx.x;
    const uint32_t i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= n_heads * head_dim) return;
    const uint32_t head = i / head_dim, d = i % head_dim;
    const float gate = q[(size_t)b * bsq + (size_t)head * q_stride + head_dim + d];
    out[(size_t)b * bso + i] *= __fdiv_rn(1.0f, 1.0f + expf(-gate));
}

// pack_mtp_prefix_hinputs / pack_mtp_concat (include/qw3/device_backend.hpp:2646-2695): row copies.
__global__ void pack_prefix_kernel(float *dst, const float *first, const float *h_batch, uint32_t batch, uint32_t h_stride) {
    QB_PDL_ENTER();
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)batch * h_stride) return;
    const uint32_t row = (uint32_t)(idx / h_stride), col = (uint32_t)(idx % h_stride);
    dst[idx] = row == 0 ? first[col] : h_batch[(size_t)(row - 1) * h_stride + col];
}
__global__ void pack_concat_kernel(float *dst, const float *left, const float *right, uint32_t batch, uint32_t ls, uint32_t rs,
                                   uint32_t cs, uint32_t width) {
    QB_PDL_ENTER();
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)batch * 2 * width) return;
    const uint32_t row = (uint32_t)(idx / (2 * width)), col = (uint32_t)(idx % (2 * width));
    dst[(size_t)row * cs + col] = col < width ? left[(size_t)row * ls + col] : right[(size_t)row * rs + col - width];
}

template <typename K, typename... A>
int launch1d(qb_ctx *ctx, const char *name, K kernel, uint64_t n, A... args) {
    if (n == 0) return QB_OK;
    QB_CUDA(qb_launch_pdl(ctx->stream, kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, args...));
    QB_LAUNCHED(ctx, name);
    return QB_OK;
}

}  // namespace

extern "C" int qb_add(qb_ctx *ctx, float *out, const float *a, const float *b, uint64_t n) {
    QB_REQUIRE(ctx && out && a && b, "qb_add: null argument");
    return launch1d(ctx, "add_kernel", add_kernel, n, out, a, b, n);
}
extern "C" int qb_mul(qb_ctx *ctx, float *out, const float *a, const float *b, uint64_t n) {
    QB_REQUIRE(ctx && out && a && b, "qb_mul: null argument");
    return launch1d(ctx, "mul_kernel", mul_kernel, n, out, a, b, n);
}
extern "C" int qb_silu(qb_ctx *ctx, float *out, const float *x, uint64_t n) {
    QB_REQUIRE(ctx && out && x, "qb_silu: null argument");
    return launch1d(ctx, "silu_kernel", silu_kernel, n, out, x, n);
}
extern "C" int qb_silu_mul(qb_ctx *ctx, float *out, const float *gate, const float *up, uint64_t n) {
    QB_REQUIRE(ctx && out && gate && up, "qb_silu_mul: null argument");
    return launch1d(ctx, "silu_mul_kernel", silu_mul_kernel, n, out, gate, up, n);
}

extern "C" int qb_rmsnorm_per_head(qb_ctx *ctx, float *x, const float *w, uint32_t batch, uint32_t batch_stride, uint32_t n_units,
                                   uint32_t per_unit_stride, uint32_t head_dim, float eps) {
    QB_REQUIRE(ctx && x && w && batch > 0 && n_units > 0 && head_dim > 0, "qb_rmsnorm_per_head: bad arguments");
    QB_CUDA(qb_launch_pdl(ctx->stream, rmsnorm_per_head_kernel, dim3(batch, (n_units + 3) / 4), dim3(128), (size_t)0, x, w, batch_stride, n_units,
                          per_unit_stride, head_dim, eps));
    QB_LAUNCHED(ctx, "rmsnorm_per_head_kernel");
    return QB_OK;
}

extern "C" int qb_rope_partial(qb_ctx *ctx, float *x, uint32_t batch, uint32_t batch_stride, uint32_t n_units, uint32_t per_unit_stride,
                               uint32_t rope_dim, uint32_t base_pos, const int32_t *positions_dev, float theta) {
    QB_REQUIRE(ctx && x && batch > 0 && n_units > 0, "qb_rope_partial: bad arguments");
    QB_REQUIRE(rope_dim >= 2 && rope_dim % 2 == 0 && rope_dim / 2 <= 1024, "qb_rope_partial: rope_dim %u must be even and <= 2048", rope_dim);
    QB_CUDA(qb_launch_pdl(ctx->stream, rope_partial_kernel, dim3(batch, n_units), dim3(((rope_dim / 2) + 31) / 32 * 32), (size_t)0, x, n_units,
                          per_unit_stride, rope_dim, base_pos, positions_dev, batch_stride, theta));
    QB_LAUNCHED(ctx, "rope_partial_kernel");
    return QB_OK;
}

extern "C" int qb_kv_append(qb_ctx *ctx, void *cache_f16, const float *src, uint32_t base_pos, uint32_t per_pos_size, uint32_t batch,
                            const int32_t *page_indices_dev, uint32_t n_pages, uint32_t page_size) {
    QB_REQUIRE(ctx && cache_f16 && src && batch > 0 && per_pos_size > 0, "qb_kv_append: bad arguments");
    QB_REQUIRE(!page_indices_dev || (page_size > 0 && (base_pos + batch - 1) / page_size < n_pages), "qb_kv_append: positions %u..%u beyond %u pages of %u",
               base_pos, base_pos + batch - 1, n_pages, page_size);
    QB_CUDA(qb_launch_pdl(ctx->stream, kv_append_kernel, dim3(batch), dim3(256), (size_t)0, (__half *)cache_f16, src, base_pos, per_pos_size,
                          page_indices_dev, n_pages, page_size, ctx->err_flag_dev));
    QB_LAUNCHED(ctx, "kv_append_kernel");
    return QB_OK;
}

extern "C" int qb_apply_attn_gate(qb_ctx *ctx, float *out, const float *q, uint32_t q_stride, uint32_t batch, uint32_t batch_stride_q,
                                  uint32_t batch_stride_out, uint32_t n_heads, uint32_t head_dim) {
    QB_REQUIRE(ctx && out && q && batch > 0, "qb_apply_attn_gate: bad arguments");
    QB_CUDA(qb_launch_pdl(ctx->stream, attn_gate_kernel, dim3(batch, (n_heads * head_dim + 255) / 256), dim3(256), (size_t)0, out, q, q_stride, n_heads,
                          head_dim, batch_stride_q, batch_stride_out));
    QB_LAUNCHED(ctx, "attn_gate_kernel");
    return QB_OK;
}

extern "C" int qb_pack_mtp_prefix_hinputs(qb_ctx *ctx, float *dst, const float *first_h, const float *h_batch, uint32_t batch, uint32_t h_stride) {
    QB_REQUIRE(ctx && dst && first_h && (batch <= 1 || h_batch), "qb_pack_mtp_prefix_hinputs: null argument");
    return launch1d(ctx, "pack_prefix_kernel", pack_prefix_kernel, (uint64_t)batch * h_stride, dst, first_h, h_batch, batch, h_stride);
}
extern "C" int qb_pack_mtp_concat(qb_ctx *ctx, float *dst, const float *left, const float *right, uint32_t batch, uint32_t left_stride,
                                  uint32_t right_stride, uint32_t concat_stride, uint32_t width) {
    QB_REQUIRE(ctx && dst && left && right, "qb_pack_mtp_concat: null argument");
    return launch1d(ctx, "pack_concat_kernel", pack_concat_kernel, (uint64_t)batch * 2 * width, dst, left, right, batch, left_stride, right_stride,
                    concat_stride, width);
}
