// B200DeviceBackend: the reference's DeviceBackend interface (include/qw3/device_backend.hpp:88-2696) implemented on the
// C ABI of libqw3b200 (include/qw3b200.h).  This is the file a kvmem-qw3 maintainer adds to the reference tree to make the
// B200 library a backend of QwenExecutor; it is compiled against the reference's own header and contains no CUDA code.
//
//   std::unique_ptr<qw3::DeviceBackend> qw3::make_b200_device_backend(int device);
//
// With -DQW3B200_PROVIDE_CUDA_FACTORY the file also defines make_cuda_device_backend / cuda_device_backend_available
// (include/qw3/device_backend.hpp:2744), so linking it in place of src/kernels_cuda.cu swaps the backend without touching
// the executor.
//
// Conventions carried over from the reference backend (src/kernels_cuda.cu:9564-9810): one stream per backend, every
// operator enqueued in call order, DeviceStatus::message points at thread-local storage, allocation failures throw from
// the tensor constructors, an operator this library does not cover returns {false, "..."} so that the executor takes its
// unfused fallback (src/qwen_executor.cpp:5550-5553).  Activations are fp32 (the reference's QW3_Q8_BF16_MAIN=0 mode);
// K/V caches are fp16.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "qw3/device_backend.hpp"
#include "qw3b200.h"

namespace qw3 {
namespace {

thread_local char g_msg[320];

DeviceStatus fail(const char *what) {
    std::snprintf(g_msg, sizeof(g_msg), "b200: %s", what ? what : "unknown");
    return {false, g_msg};
}
DeviceStatus st(int rc) {
    if (rc == QB_OK) return {};
    std::snprintf(g_msg, sizeof(g_msg), "b200: %s", qb_last_error());
    return {false, g_msg};
}

struct B200Tensor final : DeviceTensor {
    qb_ctx *ctx = nullptr;
    void *ptr = nullptr;
    bool owns = false;
    B200Tensor(qb_ctx *c, uint64_t n, uint32_t esz, DeviceTensorDType dt) : ctx(c), owns(true) {
        count = n; elem_size = esz; dtype = dt;
        if (qb_malloc(ctx, (size_t)n * esz, &ptr) != QB_OK) throw std::runtime_error(std::string("b200 tensor allocation failed: ") + qb_last_error());
        qb_memset(ctx, ptr, 0, (size_t)n * esz);
    }
    B200Tensor(qb_ctx *c, void *p, uint64_t n, uint32_t esz, DeviceTensorDType dt) : ctx(c), ptr(p), owns(false) { count = n; elem_size = esz; dtype = dt; }
    ~B200Tensor() override { if (owns && ptr) qb_free(ctx, ptr); }
};

struct B200Weight final : DeviceWeight {
    qb_ctx *ctx = nullptr;
    qb_weight *q8 = nullptr;        // Q8_0 matrix in the library's record layout
    float *f32 = nullptr;           // fp32 vector / small tensor on the device
    ~B200Weight() override {
        if (q8) qb_weight_free(ctx, q8);
        if (f32) qb_free(ctx, f32);
    }
};

struct B200ArgmaxBuffer final : DeviceArgmaxBuffer {
    qb_ctx *ctx = nullptr;
    int32_t *tok = nullptr;
    float *val = nullptr;
    ~B200ArgmaxBuffer() override {
        if (tok) qb_free(ctx, tok);
        if (val) qb_free(ctx, val);
    }
};

inline float *F(DeviceTensor &t) { return static_cast<float *>(static_cast<B200Tensor &>(t).ptr); }
inline const float *F(const DeviceTensor &t) { return static_cast<const float *>(static_cast<const B200Tensor &>(t).ptr); }
inline void *P(const DeviceTensor &t) { return static_cast<const B200Tensor &>(t).ptr; }
inline const B200Weight &W(const DeviceWeight &w) { return static_cast<const B200Weight &>(w); }
inline bool is_f32(const DeviceTensor &t) { return t.elem_size == 4 && t.dtype == DeviceTensorDType::F32; }

class B200DeviceBackend final : public DeviceBackend {
public:
    explicit B200DeviceBackend(int device) {
        if (qb_create(device, &ctx_) != QB_OK) throw std::runtime_error(std::string("b200 backend: ") + qb_last_error());
    }
    ~B200DeviceBackend() override {
        if (ident_) qb_free(ctx_, ident_);
        if (pos_) qb_free(ctx_, pos_);
        if (am_tok_) qb_free(ctx_, am_tok_);
        if (am_val_) qb_free(ctx_, am_val_);
        if (tmp_) qb_free(ctx_, tmp_);
        if (ids_) qb_free(ctx_, ids_);
        qb_destroy(ctx_);
    }

    const char *name() const override { return "b200"; }
    DeviceStatus begin() override { return {}; }
    DeviceStatus end() override { return st(qb_synchronize(ctx_)); }
    DeviceStatus synchronize() override { return st(qb_synchronize(ctx_)); }

    // ---- tensors -------------------------------------------------------------------------------------------------
    std::unique_ptr<DeviceTensor> tensor_f32(uint64_t count, const char *) override {
        return std::make_unique<B200Tensor>(ctx_, count, 4u, DeviceTensorDType::F32);
    }
    std::unique_ptr<DeviceTensor> tensor_f16(uint64_t count, const char *) override {
        return std::make_unique<B200Tensor>(ctx_, count, 2u, DeviceTensorDType::F16);
    }
    std::unique_ptr<DeviceTensor> tensor_i32(uint64_t count, const char *) override {
        return std::make_unique<B200Tensor>(ctx_, count, 4u, DeviceTensorDType::I32);
    }
    std::unique_ptr<DeviceTensor> scratch_f32(uint64_t count, const char *label) override { return tensor_f32(count, label); }
    std::unique_ptr<DeviceTensor> scratch_like(const DeviceTensor &, uint64_t count, const char *label) override { return tensor_f32(count, label); }
    bool supports_tensor_views() const override { return true; }
    std::unique_ptr<DeviceTensor> tensor_view(DeviceTensor &storage, uint64_t byte_offset, uint64_t count, uint32_t elem_size,
                                              DeviceTensorDType dtype, const char *) override {
        if (byte_offset + count * elem_size > storage.count * storage.elem_size) throw std::runtime_error("b200 tensor_view out of range");
        return std::make_unique<B200Tensor>(ctx_, static_cast<char *>(P(storage)) + byte_offset, count, elem_size, dtype);
    }
    DeviceStatus zero_tensor(DeviceTensor &x) override { return st(qb_memset(ctx_, P(x), 0, (size_t)x.count * x.elem_size)); }

    // ---- copies (element counts and offsets, device_backend.hpp:148, 2454, 2514-2644) ----------------------------------
    DeviceStatus copy_to_host(const DeviceTensor &x, float *host, uint64_t offset, uint64_t count) override {
        if (!is_f32(x) || offset + count > x.count) return fail("copy_to_host: range or dtype");
        return st(qb_memcpy_d2h(ctx_, host, F(x) + offset, (size_t)count * 4));
    }
    DeviceStatus copy_i32_from_host(DeviceTensor &dst, uint64_t dst_offset, const int32_t *src, uint64_t count) override {
        if (dst.elem_size != 4 || dst_offset + count > dst.count) return fail("copy_i32_from_host: range");
        return st(qb_memcpy_h2d(ctx_, static_cast<int32_t *>(P(dst)) + dst_offset, src, (size_t)count * 4));
    }
    DeviceStatus copy_bytes_from_host(DeviceTensor &x, uint64_t byte_offset, const void *host, uint64_t byte_count) override {
        if (byte_offset + byte_count > x.count * x.elem_size) return fail("copy_bytes_from_host: range");
        return st(qb_memcpy_h2d(ctx_, static_cast<char *>(P(x)) + byte_offset, host, (size_t)byte_count));
    }
    DeviceStatus copy_bytes_to_host(const DeviceTensor &x, void *host, uint64_t byte_offset, uint64_t byte_count) override {
        if (byte_offset + byte_count > x.count * x.elem_size) return fail("copy_bytes_to_host: range");
        return st(qb_memcpy_d2h(ctx_, host, static_cast<const char *>(P(x)) + byte_offset, (size_t)byte_count));
    }
    DeviceStatus copy_d2d(DeviceTensor &dst, const DeviceTensor &src, uint64_t src_offset, uint64_t count) override {
        return copy_d2d_into(dst, 0, src, src_offset, count);
    }
    DeviceStatus copy_d2d_into(DeviceTensor &dst, uint64_t dst_offset, const DeviceTensor &src, uint64_t src_offset, uint64_t count) override {
        if (dst.elem_size != src.elem_size) return fail("copy_d2d: element sizes differ");
        if (dst_offset + count > dst.count || src_offset + count > src.count) return fail("copy_d2d: range");
        const size_t es = dst.elem_size;
        return st(qb_memcpy_d2d(ctx_, static_cast<char *>(P(dst)) + dst_offset * es, static_cast<const char *>(P(src)) + src_offset * es, (size_t)count * es));
    }

    // ---- weights ---------------------------------------------------------------------------------------------------
    std::unique_ptr<DeviceWeight> weight_f32(const float *data, uint64_t count, const char *) override {
        auto w = std::make_unique<B200Weight>();
        w->ctx = ctx_; w->rows = 1; w->cols = count; w->format = DeviceWeightFormat::F32;
        void *p = nullptr;
        if (qb_malloc(ctx_, (size_t)count * 4, &p) != QB_OK || qb_memcpy_h2d(ctx_, p, data, (size_t)count * 4) != QB_OK)
            throw std::runtime_error(std::string("b200 weight_f32: ") + qb_last_error());
        w->f32 = static_cast<float *>(p);
        return w;
    }
    std::unique_ptr<DeviceWeight> weight_q8_0(const void *data, uint64_t rows, uint64_t cols, const char *label) override {
        auto w = std::make_unique<B200Weight>();
        w->ctx = ctx_; w->rows = rows; w->cols = cols; w->format = DeviceWeightFormat::Q8_0;
        if (qb_weight_q8_0(ctx_, data, (uint32_t)rows, (uint32_t)cols, &w->q8) != QB_OK)
            throw std::runtime_error(std::string("b200 weight_q8_0(") + (label ? label : "") + "): " + qb_last_error());
        return w;
    }

    // ---- embedding rows ----------------------------------------------------------------------------------------------
    DeviceStatus q8_0_get_row(DeviceTensor &out, const DeviceWeight &weight, uint64_t row) override {
        const uint64_t r[1] = {row};
        return q8_0_get_rows_batch(out, weight, r, 1);
    }
    DeviceStatus q8_0_get_rows_batch(DeviceTensor &out, const DeviceWeight &weight, const uint64_t *rows, uint32_t batch) override {
        const B200Weight &w = W(weight);
        if (!w.q8 || !is_f32(out) || out.count < (uint64_t)batch * w.cols) return fail("q8_0_get_rows_batch: arguments");
        std::vector<int32_t> ids(batch);
        for (uint32_t i = 0; i < batch; ++i) {
            if (rows[i] >= w.rows) return fail("q8_0_get_rows_batch: row out of range");
            ids[i] = (int32_t)rows[i];
        }
        int32_t *dev = nullptr;
        if (DeviceStatus s = ids_buffer(batch, &dev); !s.ok) return s;
        if (int rc = qb_memcpy_h2d(ctx_, dev, ids.data(), (size_t)batch * 4); rc != QB_OK) return st(rc);
        return st(qb_q8_0_get_rows(ctx_, w.q8, dev, batch, F(out), (uint32_t)w.cols));
    }
    DeviceStatus q8_0_get_row_from_argmax(DeviceTensor &out, const DeviceWeight &weight, const DeviceArgmaxBuffer &argmaxes, uint32_t index) override {
        const B200Weight &w = W(weight);
        const auto &ab = static_cast<const B200ArgmaxBuffer &>(argmaxes);
        if (!w.q8 || index >= ab.count || out.count < w.cols) return fail("q8_0_get_row_from_argmax: arguments");
        return st(qb_q8_0_get_rows(ctx_, w.q8, ab.tok + index, 1, F(out), (uint32_t)w.cols));      // the token id never leaves the device
    }

    // ---- Q8_0 products ---------------------------------------------------------------------------------------------------
    DeviceStatus q8_0_matmul(DeviceTensor &out, const DeviceWeight &weight, const DeviceTensor &x, uint32_t batch, uint32_t in_stride,
                             uint32_t out_stride) override {
        const B200Weight &w = W(weight);
        if (!w.q8 || !is_f32(out) || !is_f32(x)) return fail("q8_0_matmul: needs a Q8_0 weight and fp32 tensors");
        if (x.count < (uint64_t)(batch - 1) * in_stride + w.cols || out.count < (uint64_t)(batch - 1) * out_stride + w.rows) return fail("q8_0_matmul: range");
        return st(qb_q8_0_matmul(ctx_, w.q8, F(x), batch, in_stride, F(out), out_stride, 0, 0));
    }
    DeviceStatus q8_0_matvec(DeviceTensor &out, const DeviceWeight &weight, const DeviceTensor &x) override {
        return q8_0_matmul(out, weight, x, 1, (uint32_t)W(weight).cols, (uint32_t)W(weight).rows);
    }
    DeviceStatus q8_0_matvec_add(DeviceTensor &accum, const DeviceWeight &weight, const DeviceTensor &x) override {
        float *tmp = nullptr;
        if (DeviceStatus s = tmp_buffer(W(weight).rows, &tmp); !s.ok) return s;
        B200Tensor t(ctx_, tmp, W(weight).rows, 4u, DeviceTensorDType::F32);
        if (DeviceStatus s = q8_0_matvec(t, weight, x); !s.ok) return s;
        return st(qb_add(ctx_, F(accum), F(accum), tmp, W(weight).rows));
    }
    DeviceStatus q8_0_matvec_fanout(DeviceTensor *const *outs, const DeviceWeight *const *weights, uint32_t n, const DeviceTensor &x) override {
        for (uint32_t i = 0; i < n; ++i)
            if (DeviceStatus s = q8_0_matvec(*outs[i], *weights[i], x); !s.ok) return s;
        return {};
    }
    DeviceStatus q8_0_matmul_fanout(DeviceTensor *const *outs, const DeviceWeight *const *weights, const uint32_t *out_strides, uint32_t n,
                                    const DeviceTensor &x, uint32_t batch, uint32_t in_stride) override {
        for (uint32_t i = 0; i < n; ++i)
            if (DeviceStatus s = q8_0_matmul(*outs[i], *weights[i], x, batch, in_stride, out_strides[i]); !s.ok) return s;
        return {};
    }
    DeviceStatus q8_0_matmul_add(DeviceTensor &out, const DeviceTensor &residual, DeviceTensor &matmul_tmp, const DeviceWeight &weight,
                                 const DeviceTensor &x, uint32_t batch, uint32_t in_stride, uint32_t out_stride) override {
        if (DeviceStatus s = q8_0_matmul(matmul_tmp, weight, x, batch, in_stride, out_stride); !s.ok) return s;
        return st(qb_add(ctx_, F(out), F(residual), F(matmul_tmp), (uint64_t)(batch - 1) * out_stride + W(weight).rows));
    }
    DeviceStatus q8_0_matvec_silu_mul(DeviceTensor &out, const DeviceWeight &weight_gate, const DeviceWeight &weight_up, const DeviceTensor &x) override {
        return q8_0_matmul_silu_mul(out, weight_gate, weight_up, x, 1, (uint32_t)W(weight_gate).cols, (uint32_t)W(weight_gate).rows);
    }
    DeviceStatus q8_0_matmul_silu_mul(DeviceTensor &out, const DeviceWeight &weight_gate, const DeviceWeight &weight_up, const DeviceTensor &x,
                                      uint32_t batch, uint32_t in_stride, uint32_t out_stride) override {
        const uint64_t F_ = W(weight_gate).rows;
        if (out_stride != F_) return fail("q8_0_matmul_silu_mul: out_stride must equal the FFN dimension");
        float *tmp = nullptr;
        if (DeviceStatus s = tmp_buffer((uint64_t)batch * F_, &tmp); !s.ok) return s;
        B200Tensor up(ctx_, tmp, (uint64_t)batch * F_, 4u, DeviceTensorDType::F32);
        if (DeviceStatus s = q8_0_matmul(out, weight_gate, x, batch, in_stride, out_stride); !s.ok) return s;
        if (DeviceStatus s = q8_0_matmul(up, weight_up, x, batch, in_stride, (uint32_t)F_); !s.ok) return s;
        return st(qb_silu_mul(ctx_, F(out), F(out), tmp, (uint64_t)batch * F_));
    }
    DeviceStatus rms_norm_q8_0_matmul_fanout(DeviceTensor &normalized, DeviceTensor *const *outs, const DeviceWeight *const *weights,
                                             const uint32_t *out_strides, uint32_t fanout, const DeviceTensor &x, const DeviceWeight &norm_weight,
                                             uint32_t batch, uint32_t in_stride, float eps) override {
        const uint32_t n = (uint32_t)W(norm_weight).cols;
        if (in_stride != n) return fail("rms_norm_q8_0_matmul_fanout: in_stride must equal the row length");
        if (DeviceStatus s = rms_norm_batch(normalized, x, norm_weight, batch, n, eps); !s.ok) return s;
        return q8_0_matmul_fanout(outs, weights, out_strides, fanout, normalized, batch, in_stride);
    }

    // ---- norms and element-wise --------------------------------------------------------------------------------------------
    DeviceStatus rms_norm(DeviceTensor &out, const DeviceTensor &x, const DeviceWeight &weight, float eps) override {
        return rms_norm_batch(out, x, weight, 1, (uint32_t)W(weight).cols, eps);
    }
    DeviceStatus rms_norm_batch(DeviceTensor &out, const DeviceTensor &x, const DeviceWeight &weight, uint32_t batch, uint32_t n, float eps) override {
        if (!W(weight).f32 || !is_f32(out) || !is_f32(x) || x.count < (uint64_t)batch * n || out.count < (uint64_t)batch * n) return fail("rms_norm_batch: arguments");
        return st(qb_rms_norm(ctx_, F(x), W(weight).f32, batch, n, n, eps, F(out)));
    }
    DeviceStatus add(DeviceTensor &out, const DeviceTensor &a, const DeviceTensor &b) override { return add_n(out, a, b, out.count); }
    DeviceStatus add_n(DeviceTensor &out, const DeviceTensor &a, const DeviceTensor &b, uint64_t count) override {
        if (count > out.count || count > a.count || count > b.count) return fail("add_n: range");
        return st(qb_add(ctx_, F(out), F(a), F(b), count));
    }
    DeviceStatus silu(DeviceTensor &out, const DeviceTensor &x) override { return st(qb_silu(ctx_, F(out), F(x), out.count)); }
    DeviceStatus mul(DeviceTensor &out, const DeviceTensor &a, const DeviceTensor &b) override { return st(qb_mul(ctx_, F(out), F(a), F(b), out.count)); }
    DeviceStatus silu_mul(DeviceTensor &out, const DeviceTensor &gate, const DeviceTensor &up) override { return silu_mul_n(out, gate, up, out.count); }
    DeviceStatus silu_mul_n(DeviceTensor &out, const DeviceTensor &gate, const DeviceTensor &up, uint64_t count) override {
        if (count > out.count || count > gate.count || count > up.count) return fail("silu_mul_n: range");
        return st(qb_silu_mul(ctx_, F(out), F(gate), F(up), count));
    }

    // ---- attention preparation -------------------------------------------------------------------------------------------
    DeviceStatus rmsnorm_per_head(DeviceTensor &x, const DeviceWeight &weight, uint32_t n_units, uint32_t per_unit_stride, uint32_t head_dim,
                                  float eps) override {
        return rmsnorm_per_head_batch(x, weight, 1, 0, n_units, per_unit_stride, head_dim, eps);
    }
    DeviceStatus rmsnorm_per_head_batch(DeviceTensor &x, const DeviceWeight &weight, uint32_t batch, uint32_t batch_stride, uint32_t n_units,
                                        uint32_t per_unit_stride, uint32_t head_dim, float eps) override {
        if (!W(weight).f32 || W(weight).cols < head_dim) return fail("rmsnorm_per_head: gain vector");
        return st(qb_rmsnorm_per_head(ctx_, F(x), W(weight).f32, batch, batch_stride, n_units, per_unit_stride, head_dim, eps));
    }
    DeviceStatus rope_partial(DeviceTensor &x, uint32_t n_units, uint32_t per_unit_stride, uint32_t rope_dim, uint32_t pos, float theta) override {
        return st(qb_rope_partial(ctx_, F(x), 1, 0, n_units, per_unit_stride, rope_dim, pos, nullptr, theta));
    }
    DeviceStatus rope_partial_batch(DeviceTensor &x, uint32_t batch, uint32_t batch_stride, uint32_t n_units, uint32_t per_unit_stride,
                                    uint32_t rope_dim, uint32_t base_pos, float theta) override {
        return st(qb_rope_partial(ctx_, F(x), batch, batch_stride, n_units, per_unit_stride, rope_dim, base_pos, nullptr, theta));
    }
    DeviceStatus rope_partial_batch_positions(DeviceTensor &x, uint32_t batch, uint32_t batch_stride, uint32_t n_units, uint32_t per_unit_stride,
                                              uint32_t rope_dim, const DeviceTensor &positions, float theta) override {
        if (positions.count < batch) return fail("rope_partial_batch_positions: positions");
        return st(qb_rope_partial(ctx_, F(x), batch, batch_stride, n_units, per_unit_stride, rope_dim, 0, static_cast<const int32_t *>(P(positions)), theta));
    }
    DeviceStatus rmsnorm_rope_qk(DeviceTensor &q, DeviceTensor &k, const DeviceWeight &q_weight, const DeviceWeight &k_weight, uint32_t n_q_heads,
                                 uint32_t n_kv_heads, uint32_t q_head_stride, uint32_t k_head_stride, uint32_t head_dim, uint32_t rope_dim, uint32_t pos,
                                 float theta, float eps) override {
        if (DeviceStatus s = rmsnorm_per_head(q, q_weight, n_q_heads, q_head_stride, head_dim, eps); !s.ok) return s;
        if (DeviceStatus s = rmsnorm_per_head(k, k_weight, n_kv_heads, k_head_stride, head_dim, eps); !s.ok) return s;
        if (DeviceStatus s = rope_partial(q, n_q_heads, q_head_stride, rope_dim, pos, theta); !s.ok) return s;
        return rope_partial(k, n_kv_heads, k_head_stride, rope_dim, pos, theta);
    }

    // ---- K/V append ----------------------------------------------------------------------------------------------------------
    DeviceStatus kv_append(DeviceTensor &cache, const DeviceTensor &src, uint32_t pos, uint32_t per_pos_size) override {
        return kv_append_batch(cache, src, pos, per_pos_size, 1);
    }
    DeviceStatus kv_append_batch(DeviceTensor &cache, const DeviceTensor &src, uint32_t base_pos, uint32_t per_pos_size, uint32_t batch) override {
        if (cache.elem_size != 2 || !is_f32(src)) return fail("kv_append: this backend keeps K/V in fp16 and takes fp32 rows");
        if ((uint64_t)(base_pos + batch) * per_pos_size > cache.count || (uint64_t)batch * per_pos_size > src.count) return fail("kv_append: range");
        return st(qb_kv_append(ctx_, P(cache), F(src), base_pos, per_pos_size, batch, nullptr, 0, 0));
    }
    DeviceStatus kv_append_batch_paged_device(DeviceTensor &cache, const DeviceTensor &src, uint32_t base_logical_pos, uint32_t per_pos_size,
                                              uint32_t batch, const DeviceTensor &page_indices, uint32_t n_pages, uint32_t page_size) override {
        if (cache.elem_size != 2 || !is_f32(src) || page_indices.count < n_pages) return fail("kv_append_batch_paged_device: arguments");
        return st(qb_kv_append(ctx_, P(cache), F(src), base_logical_pos, per_pos_size, batch, static_cast<const int32_t *>(P(page_indices)), n_pages, page_size));
    }

    // ---- attention --------------------------------------------------------------------------------------------------------------
    // The library's attention reads q rows laid out as n_heads units of 2*head_dim (query, then output gate), which is the
    // executor's layout (src/qwen_executor.cpp:5592-5594), and scales by 1/sqrt(head_dim).
    DeviceStatus attention_decode_batch_paged_gated_device(DeviceTensor &out, const DeviceTensor &q, uint32_t q_stride, const DeviceTensor &k_cache,
                                                           const DeviceTensor &v_cache, const DeviceTensor &page_indices, uint32_t n_pages, uint32_t page_size,
                                                           uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t base_seq_len, uint32_t batch,
                                                           uint32_t q_batch_stride, uint32_t out_batch_stride, float scale) override {
        return attention(out, q, q_stride, k_cache, v_cache, static_cast<const int32_t *>(P(page_indices)), n_pages, page_size, n_heads, n_kv_heads, head_dim,
                         base_seq_len, batch, q_batch_stride, out_batch_stride, scale, true);
    }
    DeviceStatus attention_decode_batch_gated(DeviceTensor &out, const DeviceTensor &q, uint32_t q_stride, const DeviceTensor &k_cache,
                                              const DeviceTensor &v_cache, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t base_seq_len,
                                              uint32_t batch, uint32_t q_batch_stride, uint32_t out_batch_stride, float scale) override {
        const uint32_t page = 16, n_pages = (base_seq_len + batch + page - 1) / page + 1;
        int32_t *ident = nullptr;
        if (DeviceStatus s = identity_pages(n_pages, &ident); !s.ok) return s;
        return attention(out, q, q_stride, k_cache, v_cache, ident, n_pages, page, n_heads, n_kv_heads, head_dim, base_seq_len, batch, q_batch_stride,
                         out_batch_stride, scale, true);
    }
    DeviceStatus attention_decode(DeviceTensor &out, DeviceTensor &, const DeviceTensor &q, uint32_t q_stride, const DeviceTensor &k_cache,
                                  const DeviceTensor &v_cache, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t seq_len, float scale) override {
        if (seq_len == 0) return fail("attention_decode: empty context");
        const uint32_t page = 16, n_pages = (seq_len + page - 1) / page + 1;
        int32_t *ident = nullptr;
        if (DeviceStatus s = identity_pages(n_pages, &ident); !s.ok) return s;
        return attention(out, q, q_stride, k_cache, v_cache, ident, n_pages, page, n_heads, n_kv_heads, head_dim, seq_len - 1, 1, n_heads * q_stride,
                         n_heads * head_dim, scale, false);
    }
    DeviceStatus apply_attn_gate(DeviceTensor &out, const DeviceTensor &q, uint32_t q_stride, uint32_t n_heads, uint32_t head_dim) override {
        return st(qb_apply_attn_gate(ctx_, F(out), F(q), q_stride, 1, 0, 0, n_heads, head_dim));
    }
    DeviceStatus apply_attn_gate_batch(DeviceTensor &out, const DeviceTensor &q, uint32_t q_stride, uint32_t batch, uint32_t batch_stride_q,
                                       uint32_t batch_stride_out, uint32_t n_heads, uint32_t head_dim) override {
        return st(qb_apply_attn_gate(ctx_, F(out), F(q), q_stride, batch, batch_stride_q, batch_stride_out, n_heads, head_dim));
    }
    // One token through norm + attention over nothing but itself is not a shape this path uses; the executor's decode goes
    // through rmsnorm_per_head / rope_partial / kv_append / attention_decode.
    DeviceStatus attention_single_token(DeviceTensor &, DeviceTensor &, DeviceTensor &, const DeviceTensor &, const DeviceWeight &, const DeviceWeight &,
                                        uint32_t, uint32_t, uint32_t, float) override {
        return fail("attention_single_token is not provided: use rmsnorm_per_head + rope_partial + kv_append + attention_decode");
    }

    // ---- gated DeltaNet -------------------------------------------------------------------------------------------------------------
    DeviceStatus recurrent_single_token(DeviceTensor &core, DeviceTensor &state, DeviceTensor &conv_state, DeviceTensor &conv_out, const DeviceTensor &proj,
                                        const DeviceTensor &gate, const DeviceTensor &alpha, const DeviceTensor &beta, const DeviceWeight &conv,
                                        const DeviceWeight &ssm_a, const DeviceWeight &dt_bias, const DeviceWeight &ssm_norm, uint32_t num_k_heads,
                                        uint32_t num_v_heads, uint32_t head_k_dim, uint32_t head_v_dim, uint32_t conv_kernel_size, float eps) override {
        const uint32_t C = (2 * num_k_heads + num_v_heads) * head_k_dim, vdim = num_v_heads * head_v_dim;
        return recurrent_batch(core, state, conv_state, conv_out, proj, gate, alpha, beta, conv, ssm_a, dt_bias, ssm_norm, 1, num_k_heads, num_v_heads,
                               head_k_dim, head_v_dim, conv_kernel_size, C, C, vdim, num_v_heads, num_v_heads, vdim, eps);
    }
    DeviceStatus recurrent_batch(DeviceTensor &core, DeviceTensor &state, DeviceTensor &conv_state, DeviceTensor &, const DeviceTensor &proj,
                                 const DeviceTensor &gate, const DeviceTensor &alpha, const DeviceTensor &beta, const DeviceWeight &conv,
                                 const DeviceWeight &ssm_a, const DeviceWeight &dt_bias, const DeviceWeight &ssm_norm, uint32_t batch, uint32_t num_k_heads,
                                 uint32_t num_v_heads, uint32_t head_k_dim, uint32_t head_v_dim, uint32_t conv_kernel_size, uint32_t proj_count,
                                 uint32_t proj_stride, uint32_t gate_stride, uint32_t alpha_stride, uint32_t beta_stride, uint32_t core_stride, float eps,
                                 DeviceTensor *state_checkpoints = nullptr, DeviceTensor *conv_state_checkpoints = nullptr, uint32_t checkpoint_count = 0,
                                 DeviceTensor *dn_state_snap = nullptr, DeviceTensor *dn_decaysum = nullptr, uint64_t = 0, uint64_t = 0, uint32_t = 0,
                                 uint32_t = 0, uint32_t = 0) override {
        if (dn_state_snap || dn_decaysum) return fail("recurrent_batch: block-boundary state capture (KVMem retrieval) is outside this path");
        if (head_k_dim != head_v_dim || conv_kernel_size != 4) return fail("recurrent_batch: equal key/value head sizes and a conv kernel of 4 only");
        if (proj_count != (2 * num_k_heads + num_v_heads) * head_k_dim) return fail("recurrent_batch: proj_count is not 2*k_heads*dim + v_heads*dim");
        const uint32_t ck = state_checkpoints && conv_state_checkpoints ? std::min(checkpoint_count, batch) : 0;
        return st(qb_recurrent_batch(ctx_, F(core), core_stride, F(state), F(conv_state), F(proj), proj_stride, F(gate), gate_stride, F(alpha), alpha_stride,
                                     F(beta), beta_stride, W(conv).f32, W(ssm_a).f32, W(dt_bias).f32, W(ssm_norm).f32, batch, num_k_heads, num_v_heads,
                                     head_k_dim, eps, ck ? F(*state_checkpoints) : nullptr, ck ? F(*conv_state_checkpoints) : nullptr, ck));
    }

    // ---- argmax -----------------------------------------------------------------------------------------------------------------------
    DeviceArgmax argmax(const DeviceTensor &x) override {
        std::vector<DeviceArgmax> out;
        DeviceStatus s = argmax_batch(x, 1, (uint32_t)x.count, out);
        return s.ok && !out.empty() ? out[0] : DeviceArgmax{};
    }
    DeviceStatus argmax_batch(const DeviceTensor &x, uint32_t batch, uint32_t row_stride, std::vector<DeviceArgmax> &out) override {
        if (batch == 0 || x.count < (uint64_t)batch * row_stride) return fail("argmax_batch: range");
        if (DeviceStatus s = argmax_scratch(batch); !s.ok) return s;
        if (int rc = qb_argmax_rows_val(ctx_, F(x), batch, row_stride, row_stride, am_tok_, am_val_, 0); rc != QB_OK) return st(rc);
        std::vector<int32_t> tok(batch);
        std::vector<float> val(batch);
        if (int rc = qb_memcpy_d2h(ctx_, tok.data(), am_tok_, (size_t)batch * 4); rc != QB_OK) return st(rc);
        if (int rc = qb_memcpy_d2h(ctx_, val.data(), am_val_, (size_t)batch * 4); rc != QB_OK) return st(rc);
        out.resize(batch);
        for (uint32_t i = 0; i < batch; ++i) { out[i].token = tok[i]; out[i].logit = val[i]; }
        return {};
    }
    std::unique_ptr<DeviceArgmaxBuffer> argmax_buffer(uint64_t count) override {
        auto b = std::make_unique<B200ArgmaxBuffer>();
        b->ctx = ctx_; b->count = count;
        void *t = nullptr, *v = nullptr;
        if (qb_malloc(ctx_, (size_t)count * 4, &t) != QB_OK || qb_malloc(ctx_, (size_t)count * 4, &v) != QB_OK)
            throw std::runtime_error(std::string("b200 argmax_buffer: ") + qb_last_error());
        b->tok = static_cast<int32_t *>(t); b->val = static_cast<float *>(v);
        return b;
    }
    DeviceStatus argmax_to_buffer(const DeviceTensor &x, DeviceArgmaxBuffer &out, uint32_t index) override {
        auto &ab = static_cast<B200ArgmaxBuffer &>(out);
        if (index >= ab.count) return fail("argmax_to_buffer: index");
        return st(qb_argmax_rows_val(ctx_, F(x), 1, (uint32_t)x.count, (uint32_t)x.count, ab.tok, ab.val, index));
    }
    DeviceStatus copy_argmax_buffer_to_host(const DeviceArgmaxBuffer &src, DeviceArgmax *host, uint32_t count) override {
        const auto &ab = static_cast<const B200ArgmaxBuffer &>(src);
        if (count > ab.count) return fail("copy_argmax_buffer_to_host: count");
        std::vector<int32_t> tok(count);
        std::vector<float> val(count);
        if (int rc = qb_memcpy_d2h(ctx_, tok.data(), ab.tok, (size_t)count * 4); rc != QB_OK) return st(rc);
        if (int rc = qb_memcpy_d2h(ctx_, val.data(), ab.val, (size_t)count * 4); rc != QB_OK) return st(rc);
        for (uint32_t i = 0; i < count; ++i) { host[i].token = tok[i]; host[i].logit = val[i]; }
        return {};
    }

    // ---- MTP packing ----------------------------------------------------------------------------------------------------------------------
    DeviceStatus pack_mtp_prefix_hinputs(DeviceTensor &dst, const DeviceTensor &first_h, const DeviceTensor &h_batch, uint32_t batch, uint32_t h_stride) override {
        if (batch == 0 || h_stride == 0) return {};
        if (dst.count < (uint64_t)batch * h_stride || first_h.count < h_stride || (batch > 1 && h_batch.count < (uint64_t)(batch - 1) * h_stride))
            return fail("pack_mtp_prefix_hinputs: range");
        return st(qb_pack_mtp_prefix_hinputs(ctx_, F(dst), F(first_h), F(h_batch), batch, h_stride));
    }
    DeviceStatus pack_mtp_concat(DeviceTensor &dst, const DeviceTensor &left, const DeviceTensor &right, uint32_t batch, uint32_t left_stride,
                                 uint32_t right_stride, uint32_t concat_stride, uint32_t width) override {
        if (batch == 0 || width == 0) return {};
        return st(qb_pack_mtp_concat(ctx_, F(dst), F(left), F(right), batch, left_stride, right_stride, concat_stride, width));
    }

    qb_ctx *context() const { return ctx_; }

private:
    DeviceStatus attention(DeviceTensor &out, const DeviceTensor &q, uint32_t q_stride, const DeviceTensor &k_cache, const DeviceTensor &v_cache,
                           const int32_t *pages, uint32_t n_pages, uint32_t page_size, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                           uint32_t base_pos, uint32_t batch, uint32_t q_batch_stride, uint32_t out_batch_stride, float scale, bool gated) {
        if (k_cache.elem_size != 2 || v_cache.elem_size != 2) return fail("attention: this backend keeps K/V in fp16");
        if (q_stride != 2 * head_dim) return fail("attention: q units must be [query | gate] of 2*head_dim");
        if (out_batch_stride != n_heads * head_dim) return fail("attention: output rows must be dense");
        if (std::fabs(scale * std::sqrt((float)head_dim) - 1.0f) > 1e-5f) return fail("attention: scale must be 1/sqrt(head_dim)");
        if ((uint64_t)(base_pos + batch + page_size - 1) / page_size > n_pages) return fail("attention: positions beyond the page list");
        if (DeviceStatus s = position(base_pos); !s.ok) return s;
        const int rc = gated ? qb_attention_paged_gated(ctx_, F(q), batch, q_batch_stride, n_heads, n_kv_heads, head_dim, pos_, 1, pages, n_pages, page_size,
                                                        P(k_cache), P(v_cache), base_pos + batch, F(out))
                             : qb_attention_paged(ctx_, F(q), batch, q_batch_stride, n_heads, n_kv_heads, head_dim, pos_, 1, pages, n_pages, page_size,
                                                  P(k_cache), P(v_cache), base_pos + batch, F(out));
        return st(rc);
    }
    DeviceStatus position(uint32_t base_pos) {
        if (!pos_) { void *p = nullptr; if (int rc = qb_malloc(ctx_, 64, &p); rc != QB_OK) return st(rc); pos_ = static_cast<int32_t *>(p); }
        const int32_t v = (int32_t)base_pos;
        return st(qb_memcpy_h2d(ctx_, pos_, &v, 4));
    }
    DeviceStatus identity_pages(uint32_t n, int32_t **out) {
        if (n > ident_n_) {
            if (ident_) qb_free(ctx_, ident_);
            ident_ = nullptr;
            const uint32_t want = std::max(n * 2, 4096u);
            void *p = nullptr;
            if (int rc = qb_malloc(ctx_, (size_t)want * 4, &p); rc != QB_OK) return st(rc);
            std::vector<int32_t> id(want);
            for (uint32_t i = 0; i < want; ++i) id[i] = (int32_t)i;
            if (int rc = qb_memcpy_h2d(ctx_, p, id.data(), (size_t)want * 4); rc != QB_OK) return st(rc);
            ident_ = static_cast<int32_t *>(p); ident_n_ = want;
        }
        *out = ident_;
        return {};
    }
    DeviceStatus grow(void **buf, uint64_t *cap, uint64_t bytes) {
        if (bytes <= *cap) return {};
        if (*buf) qb_free(ctx_, *buf);
        *buf = nullptr; *cap = 0;
        if (int rc = qb_malloc(ctx_, (size_t)bytes * 2, buf); rc != QB_OK) return st(rc);
        *cap = bytes * 2;
        return {};
    }
    DeviceStatus tmp_buffer(uint64_t floats, float **out) {
        DeviceStatus s = grow(&tmp_, &tmp_cap_, floats * 4);
        *out = static_cast<float *>(tmp_);
        return s;
    }
    DeviceStatus ids_buffer(uint32_t n, int32_t **out) {
        DeviceStatus s = grow(&ids_, &ids_cap_, (uint64_t)n * 4);
        *out = static_cast<int32_t *>(ids_);
        return s;
    }
    DeviceStatus argmax_scratch(uint32_t batch) {
        if (batch <= am_n_) return {};
        if (am_tok_) qb_free(ctx_, am_tok_);
        if (am_val_) qb_free(ctx_, am_val_);
        am_tok_ = nullptr; am_val_ = nullptr; am_n_ = 0;
        void *t = nullptr, *v = nullptr;
        if (int rc = qb_malloc(ctx_, (size_t)batch * 8, &t); rc != QB_OK) return st(rc);
        if (int rc = qb_malloc(ctx_, (size_t)batch * 8, &v); rc != QB_OK) return st(rc);
        am_tok_ = static_cast<int32_t *>(t); am_val_ = static_cast<float *>(v); am_n_ = batch * 2;
        return {};
    }

    qb_ctx *ctx_ = nullptr;
    int32_t *ident_ = nullptr; uint32_t ident_n_ = 0;
    int32_t *pos_ = nullptr;
    void *tmp_ = nullptr; uint64_t tmp_cap_ = 0;
    void *ids_ = nullptr; uint64_t ids_cap_ = 0;
    int32_t *am_tok_ = nullptr; float *am_val_ = nullptr; uint32_t am_n_ = 0;
};

}  // namespace

std::unique_ptr<DeviceBackend> make_b200_device_backend(int device) { return std::make_unique<B200DeviceBackend>(device); }

#ifdef QW3B200_PROVIDE_CUDA_FACTORY
bool cuda_device_backend_available() {
    qb_ctx *c = nullptr;
    if (qb_create(0, &c) != QB_OK) return false;
    qb_destroy(c);
    return true;
}
std::unique_ptr<DeviceBackend> make_cuda_device_backend(LinearBackend) { return make_b200_device_backend(0); }
#endif

}  // namespace qw3
