// TEST INFRASTRUCTURE ONLY.  A C ABI over the reference's own CUDA DeviceBackend
// (make_cuda_device_backend, include/qw3/device_backend.hpp:2744; class CudaDeviceBackend,
// src/kernels_cuda.cu:9564), compiled from the reference sources where they lie into
// oracle/_ref/libqw3ref_backend.so.  The GPU parity tests drive the reference backend's operators
// through it (its own tensors, weights, streams and kernel dispatch) and compare them with this
// project's CUDA path and with the CPU oracle.  Nothing here is linked into the product library.
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "qw3/device_backend.hpp"

using namespace qw3;

namespace {
thread_local std::string g_err;
int fail(const char *what) { g_err = what ? what : "unknown"; return 1; }
int st(const DeviceStatus &s) { return s.ok ? 0 : fail(s.message); }
inline DeviceBackend &B(void *b) { return *static_cast<DeviceBackend *>(b); }
inline DeviceTensor &T(void *t) { return *static_cast<DeviceTensor *>(t); }
inline const DeviceWeight &W(void *w) { return *static_cast<const DeviceWeight *>(w); }
}  // namespace

extern "C" {

const char *rb_last_error() { return g_err.c_str(); }

// linear: 0 = Auto, 1 = Custom (the reference's own Q8_0 kernels), 2 = Cublas
void *rb_create(int linear) {
    try {
        auto be = make_cuda_device_backend(linear == 2 ? LinearBackend::Cublas : linear == 1 ? LinearBackend::Custom : LinearBackend::Auto);
        if (!be) { fail("make_cuda_device_backend returned null"); return nullptr; }
        DeviceStatus s = be->begin();
        if (!s.ok) { fail(s.message); return nullptr; }
        return be.release();
    } catch (const std::exception &e) { fail(e.what()); return nullptr; }
}
void rb_destroy(void *b) { if (b) { B(b).end(); delete static_cast<DeviceBackend *>(b); } }
const char *rb_name(void *b) { return B(b).name(); }
int rb_sync(void *b) { return st(B(b).synchronize()); }

// CUDA-graph hooks of the backend (include/qw3/device_backend.hpp:96-116): the timing tests capture a run of
// operator calls once and replay it, as the reference's decode loop does.
int rb_begin_capture(void *b) { return B(b).begin_capture() ? 0 : fail("begin_capture refused"); }
int rb_end_capture(void *b) { return st(B(b).end_capture()); }
int rb_replay_graph(void *b) { return st(B(b).replay_graph()); }

// kind: 0 = f32, 1 = f16, 2 = i32
void *rb_tensor(void *b, int kind, uint64_t count) {
    try {
        auto t = kind == 1 ? B(b).tensor_f16(count, "pin") : kind == 2 ? B(b).tensor_i32(count, "pin") : B(b).tensor_f32(count, "pin");
        return t.release();
    } catch (const std::exception &e) { fail(e.what()); return nullptr; }
}
void rb_tensor_free(void *t) { delete static_cast<DeviceTensor *>(t); }
uint32_t rb_tensor_elem_size(void *t) { return T(t).elem_size; }
int rb_upload(void *b, void *t, uint64_t byte_offset, const void *host, uint64_t bytes) {
    if (int r = st(B(b).copy_bytes_from_host(T(t), byte_offset, host, bytes))) return r;
    return st(B(b).synchronize());
}
int rb_download(void *b, void *t, uint64_t byte_offset, void *host, uint64_t bytes) {
    if (int r = st(B(b).synchronize())) return r;
    return st(B(b).copy_bytes_to_host(T(t), host, byte_offset, bytes));
}

void *rb_weight_f32(void *b, const float *data, uint64_t count) {
    try { return B(b).weight_f32(data, count, "pin").release(); } catch (const std::exception &e) { fail(e.what()); return nullptr; }
}
void *rb_weight_q8_0(void *b, const void *blocks, uint64_t rows, uint64_t cols) {
    try { return B(b).weight_q8_0(blocks, rows, cols, "pin").release(); } catch (const std::exception &e) { fail(e.what()); return nullptr; }
}
void rb_weight_free(void *w) { delete static_cast<DeviceWeight *>(w); }

int rb_rms_norm_batch(void *b, void *out, void *x, void *w, uint32_t batch, uint32_t n, float eps) {
    return st(B(b).rms_norm_batch(T(out), T(x), W(w), batch, n, eps));
}
int rb_rmsnorm_per_head_batch(void *b, void *x, void *w, uint32_t batch, uint32_t batch_stride, uint32_t n_units,
                              uint32_t per_unit_stride, uint32_t head_dim, float eps) {
    return st(B(b).rmsnorm_per_head_batch(T(x), W(w), batch, batch_stride, n_units, per_unit_stride, head_dim, eps));
}
int rb_rope_partial_batch(void *b, void *x, uint32_t batch, uint32_t batch_stride, uint32_t n_units, uint32_t per_unit_stride,
                          uint32_t rope_dim, uint32_t base_pos, float theta) {
    return st(B(b).rope_partial_batch(T(x), batch, batch_stride, n_units, per_unit_stride, rope_dim, base_pos, theta));
}
int rb_kv_append_batch(void *b, void *cache, void *src, uint32_t base_pos, uint32_t per_pos_size, uint32_t batch) {
    return st(B(b).kv_append_batch(T(cache), T(src), base_pos, per_pos_size, batch));
}
int rb_attention_decode_batch_gated(void *b, void *out, void *q, uint32_t q_stride, void *k_cache, void *v_cache, uint32_t n_heads,
                                    uint32_t n_kv_heads, uint32_t head_dim, uint32_t base_seq_len, uint32_t batch,
                                    uint32_t q_batch_stride, uint32_t out_batch_stride, float scale) {
    return st(B(b).attention_decode_batch_gated(T(out), T(q), q_stride, T(k_cache), T(v_cache), n_heads, n_kv_heads, head_dim,
                                                base_seq_len, batch, q_batch_stride, out_batch_stride, scale));
}
int rb_recurrent_batch(void *b, void *core, void *state, void *conv_state, void *conv_out, void *proj, void *gate, void *alpha,
                       void *beta, void *conv_w, void *ssm_a, void *dt_bias, void *ssm_norm, uint32_t batch, uint32_t nk,
                       uint32_t nv, uint32_t hk, uint32_t hv, uint32_t conv_k, uint32_t proj_count, uint32_t proj_stride,
                       uint32_t gate_stride, uint32_t alpha_stride, uint32_t beta_stride, uint32_t core_stride, float eps,
                       void *state_ckpt, void *conv_ckpt, uint32_t ckpt_count) {
    return st(B(b).recurrent_batch(T(core), T(state), T(conv_state), T(conv_out), T(proj), T(gate), T(alpha), T(beta), W(conv_w),
                                   W(ssm_a), W(dt_bias), W(ssm_norm), batch, nk, nv, hk, hv, conv_k, proj_count, proj_stride,
                                   gate_stride, alpha_stride, beta_stride, core_stride, eps,
                                   state_ckpt ? &T(state_ckpt) : nullptr, conv_ckpt ? &T(conv_ckpt) : nullptr, ckpt_count));
}
int rb_argmax_batch(void *b, void *x, uint32_t batch, uint32_t row_stride, int32_t *tokens, float *logits) {
    std::vector<DeviceArgmax> out;
    if (int r = st(B(b).argmax_batch(T(x), batch, row_stride, out))) return r;
    for (uint32_t i = 0; i < batch && i < out.size(); ++i) { tokens[i] = out[i].token; logits[i] = out[i].logit; }
    return 0;
}
int rb_q8_0_matmul(void *b, void *out, void *w, void *x, uint32_t batch, uint32_t in_stride, uint32_t out_stride) {
    return st(B(b).q8_0_matmul(T(out), W(w), T(x), batch, in_stride, out_stride));
}
int rb_q8_0_matmul_silu_mul(void *b, void *out, void *w_gate, void *w_up, void *x, uint32_t batch, uint32_t in_stride,
                            uint32_t out_stride) {
    return st(B(b).q8_0_matmul_silu_mul(T(out), W(w_gate), W(w_up), T(x), batch, in_stride, out_stride));
}
int rb_q8_0_matvec_silu_mul(void *b, void *out, void *w_gate, void *w_up, void *x) {
    return st(B(b).q8_0_matvec_silu_mul(T(out), W(w_gate), W(w_up), T(x)));
}
int rb_q8_0_get_rows_batch(void *b, void *out, void *w, const uint64_t *rows, uint32_t batch) {
    return st(B(b).q8_0_get_rows_batch(T(out), W(w), rows, batch));
}
int rb_silu_mul_n(void *b, void *out, void *gate, void *up, uint64_t count) {
    return st(B(b).silu_mul_n(T(out), T(gate), T(up), count));
}
int rb_add_n(void *b, void *out, void *a, void *c, uint64_t count) { return st(B(b).add_n(T(out), T(a), T(c), count)); }
int rb_kv_append_batch_paged_device(void *b, void *cache, void *src, uint32_t base_pos, uint32_t per_pos_size, uint32_t batch, void *pages,
                                    uint32_t n_pages, uint32_t page_size) {
    return st(B(b).kv_append_batch_paged_device(T(cache), T(src), base_pos, per_pos_size, batch, T(pages), n_pages, page_size));
}
int rb_attention_decode_batch_paged_gated_device(void *b, void *out, void *q, uint32_t q_stride, void *k_cache, void *v_cache, void *pages,
                                                 uint32_t n_pages, uint32_t page_size, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                                                 uint32_t base_seq_len, uint32_t batch, uint32_t q_batch_stride, uint32_t out_batch_stride, float scale) {
    return st(B(b).attention_decode_batch_paged_gated_device(T(out), T(q), q_stride, T(k_cache), T(v_cache), T(pages), n_pages, page_size, n_heads,
                                                             n_kv_heads, head_dim, base_seq_len, batch, q_batch_stride, out_batch_stride, scale));
}
int rb_q8_0_matvec(void *b, void *out, void *w, void *x) { return st(B(b).q8_0_matvec(T(out), W(w), T(x))); }
int rb_q8_0_matvec_add(void *b, void *accum, void *w, void *x) { return st(B(b).q8_0_matvec_add(T(accum), W(w), T(x))); }
int rb_argmax_to_buffer_roundtrip(void *b, void *x, uint32_t slots, uint32_t index, int32_t *token, float *logit) {
    try {
        auto buf = B(b).argmax_buffer(slots);
        if (int r = st(B(b).argmax_to_buffer(T(x), *buf, index))) return r;
        std::vector<DeviceArgmax> host(slots);
        if (int r = st(B(b).copy_argmax_buffer_to_host(*buf, host.data(), slots))) return r;
        *token = host[index].token; *logit = host[index].logit;
        return 0;
    } catch (const std::exception &e) { return fail(e.what()); }
}
int rb_pack_mtp_concat(void *b, void *dst, void *left, void *right, uint32_t batch, uint32_t ls, uint32_t rs, uint32_t cs, uint32_t width) {
    return st(B(b).pack_mtp_concat(T(dst), T(left), T(right), batch, ls, rs, cs, width));
}
int rb_pack_mtp_prefix_hinputs(void *b, void *dst, void *first_h, void *h_batch, uint32_t batch, uint32_t h_stride) {
    return st(B(b).pack_mtp_prefix_hinputs(T(dst), T(first_h), T(h_batch), batch, h_stride));
}
int rb_rms_norm_q8_0_matmul_fanout2(void *b, void *normalized, void *out0, void *out1, void *w0, void *w1, uint32_t os0, uint32_t os1, void *x,
                                    void *norm_w, uint32_t batch, uint32_t in_stride, float eps) {
    DeviceTensor *outs[2] = {&T(out0), &T(out1)};
    const DeviceWeight *ws[2] = {&W(w0), &W(w1)};
    const uint32_t strides[2] = {os0, os1};
    return st(B(b).rms_norm_q8_0_matmul_fanout(T(normalized), outs, ws, strides, 2, T(x), W(norm_w), batch, in_stride, eps));
}

}  // extern "C"
