// extern "C" forwarders to the reference's own CUDA launchers for this path, so the GPU tests can
// run the reference kernels (compiled from the reference sources where they lie, see Makefile
// target `ref`) beside the oracle and the product kernels.  Test infrastructure only.
#include <cuda_runtime.h>
#include <cstdint>

namespace qw3 { namespace ported {
bool launch_quantize_q8_1(const float *, void *, uint32_t, uint32_t, uint32_t, cudaStream_t);
bool launch_quantize_mmq_q8_1(const float *, void *, uint32_t, uint32_t, uint32_t, cudaStream_t);
bool launch_mmvq_q8_0(const uint8_t *, const void *, float *, uint32_t, uint32_t, uint32_t, uint32_t, cudaStream_t);
bool launch_mmq_q8_0(const uint8_t *, const void *, float *, uint32_t, uint32_t, uint32_t, uint32_t, cudaStream_t);
bool launch_mmq_q8_0_medium(const uint8_t *, const void *, float *, uint32_t, uint32_t, uint32_t, uint32_t, cudaStream_t);
bool launch_gated_delta_net(float *alpha_inout, float *beta_inout, const float *dt_bias, const float *ssm_a,
                            const float *conv_qkv, uint32_t q_offset, uint32_t k_offset, uint32_t v_offset, float *state,
                            float *core_out, uint32_t T, uint32_t num_k_heads, uint32_t num_v_heads, uint32_t head_dim,
                            uint32_t qkv_row_stride, uint32_t gb_row_stride, uint32_t out_row_stride, bool prep_decay,
                            float *state_checkpoints, uint32_t checkpoint_count, cudaStream_t stream);
}}

static int finish(bool ok) {
    if (!ok) return -1;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}

extern "C" {
int ref_quantize_q8_1(const float *x, void *y, uint32_t batch, uint32_t cols) {
    return finish(qw3::ported::launch_quantize_q8_1(x, y, batch, cols, cols, 0));
}
int ref_quantize_mmq_q8_1(const float *x, void *y, uint32_t batch, uint32_t cols) {
    return finish(qw3::ported::launch_quantize_mmq_q8_1(x, y, batch, cols, cols, 0));
}
int ref_mmvq_q8_0(const uint8_t *w, const void *y, float *dst, uint32_t rows, uint32_t cols, uint32_t batch) {
    return finish(qw3::ported::launch_mmvq_q8_0(w, y, dst, rows, cols, batch, rows, 0));
}
int ref_mmq_q8_0(const uint8_t *w, const void *y, float *dst, uint32_t rows, uint32_t cols, uint32_t batch) {
    return finish(qw3::ported::launch_mmq_q8_0(w, y, dst, rows, cols, batch, rows, 0));
}
int ref_mmq_q8_0_medium(const uint8_t *w, const void *y, float *dst, uint32_t rows, uint32_t cols, uint32_t batch) {
    return finish(qw3::ported::launch_mmq_q8_0_medium(w, y, dst, rows, cols, batch, rows, 0));
}
int ref_gated_delta_net(float *alpha, float *beta, const float *dt_bias, const float *ssm_a, const float *conv_qkv,
                        uint32_t q_off, uint32_t k_off, uint32_t v_off, float *state, float *core, uint32_t T, uint32_t nk,
                        uint32_t nv, uint32_t hd, uint32_t qkv_stride, uint32_t gb_stride, uint32_t out_stride,
                        float *ckpt, uint32_t ckpt_count) {
    return finish(qw3::ported::launch_gated_delta_net(alpha, beta, dt_bias, ssm_a, conv_qkv, q_off, k_off, v_off, state, core,
                                                      T, nk, nv, hd, qkv_stride, gb_stride, out_stride, true, ckpt,
                                                      ckpt_count, 0));
}

// Device time of one launch of a reference GEMM kernel (kind 0 = mul_mat_vec_q8_0, 1 = mmq_q8_0, 2 = mmq_q8_0_medium):
// median of `iters` launches, each after `flush` (a buffer larger than L2) has been rewritten, CUDA events on the
// launching stream.  Returns -1 when the launcher declines the shape.
int ref_time_gemm(int kind, const uint8_t *w, const void *y, float *dst, uint32_t rows, uint32_t cols, uint32_t batch,
                  int iters, void *flush, size_t flush_bytes, float *us_out) {
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    float t[64];
    if (iters > 64) iters = 64;
    int n = 0;
    for (int it = 0; it < iters + 2; ++it) {
        if (flush) cudaMemsetAsync(flush, it & 0xff, flush_bytes, 0);
        cudaEventRecord(e0, 0);
        bool ok = kind == 0 ? qw3::ported::launch_mmvq_q8_0(w, y, dst, rows, cols, batch, rows, 0)
                : kind == 1 ? qw3::ported::launch_mmq_q8_0(w, y, dst, rows, cols, batch, rows, 0)
                            : qw3::ported::launch_mmq_q8_0_medium(w, y, dst, rows, cols, batch, rows, 0);
        cudaEventRecord(e1, 0);
        if (!ok) { cudaEventDestroy(e0); cudaEventDestroy(e1); return -1; }
        if (cudaDeviceSynchronize() != cudaSuccess) { cudaEventDestroy(e0); cudaEventDestroy(e1); return (int)cudaGetLastError(); }
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (it >= 2) t[n++] = ms * 1e3f;
    }
    for (int i = 1; i < n; ++i) for (int j = i; j > 0 && t[j] < t[j - 1]; --j) { float x = t[j]; t[j] = t[j - 1]; t[j - 1] = x; }
    *us_out = t[n / 2];
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return 0;
}
}
