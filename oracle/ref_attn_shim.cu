// extern "C" forwarder to the reference's native decode attention (src/fattn_vec_decode.cu, launcher at :514-537),
// compiled from the reference source where it lies (Makefile target `ref-attn`; a long compile, hence a library
// of its own).  Test infrastructure only: the GPU tests run it beside the product's paged attention.
#include <cuda_runtime.h>
#include <cstdint>

namespace qw3 { namespace ported {
bool launch_fattn_vec_decode_f16(float *out, const float *q, uint32_t q_stride, const void *k_cache, const void *v_cache,
                                 uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t seq_len, uint32_t batch,
                                 uint32_t q_batch_stride, uint32_t out_batch_stride, float scale, cudaStream_t stream);
}}

extern "C" {
// Row b of `batch` consecutive positions attends keys [0, seq_len + b); q rows are [n_heads][q_stride] (gate after the
// head_dim query values), caches are dense fp16 [position][n_kv_heads][head_dim]; out = [batch][n_heads][head_dim].
int ref_fattn_vec_decode_f16(float *out, const float *q, uint32_t q_stride, const void *k_cache, const void *v_cache,
                             uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t seq_len, uint32_t batch,
                             uint32_t q_batch_stride, uint32_t out_batch_stride, float scale) {
    if (!qw3::ported::launch_fattn_vec_decode_f16(out, q, q_stride, k_cache, v_cache, n_heads, n_kv_heads, head_dim, seq_len, batch,
                                                  q_batch_stride, out_batch_stride, scale, 0))
        return -1;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}
}
