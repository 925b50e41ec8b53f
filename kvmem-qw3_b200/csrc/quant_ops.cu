// Activation quantisers and the fused element-wise kernels around the Q8 GEMMs.
#include "qb_internal.h"

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One warp quantises one 32-block with the arithmetic of quantize_mmq_q8_1_kernel
// (src/mmvq_q8.cu:694-721): d_inv = 127/amax, q = rint(x*d_inv), d = 1/d_inv.
__device__ __forceinline__ void quant_block_store(float v, int lane, int8_t *q_blk, float *d_out) {
    const float amax = warp_max(fabsf(v));
    const float d_inv = (amax == 0.0f) ? 0.0f : __fdiv_rn(127.0f, amax);
    const int qi = (amax == 0.0f) ? 0 : __float2int_rn(__fmul_rn(v, d_inv));
    q_blk[lane] = (int8_t)qi;
    if (lane == 0) *d_out = (amax == 0.0f) ? 0.0f : __fdiv_rn(1.0f, d_inv);
}

// ---- reference-format quantisers (parity tests against the reference kernels) --------------

// quantize_q8_1_kernel (src/mmvq_q8.cu:83-112): 36-byte blocks {half d, half sum, int8 q[32]}.
__global__ void quantize_q8_1_ref_kernel(const float *__restrict__ x, uint32_t K, uint32_t x_stride, uint8_t *out) {
    const uint32_t nb = K / 32;
    const uint32_t kb = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const uint32_t m = blockIdx.y, lane = threadIdx.x & 31;
    if (kb >= nb) return;
    const float v = x[(size_t)m * x_stride + kb * 32 + lane];
    const float amax = warp_max(fabsf(v));
    const float sum = warp_sum(v);
    const float d = __fdiv_rn(amax, 127.0f);
    uint8_t *blk = out + ((size_t)m * nb + kb) * 36;
    blk[4 + lane] = (uint8_t)(int8_t)((amax == 0.0f) ? 0 : __float2int_rn(__fdiv_rn(v, d)));
    if (lane == 0) {
        reinterpret_cast<__half *>(blk)[0] = __float2half_rn(d);
        reinterpret_cast<__half *>(blk)[1] = __float2half_rn(sum);
    }
}

// quantize_mmq_q8_1_kernel (src/mmvq_q8.cu:669-722): 144-byte blocks, index sb*M + row.
__global__ void quantize_q8_1_mmq_ref_kernel(const float *__restrict__ x, uint32_t M, uint32_t K, uint32_t x_stride,
                                             uint8_t *out) {
    const uint32_t nb = K / 32;
    const uint32_t kb = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const uint32_t m = blockIdx.y, lane = threadIdx.x & 31;
    if (kb >= nb) return;
    const float v = x[(size_t)m * x_stride + kb * 32 + lane];
    uint8_t *blk = out + ((size_t)(kb / 4) * M + m) * 144;
    quant_block_store(v, lane, reinterpret_cast<int8_t *>(blk + 16 + (kb % 4) * 32),
                      reinterpret_cast<float *>(blk) + (kb % 4));
}

extern "C" int qb_quantize_q8_1(qb_ctx *ctx, const float *x_dev, uint32_t M, uint32_t K, uint32_t x_stride, void *out_dev) {
    QB_REQUIRE(ctx && x_dev && out_dev && K % 32 == 0 && M > 0, "qb_quantize_q8_1: bad arguments");
    dim3 grid((K / 32 + 7) / 8, M);
    quantize_q8_1_ref_kernel<<<grid, 256, 0, ctx->stream>>>(x_dev, K, x_stride, (uint8_t *)out_dev);
    QB_LAUNCHED(ctx, "quantize_q8_1_ref_kernel");
    return QB_OK;
}

extern "C" int qb_quantize_q8_1_mmq(qb_ctx *ctx, const float *x_dev, uint32_t M, uint32_t K, uint32_t x_stride,
                                    void *out_dev) {
    QB_REQUIRE(ctx && x_dev && out_dev && K % 128 == 0 && M > 0, "qb_quantize_q8_1_mmq: bad arguments");
    dim3 grid((K / 32 + 7) / 8, M);
    quantize_q8_1_mmq_ref_kernel<<<grid, 256, 0, ctx->stream>>>(x_dev, M, K, x_stride, (uint8_t *)out_dev);
    QB_LAUNCHED(ctx, "quantize_q8_1_mmq_ref_kernel");
    return QB_OK;
}

// ---- fused: (x + split partials) -> residual stream -> RMSNorm -> int8 ----------------------
// One CTA of 1024 threads per row.  Pass 1 only loads (x and the split partials, independent loads the
// compiler can keep in flight together) and stages the row in shared memory; pass 2 writes the residual
// stream, the normalised copy and the int8 blocks.
template <int THREADS>
__global__ void __launch_bounds__(THREADS) norm_quant_kernel(NormQuantArgs a) {
    QB_PDL_ENTER();
    extern __shared__ float row[];
    __shared__ float red[THREADS / 32];
    float *wsm = row + a.n;
    const uint32_t m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t src = a.row_map ? (uint32_t)a.row_map[m] : m;
    const float *__restrict__ x = a.x ? a.x + (size_t)src * a.x_stride : nullptr;
    const float *__restrict__ parts = a.parts ? a.parts + (size_t)m * a.part_ld : nullptr;
    const size_t pstride = (size_t)a.M * a.part_ld;
    float ss = 0.0f;
#pragma unroll 4
    for (uint32_t i = tid; i < a.n; i += THREADS) {
        float v = x ? x[i] : 0.0f;
        if (a.S > 0) {   // GEMM result first (segments ascending), then the residual
            float p[8];  // all segment loads are issued before the first add (S <= 8)
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s) p[s] = s < a.S ? parts[s * pstride + i] : 0.0f;
            float y = p[0];
#pragma unroll
            for (uint32_t s = 1; s < 8; ++s) if (s < a.S) y += p[s];
            v = x ? v + y : y;
        }
        row[i] = v;
        wsm[i] = a.w ? a.w[i] : 1.0f;    // gains staged now: pass 2 has no global load in its dependency chain
        ss += v * v;
    }
    float scale = 1.0f;
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (a.w) {
        float tot = 0.0f;
#pragma unroll
        for (int i = 0; i < THREADS / 32; ++i) tot += red[i];
        scale = rsqrtf(tot / (float)a.n + a.eps);
    }
    const uint32_t nblk = a.n / 32;
    for (uint32_t b = warp; b < nblk; b += THREADS / 32) {
        const uint32_t i = b * 32 + lane;
        float v = row[i];
        if (a.h_out) a.h_out[(size_t)m * a.h_stride + i] = v;
        if (a.w) v = v * scale * wsm[i];
        if (a.normed_out) a.normed_out[(size_t)m * a.n + i] = v;
        if (a.q)
            quant_block_store(v, lane, a.q + (size_t)m * a.q_pitch + a.q_col_off + b * 32,
                              a.d + (size_t)(a.d_kb_off + b) * a.d_ld + m);
    }
}

int qb_launch_norm_quant(qb_ctx *ctx, const NormQuantArgs &a) {
    QB_REQUIRE(a.M > 0 && a.n > 0 && a.n % 32 == 0 && a.S <= 8, "norm_quant: bad shape M=%u n=%u S=%u", a.M, a.n, a.S);
    const size_t smem = 2 * (size_t)a.n * sizeof(float);
    static bool attr_set = false;
    if (!attr_set) {
        QB_CUDA(cudaFuncSetAttribute(norm_quant_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        attr_set = true;
    }
    QB_REQUIRE(smem <= 160 * 1024, "norm_quant: row of %u floats does not fit shared memory", a.n);
    QB_CUDA(qb_launch_pdl(ctx->stream, norm_quant_kernel<1024>, dim3(a.M), dim3(1024), (size_t)(smem), a));
    QB_LAUNCHED(ctx, "norm_quant_kernel");
    return QB_OK;
}

extern "C" int qb_quantize_act(qb_ctx *ctx, const float *x_dev, uint32_t M, uint32_t K, uint32_t x_stride, int8_t *q_dev,
                               float *d_dev) {
    QB_REQUIRE(ctx && x_dev && q_dev && d_dev && K % 32 == 0, "qb_quantize_act: bad arguments");
    NormQuantArgs a;
    a.x = x_dev; a.x_stride = x_stride; a.n = K; a.M = M;
    a.q = q_dev; a.q_pitch = K; a.d = d_dev; a.d_ld = qb_act_ld(M);
    return qb_launch_norm_quant(ctx, a);
}

extern "C" int qb_rms_norm(qb_ctx *ctx, const float *x_dev, const float *w_dev, uint32_t M, uint32_t n, uint32_t stride,
                           float eps, float *out_dev) {
    QB_REQUIRE(ctx && x_dev && w_dev && out_dev && n % 32 == 0 && stride == n, "qb_rms_norm: bad arguments (stride must equal n)");
    NormQuantArgs a;
    a.x = x_dev; a.x_stride = stride; a.n = n; a.M = M; a.w = w_dev; a.eps = eps; a.normed_out = out_dev;
    return qb_launch_norm_quant(ctx, a);
}

// silu(gate) * up -> int8 (silu_mul_kernel src/kernels_cuda.cu:1894-1903 fused with the quantiser).
__global__ void swiglu_quant_kernel(const float *__restrict__ gu, uint32_t gu_stride, uint32_t F, int8_t *q,
                                    uint32_t q_pitch, float *d, uint32_t d_ld) {
    QB_PDL_ENTER();
    const uint32_t b = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, m = blockIdx.y, lane = threadIdx.x & 31;
    if (b >= F / 32) return;
    const float g = gu[(size_t)m * gu_stride + b * 32 + lane];
    const float u = gu[(size_t)m * gu_stride + F + b * 32 + lane];
    const float v = __fdiv_rn(g, 1.0f + expf(-g)) * u;
    quant_block_store(v, lane, q + (size_t)m * q_pitch + b * 32, d + (size_t)b * d_ld + m);
}

int qb_launch_swiglu_quant(qb_ctx *ctx, const float *gu, uint32_t gu_stride, uint32_t M, uint32_t F, int8_t *q,
                           uint32_t q_pitch, float *d, uint32_t d_ld) {
    dim3 grid((F / 32 + 7) / 8, M);
    QB_CUDA(qb_launch_pdl(ctx->stream, swiglu_quant_kernel, dim3(grid), dim3(256), (size_t)(0), gu, gu_stride, F, q, q_pitch, d, d_ld));
    QB_LAUNCHED(ctx, "swiglu_quant_kernel");
    return QB_OK;
}

__global__ void reduce_parts_kernel(const float *__restrict__ part, uint32_t S, uint32_t M, uint32_t N, float *y,
                                    uint32_t y_stride) {
    QB_PDL_ENTER();
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
    if (n >= N) return;
    float v = part[(size_t)m * N + n];
    for (uint32_t s = 1; s < S; ++s) v += part[((size_t)s * M + m) * N + n];
    y[(size_t)m * y_stride + n] = v;
}

int qb_launch_reduce_parts(qb_ctx *ctx, const float *part, uint32_t S, uint32_t M, uint32_t N, float *y,
                           uint32_t y_stride) {
    dim3 grid((N + 255) / 256, M);
    QB_CUDA(qb_launch_pdl(ctx->stream, reduce_parts_kernel, dim3(grid), dim3(256), (size_t)(0), part, S, M, N, y, y_stride));
    QB_LAUNCHED(ctx, "reduce_parts_kernel");
    return QB_OK;
}

// ---- argmax: lowest index wins ties (argmax_kernel src/kernels_cuda.cu:1765-1771) ----------
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
    return v > bv || (v == bv && i < bi);
}

__global__ void argmax_partial_kernel(const float *__restrict__ x, uint32_t n, uint32_t stride, float *pval, int32_t *pidx,
                                      uint32_t nblk) {
    QB_PDL_ENTER();
    __shared__ float sv[8];
    __shared__ int si[8];
    const uint32_t m = blockIdx.y, blk = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t per = (n + nblk - 1) / nblk;
    const uint32_t lo = blk * per, hi = min(n, lo + per);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (uint32_t i = lo + tid; i < hi; i += blockDim.x) {
        const float v = x[(size_t)m * stride + i];
        if (better(v, (int)i, bv, bi)) { bv = v; bi = (int)i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 8; ++w) if (better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
        pval[(size_t)m * nblk + blk] = bv;
        pidx[(size_t)m * nblk + blk] = bi;
    }
}

int qb_launch_argmax_partial(qb_ctx *ctx, const float *x, uint32_t M, uint32_t n, uint32_t stride, float *pval,
                             int32_t *pidx, uint32_t nblk) {
    dim3 grid(nblk, M);
    QB_CUDA(qb_launch_pdl(ctx->stream, argmax_partial_kernel, dim3(grid), dim3(256), (size_t)(0), x, n, stride, pval, pidx, nblk));
    QB_LAUNCHED(ctx, "argmax_partial_kernel");
    return QB_OK;
}

__global__ void argmax_final_kernel(const float *pval, const int32_t *pidx, uint32_t nblk, int32_t *out) {
    const uint32_t m = blockIdx.x;
    if (threadIdx.x != 0) return;
    float bv = pval[(size_t)m * nblk];
    int bi = pidx[(size_t)m * nblk];
    for (uint32_t b = 1; b < nblk; ++b)
        if (better(pval[(size_t)m * nblk + b], pidx[(size_t)m * nblk + b], bv, bi)) {
            bv = pval[(size_t)m * nblk + b];
            bi = pidx[(size_t)m * nblk + b];
        }
    out[m] = bi;
}

extern "C" int qb_argmax_rows(qb_ctx *ctx, const float *x_dev, uint32_t M, uint32_t n, uint32_t stride, int32_t *out_dev) {
    QB_REQUIRE(ctx && x_dev && out_dev && M > 0 && n > 0, "qb_argmax_rows: bad arguments");
    void *scr = nullptr;
    const uint32_t nblk = QB_ARGMAX_BLOCKS;
    QB_TRY(qb_ctx_scratch(ctx, (size_t)M * nblk * 8, &scr));
    float *pval = (float *)scr;
    int32_t *pidx = (int32_t *)(pval + (size_t)M * nblk);
    QB_TRY(qb_launch_argmax_partial(ctx, x_dev, M, n, stride, pval, pidx, nblk));
    argmax_final_kernel<<<M, 32, 0, ctx->stream>>>(pval, pidx, nblk, out_dev);
    QB_LAUNCHED(ctx, "argmax_final_kernel");
    return QB_OK;
}
