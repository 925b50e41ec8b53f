// Activation quantisers and the fused element-wise kernels around the Q8 GEMMs.
#include "qb_internal.h"

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
// A thread-block cluster of 8 CTAs works on one row: CTA c owns a contiguous eighth of the row's 32-blocks,
// a thread owns 4 consecutive elements (8 threads per 32-block, 16-byte loads and stores), everything stays in
// registers.  The sum of squares crosses the cluster once: every CTA pushes its partial into the shared memory
// of all 8 (st.shared::cluster) and one cluster barrier later each CTA adds the 8 partials in rank order, so all
// of them apply the same scale.  P = passes of 32 blocks per CTA.
constexpr uint32_t NQ_CLUSTER = 8, NQ_THREADS = 256;

__device__ __forceinline__ float4 ld4(const float *p, bool vec) {
    if (vec) return *reinterpret_cast<const float4 *>(p);
    return make_float4(p[0], p[1], p[2], p[3]);
}
__device__ __forceinline__ void st4(float *p, float4 v, bool vec) {
    if (vec) *reinterpret_cast<float4 *>(p) = v;
    else { p[0] = v.x; p[1] = v.y; p[2] = v.z; p[3] = v.w; }
}

// The two phases of one thread's 4 consecutive elements.
struct NqRow {
    const float *x, *parts;
    size_t pstride;
    bool vx, vp, vh;
};
__device__ __forceinline__ NqRow nq_row(const NormQuantArgs &a, uint32_t m, uint32_t vec) {
    NqRow r;
    const uint32_t src = a.row_map ? (uint32_t)a.row_map[m] : m;
    r.x = a.x ? a.x + (size_t)src * a.x_stride : nullptr;
    r.parts = a.parts ? a.parts + (size_t)m * a.part_ld : nullptr;
    r.pstride = (size_t)a.M * a.part_ld;
    r.vx = vec & 1; r.vp = vec & 2; r.vh = vec & 4;
    return r;
}
// loads: x + split partials (segments ascending, then the residual), gains; returns the 4 values and adds their
// squares to ss in element order
__device__ __forceinline__ void nq_load(const NormQuantArgs &a, const NqRow &r, uint32_t i, float4 &v, float4 &g, float &ss) {
    float4 xv = r.x ? ld4(r.x + i, r.vx) : make_float4(0.f, 0.f, 0.f, 0.f);
    g = a.w ? ld4(a.w + i, true) : make_float4(1.f, 1.f, 1.f, 1.f);
    if (a.S > 0) {
        float4 q[8];  // all segment loads are issued before the first add (S <= 8)
#pragma unroll
        for (uint32_t s = 0; s < 8; ++s) q[s] = s < a.S ? ld4(r.parts + s * r.pstride + i, r.vp) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 y = q[0];
#pragma unroll
        for (uint32_t s = 1; s < 8; ++s)
            if (s < a.S) { y.x += q[s].x; y.y += q[s].y; y.z += q[s].z; y.w += q[s].w; }
        if (r.x) { xv.x += y.x; xv.y += y.y; xv.z += y.z; xv.w += y.w; } else xv = y;
    }
    v = xv;
    ss = __fmaf_rn(xv.x, xv.x, ss); ss = __fmaf_rn(xv.y, xv.y, ss); ss = __fmaf_rn(xv.z, xv.z, ss); ss = __fmaf_rn(xv.w, xv.w, ss);
}
// residual stream out, normalise, quantise (8 lanes = one 32-block); b = block index, i = first element
__device__ __forceinline__ void nq_finish(const NormQuantArgs &a, const NqRow &r, uint32_t m, uint32_t b, uint32_t i, uint32_t lane,
                                          float4 t, float4 g, float scale) {
    if (a.h_out) st4(a.h_out + (size_t)m * a.h_stride + i, t, r.vh);
    if (a.w) {
        t.x = __fmul_rn(__fmul_rn(t.x, scale), g.x); t.y = __fmul_rn(__fmul_rn(t.y, scale), g.y);
        t.z = __fmul_rn(__fmul_rn(t.z, scale), g.z); t.w = __fmul_rn(__fmul_rn(t.w, scale), g.w);
    }
    if (a.normed_out) st4(a.normed_out + (size_t)m * a.n + i, t, true);
    if (a.q) {
        // arithmetic of quantize_mmq_q8_1_kernel (src/mmvq_q8.cu:694-721)
        const uint32_t grp = 0xffu << (lane & 24);
        float amax = fmaxf(fmaxf(fabsf(t.x), fabsf(t.y)), fmaxf(fabsf(t.z), fabsf(t.w)));
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(grp, amax, o));
        const float d_inv = (amax == 0.0f) ? 0.0f : __fdiv_rn(127.0f, amax);
        uint32_t packed = 0;
        if (amax != 0.0f) {
            const int q0 = __float2int_rn(__fmul_rn(t.x, d_inv)), q1 = __float2int_rn(__fmul_rn(t.y, d_inv));
            const int q2 = __float2int_rn(__fmul_rn(t.z, d_inv)), q3 = __float2int_rn(__fmul_rn(t.w, d_inv));
            packed = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
        }
        *reinterpret_cast<uint32_t *>(a.q + (size_t)m * a.q_pitch + a.q_col_off + i) = packed;
        if ((lane & 7) == 0) a.d[(size_t)(a.d_kb_off + b) * a.d_ld + m] = (amax == 0.0f) ? 0.0f : __fdiv_rn(1.0f, d_inv);
    }
}

template <int P>
__global__ void __launch_bounds__(NQ_THREADS) norm_quant_kernel(NormQuantArgs a, uint32_t vec) {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");   // "this CTA runs": awaited before the pushes
    QB_PDL_ENTER();
    __shared__ float red[NQ_THREADS / 32];
    __shared__ float cl_part[NQ_CLUSTER];
    uint32_t crank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
    const uint32_t m = blockIdx.x / NQ_CLUSTER, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t nblk = a.n / 32, per = (nblk + NQ_CLUSTER - 1) / NQ_CLUSTER;
    const uint32_t b0 = crank * per, b1 = min(nblk, b0 + per), sub = tid & 7;
    const NqRow r = nq_row(a, m, vec);

    float4 v[P], g[P];
    float ss = 0.0f;
#pragma unroll
    for (int p = 0; p < P; ++p) {
        const uint32_t b = b0 + (tid >> 3) + 32 * p;
        v[p] = make_float4(0.f, 0.f, 0.f, 0.f);
        g[p] = make_float4(1.f, 1.f, 1.f, 1.f);
        if (b < b1) nq_load(a, r, b * 32 + sub * 4, v[p], g[p], ss);
    }
    float scale = 1.0f;
    if (a.w) {   // uniform over the cluster
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");            // all 8 CTAs are running
        if (tid < NQ_CLUSTER) {
            float tot = 0.0f;
#pragma unroll
            for (int i = 0; i < (int)NQ_THREADS / 32; ++i) tot += red[i];
            uint32_t local = (uint32_t)__cvta_generic_to_shared(&cl_part[crank]), remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(tid));
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(tot) : "memory");
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        float tot = 0.0f;
#pragma unroll
        for (int i = 0; i < (int)NQ_CLUSTER; ++i) tot += cl_part[i];
        scale = rsqrtf(tot / (float)a.n + a.eps);
    }
#pragma unroll
    for (int p = 0; p < P; ++p) {
        const uint32_t b = b0 + (tid >> 3) + 32 * p;
        if (b >= b1) continue;          // whole 8-thread groups leave together; the shuffles stay inside a group
        nq_finish(a, r, m, b, b * 32 + sub * 4, lane, v[p], g[p], scale);
    }
    if (!a.w) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // complete the opening arrive
}

template <int P>
static cudaError_t launch_norm_quant(cudaStream_t stream, const NormQuantArgs &a, uint32_t vec) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.M * NQ_CLUSTER);
    cfg.blockDim = dim3(NQ_THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = NQ_CLUSTER;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, norm_quant_kernel<P>, a, vec);
}

int qb_launch_norm_quant(qb_ctx *ctx, const NormQuantArgs &a) {
    QB_REQUIRE(a.M > 0 && a.n > 0 && a.n % 32 == 0 && a.S <= 8, "norm_quant: bad shape M=%u n=%u S=%u", a.M, a.n, a.S);
    const uint32_t per = (a.n / 32 + NQ_CLUSTER - 1) / NQ_CLUSTER;
    QB_REQUIRE(per <= 128, "norm_quant: row of %u floats is longer than the kernel's 32768", a.n);
    QB_REQUIRE(((uintptr_t)a.w & 15) == 0 && ((uintptr_t)a.normed_out & 15) == 0 && ((uintptr_t)a.q & 3) == 0 &&
               a.q_pitch % 4 == 0 && a.q_col_off % 4 == 0, "norm_quant: gain / output buffers must be 16-byte aligned");
    auto al = [](const void *p, size_t stride) { return ((uintptr_t)p & 15) == 0 && stride % 4 == 0; };
    const uint32_t vec = (al(a.x, a.x_stride) ? 1u : 0u) | (al(a.parts, a.part_ld) ? 2u : 0u) | (al(a.h_out, a.h_stride) ? 4u : 0u);
    if (per <= 32) QB_CUDA(launch_norm_quant<1>(ctx->stream, a, vec));
    else if (per <= 64) QB_CUDA(launch_norm_quant<2>(ctx->stream, a, vec));
    else QB_CUDA(launch_norm_quant<4>(ctx->stream, a, vec));
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
// ileave = 0: gate cols [0,F), up cols [F,2F); ileave = 64: the fused weight's interleaved order (hidden index c
// has its gate at (c/64)*128 + c%64 and its up 64 further).
__global__ void swiglu_quant_kernel(const float *__restrict__ gu, uint32_t gu_stride, uint32_t F, int8_t *q,
                                    uint32_t q_pitch, float *d, uint32_t d_ld, uint32_t S, size_t pstride, uint32_t ileave) {
    QB_PDL_ENTER();
    const uint32_t b = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, m = blockIdx.y, lane = threadIdx.x & 31;
    if (b >= F / 32) return;
    const uint32_t c = b * 32 + lane;
    const uint32_t gi = ileave ? (c / ileave) * 2 * ileave + c % ileave : c, ui = ileave ? gi + ileave : F + c;
    const float g = qb_ldsum(gu, (size_t)m * gu_stride + gi, S, pstride);
    const float u = qb_ldsum(gu, (size_t)m * gu_stride + ui, S, pstride);
    quant_block_store(qb_swiglu(g, u), lane, q + (size_t)m * q_pitch + b * 32, d + (size_t)b * d_ld + m);
}

int qb_launch_swiglu_quant(qb_ctx *ctx, const float *gu, uint32_t gu_stride, uint32_t M, uint32_t F, int8_t *q,
                           uint32_t q_pitch, float *d, uint32_t d_ld, uint32_t S, size_t pstride, uint32_t ileave) {
    dim3 grid((F / 32 + 7) / 8, M);
    QB_CUDA(qb_launch_pdl(ctx->stream, swiglu_quant_kernel, dim3(grid), dim3(256), (size_t)(0), gu, gu_stride, F, q, q_pitch, d, d_ld, S, pstride,
                          ileave));
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

// Same reduction, leaving the winning value beside the index (DeviceArgmax {token, logit}).
__global__ void argmax_final_val_kernel(const float *pval, const int32_t *pidx, uint32_t nblk, int32_t *out, float *out_val, uint32_t out_off) {
    const uint32_t m = blockIdx.x, lane = threadIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (uint32_t j = lane; j < nblk; j += 32) {
        const float v = pval[(size_t)m * nblk + j];
        const int i = pidx[(size_t)m * nblk + j];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, bv, o);
        const int i = __shfl_xor_sync(0xffffffffu, bi, o);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    if (lane == 0) { out[out_off + m] = bi; out_val[out_off + m] = bv; }
}

// argmax_to_buffer / argmax_batch with logits (include/qw3/device_backend.hpp:2456-2497): token and value of row m go to
// tok_dev[out_offset + m], val_dev[out_offset + m].
extern "C" int qb_argmax_rows_val(qb_ctx *ctx, const float *x_dev, uint32_t M, uint32_t n, uint32_t stride, int32_t *tok_dev, float *val_dev,
                                  uint32_t out_offset) {
    QB_REQUIRE(ctx && x_dev && tok_dev && val_dev && M > 0 && n > 0, "qb_argmax_rows_val: bad arguments");
    void *scr = nullptr;
    const uint32_t nblk = QB_ARGMAX_BLOCKS;
    QB_TRY(qb_ctx_scratch(ctx, (size_t)M * nblk * 8, &scr));
    float *pval = (float *)scr;
    int32_t *pidx = (int32_t *)(pval + (size_t)M * nblk);
    QB_TRY(qb_launch_argmax_partial(ctx, x_dev, M, n, stride, pval, pidx, nblk));
    argmax_final_val_kernel<<<M, 32, 0, ctx->stream>>>(pval, pidx, nblk, tok_dev, val_dev, out_offset);
    QB_LAUNCHED(ctx, "argmax_final_val_kernel");
    return QB_OK;
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
