// Q8_0 x Q8 product on CUDA cores: weight-streaming kernel for a handful of activation rows.
//
// Stands in for mul_mat_vec_q8_0_kernel and its fused variants (src/mmvq_q8.cu:195-1113) on the
// decode / draft / (k+1)-row verify shapes.  Arithmetic per output: exact int32 dot of each
// 32-block (dp4a), acc = fma(d_w*d_x, float(dot), acc) over the blocks of a K segment in ascending
// order (the per-output update of src/mmq_q8.cu:1738-1748); one partial sum per segment.
//
// Data movement: a CTA owns 128 weight rows and one K segment.  Each stage of a 4-deep cp.async
// pipeline copies one 17 KB weight record (128 rows x 128 bytes of quants, already in the 16-byte
// XOR-swizzled order that makes "one thread = one weight row" reads bank-conflict free, followed by
// its fp16 scales) as one contiguous read; activations of the pass are staged beside it and read as
// warp broadcasts.
#include "qb_internal.h"

#include <mutex>

int qb_prof_begin(qb_ctx *ctx);
int qb_prof_end(qb_ctx *ctx, double bytes);

namespace {

constexpr int TILE_N = 128;
constexpr int CHUNK = 128;
constexpr int NSTAGE = 4;
constexpr int THREADS = 256;

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__host__ __device__ inline uint32_t seg_begin(uint32_t s, uint32_t S, uint32_t nchunks) {
    return (uint32_t)(((uint64_t)s * nchunks) / S);
}

template <int MPT>
struct Smem {
    static constexpr int NC = 2 * MPT;
    static constexpr int WQ = TILE_N * CHUNK;          // 16384
    static constexpr int WD = 4 * TILE_N * 2;          // 1024
    static constexpr int XQ = NC * CHUNK;
    static constexpr int STAGE = WQ + WD + XQ;
    static constexpr int TOTAL = STAGE * NSTAGE;
};

template <int MPT>
__global__ void __launch_bounds__(THREADS) gemm_dp4a_kernel(const uint8_t *__restrict__ rec, uint32_t K, uint32_t N,
                                                            const int8_t *__restrict__ xq, const float *__restrict__ xd,
                                                            uint32_t M, uint32_t xld, float *__restrict__ part, uint32_t S) {
    QB_PDL_ENTER();
    using L = Smem<MPT>;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t tid = threadIdx.x;
    const uint32_t row0 = blockIdx.x * TILE_N;
    const uint32_t seg = blockIdx.y;
    const uint32_t m0 = blockIdx.z * L::NC;
    const uint32_t nchunks = K / CHUNK;
    const uint32_t c_begin = seg_begin(seg, S, nchunks), c_end = seg_begin(seg + 1, S, nchunks);
    const uint32_t n_it = c_end - c_begin;

    auto load_stage = [&](uint32_t it, uint32_t slot) {
        uint8_t *st = smem + (size_t)slot * L::STAGE;
        const uint32_t k0 = (c_begin + it) * CHUNK;
        // the record of (row tile, chunk) is already the shared-memory image: a straight 17 KB copy
        const uint8_t *src = rec + ((size_t)blockIdx.x * nchunks + c_begin + it) * QB_REC_BYTES;
        for (uint32_t c = tid; c < QB_REC_BYTES / 16; c += THREADS) cp_async16(st + c * 16, src + c * 16, true);
        if (tid < L::NC * 8) {
            const uint32_t c = tid, col = c >> 3, p = c & 7;
            const bool valid = m0 + col < M;
            cp_async16(st + L::WQ + L::WD + col * CHUNK + p * 16, xq + (size_t)(valid ? m0 + col : 0) * K + k0 + p * 16, valid);
        }
    };

    const uint32_t r = tid & 127, cg = tid >> 7;
    float acc[MPT];
#pragma unroll
    for (int j = 0; j < MPT; ++j) acc[j] = 0.0f;

    for (uint32_t s = 0; s < NSTAGE - 1; ++s) {
        if (s < n_it) load_stage(s, s);
        cp_async_commit();
    }
    for (uint32_t it = 0; it < n_it; ++it) {
        cp_async_wait<NSTAGE - 2>();
        __syncthreads();
        if (it + NSTAGE - 1 < n_it) load_stage(it + NSTAGE - 1, (it + NSTAGE - 1) % NSTAGE);
        cp_async_commit();

        const uint8_t *st = smem + (size_t)(it % NSTAGE) * L::STAGE;
        const uint32_t kb0 = (c_begin + it) * 4;
        float sx[4][MPT];
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
#pragma unroll
            for (int j = 0; j < MPT; ++j) {
                const uint32_t m = m0 + cg * MPT + j;
                sx[kb][j] = (m < M) ? __ldg(xd + (size_t)(kb0 + kb) * xld + m) : 0.0f;
            }
        const __half *sd = reinterpret_cast<const __half *>(st + L::WQ);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            const int4 w0 = *reinterpret_cast<const int4 *>(st + r * CHUNK + (((2 * kb) ^ (r & 7)) << 4));
            const int4 w1 = *reinterpret_cast<const int4 *>(st + r * CHUNK + (((2 * kb + 1) ^ (r & 7)) << 4));
            const float dw = __half2float(sd[kb * TILE_N + r]);
#pragma unroll
            for (int j = 0; j < MPT; ++j) {
                const uint8_t *xb = st + L::WQ + L::WD + (cg * MPT + j) * CHUNK + kb * 32;
                const int4 x0 = *reinterpret_cast<const int4 *>(xb);
                const int4 x1 = *reinterpret_cast<const int4 *>(xb + 16);
                int c = __dp4a(w0.x, x0.x, 0);
                c = __dp4a(w0.y, x0.y, c);
                c = __dp4a(w0.z, x0.z, c);
                c = __dp4a(w0.w, x0.w, c);
                c = __dp4a(w1.x, x1.x, c);
                c = __dp4a(w1.y, x1.y, c);
                c = __dp4a(w1.z, x1.z, c);
                c = __dp4a(w1.w, x1.w, c);
                acc[j] = __fmaf_rn(__fmul_rn(dw, sx[kb][j]), (float)c, acc[j]);
            }
        }
    }
    cp_async_wait<0>();
    const uint32_t row = row0 + r;
    if (row < N) {
#pragma unroll
        for (int j = 0; j < MPT; ++j) {
            const uint32_t m = m0 + cg * MPT + j;
            if (m < M) part[((size_t)seg * M + m) * N + row] = acc[j];
        }
    }
}

template <int MPT>
int launch(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part, uint32_t S) {
    using L = Smem<MPT>;
    // the attribute belongs to the current device: set on every launch (a process may drive several GPUs)
    QB_CUDA(cudaFuncSetAttribute(gemm_dp4a_kernel<MPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    dim3 grid(w->rows_pad / TILE_N, S, (M + L::NC - 1) / L::NC);
    QB_CUDA(qb_launch_pdl(ctx->stream, gemm_dp4a_kernel<MPT>, dim3(grid), dim3(THREADS), (size_t)(L::TOTAL), w->rec, w->cols, w->rows, q, d, M, qb_act_ld(M), part, S));
    QB_LAUNCHED(ctx, "gemm_dp4a_kernel");
    return QB_OK;
}

// Exact int32 block dots, out[m][n][kb] (test aid for the integer part).
__global__ void block_dots_kernel(const uint8_t *__restrict__ rec, uint32_t K, uint32_t N, const int8_t *__restrict__ xq,
                                  uint32_t M, int32_t *out) {
    const uint32_t nb = K / 32;
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)N * nb) return;
    const uint32_t n = (uint32_t)(idx / nb), kb = (uint32_t)(idx % nb);
    int wv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) wv[i] = *reinterpret_cast<const int *>(rec + qb_q_offset(K, n, kb * 32 + i * 4));
    for (uint32_t m = 0; m < M; ++m) {
        const int *xp = reinterpret_cast<const int *>(xq + (size_t)m * K + (size_t)kb * 32);
        int c = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) c = __dp4a(wv[i], xp[i], c);
        out[((size_t)m * N + n) * nb + kb] = c;
    }
}

}  // namespace

uint32_t qb_ksplit(uint32_t N, uint32_t K) {
    const uint32_t tiles = (N + 127) / 128, nchunks = K / 128;
    // about one (row tile, segment) unit per resident CTA of the small-batch kernel (two per SM on a 148-SM
    // part), at most 8 segments.  The count depends on the weight's shape only, never on the batch.
    uint32_t S = 296 / std::max(tiles, 1u);
    S = std::max(1u, std::min(S, 8u));
    S = std::min(S, std::max(nchunks, 1u));
    return S;
}
extern "C" uint32_t qb_ksplit_policy(uint32_t N, uint32_t K) { return qb_ksplit(N, K); }

int qb_ffn_gate_up_swiglu(qb_ctx *ctx, const qb_weight *w, const int8_t *xq, const float *xd, uint32_t M, float *act, float *parts,
                          size_t parts_floats, int8_t *hq, uint32_t hq_pitch, float *hd, uint32_t hd_ld, int gemm_impl, int mode) {
    const uint32_t F = w->rows / 2, S = qb_ksplit(w->rows, w->cols);
    const bool can_fuse = M <= 16 && S == 1 && w->rows % 128 == 0 && w->cols / 128 > 8 && qb_gemm_tc_supported(w, M) && gemm_impl != 1;
    QB_REQUIRE(mode != 2 || can_fuse, "gate/up + SwiGLU in one launch needs M <= 16, one K segment and K > 1024");
    if (can_fuse && mode != 1) {
        QbGemmSwiglu sw;
        sw.q = hq; sw.d = hd; sw.q_pitch = hq_pitch; sw.d_ld = hd_ld;
        if (!ctx->prof_on) return qb_launch_gemm_tc(ctx, w, xq, xd, M, nullptr, 1, nullptr, nullptr, &sw);
        QB_TRY(qb_prof_begin(ctx));
        const int st = qb_launch_gemm_tc(ctx, w, xq, xd, M, nullptr, 1, nullptr, nullptr, &sw);
        // weight once, int8 activations + scales in, int8 hidden + scales out (no fp32 partials leave the kernel)
        QB_TRY(qb_prof_end(ctx, (double)w->rows * w->cols / 32.0 * 34.0 + (double)M * w->cols * 1.125 + (double)M * F * 1.125));
        return st;
    }
    if (S == 1) {
        QB_TRY(qb_launch_gemm(ctx, w, xq, xd, M, act, 1, gemm_impl));
        return qb_launch_swiglu_quant(ctx, act, w->rows, M, F, hq, hq_pitch, hd, hd_ld, 1, 0, 64);
    }
    QB_REQUIRE((size_t)S * M * w->rows <= parts_floats, "split scratch too small");
    QB_TRY(qb_launch_gemm(ctx, w, xq, xd, M, parts, S, gemm_impl));
    return qb_launch_swiglu_quant(ctx, parts, w->rows, M, F, hq, hq_pitch, hd, hd_ld, S, (size_t)M * w->rows, 64);
}

int qb_launch_gemm_dp4a(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part,
                        uint32_t S) {
    QB_REQUIRE(M > 0 && S > 0 && S <= w->cols / 128, "gemm: bad M=%u or ksplit=%u", M, S);
    if (M <= 2) return launch<1>(ctx, w, q, d, M, part, S);
    if (M <= 4) return launch<2>(ctx, w, q, d, M, part, S);
    return launch<4>(ctx, w, q, d, M, part, S);
}

static int gemm_dispatch(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part,
                         uint32_t S, int impl);

// Algorithmic bytes of one launch: the Q8_0 weight once (34 B per 32 weights), the quantised
// activations (int8 + one fp32 scale per 32) and the fp32 partial sums written.
static double gemm_bytes(const qb_weight *w, uint32_t M, uint32_t S) {
    return (double)w->rows * w->cols / 32.0 * 34.0 + (double)M * w->cols * 1.125 + (double)S * M * w->rows * 4.0;
}

// Per-launch timing of the GEMM kernels (qb_prof_*): an event pair around the launch and its algorithmic bytes.
int qb_prof_begin(qb_ctx *ctx) {
    if (ctx->prof_used + 2 > ctx->prof_ev.size()) {
        for (int i = 0; i < 256; ++i) {
            cudaEvent_t e;
            QB_CUDA(cudaEventCreate(&e));
            ctx->prof_ev.push_back(e);
        }
    }
    QB_CUDA(cudaEventRecord(ctx->prof_ev[ctx->prof_used], ctx->stream));
    return QB_OK;
}
int qb_prof_end(qb_ctx *ctx, double bytes) {
    QB_CUDA(cudaEventRecord(ctx->prof_ev[ctx->prof_used + 1], ctx->stream));
    ctx->prof_used += 2;
    ctx->prof_bytes.push_back(bytes);
    return QB_OK;
}

int qb_launch_gemm(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part,
                   uint32_t S, int impl) {
    if (!ctx->prof_on) return gemm_dispatch(ctx, w, q, d, M, part, S, impl);
    QB_TRY(qb_prof_begin(ctx));
    const int st = gemm_dispatch(ctx, w, q, d, M, part, S, impl);
    QB_TRY(qb_prof_end(ctx, gemm_bytes(w, M, S)));
    return st;
}

extern "C" int qb_prof_enable(qb_ctx *ctx, int on) {
    ctx->prof_on = on != 0;
    ctx->prof_used = 0;
    ctx->prof_bytes.clear();
    return QB_OK;
}

extern "C" int qb_prof_summary(qb_ctx *ctx, double *total_ms, double *total_bytes, int64_t *launches) {
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    double ms = 0.0, bytes = 0.0;
    for (size_t i = 0; i + 1 < ctx->prof_used; i += 2) {
        float t = 0.0f;
        QB_CUDA(cudaEventElapsedTime(&t, ctx->prof_ev[i], ctx->prof_ev[i + 1]));
        ms += t;
        bytes += ctx->prof_bytes[i / 2];
    }
    *total_ms = ms; *total_bytes = bytes; *launches = (int64_t)(ctx->prof_used / 2);
    return QB_OK;
}

static int gemm_dispatch(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part,
                         uint32_t S, int impl) {
    if (impl == 2) {
        if (!qb_gemm_tc_supported(w, M))
            return qb_fail(QB_ERR_UNSUPPORTED, "tensor-core GEMM does not support this shape");
        return qb_launch_gemm_tc(ctx, w, q, d, M, part, S);
    }
    // automatic choice (measured): the tensor-core kernel everywhere except the matvec over a very tall weight
    // (the LM head at M <= 2), where three CUDA-core CTAs per SM stream a little faster.  QW3B200_TC_MIN_M
    // overrides: the tensor-core kernel is then used from that many activation rows upwards only.
    static const uint32_t tc_min_m = []() {
        const char *e = getenv("QW3B200_TC_MIN_M");
        return (e && *e) ? (uint32_t)strtoul(e, nullptr, 10) : 0u;
    }();
    const bool tall_matvec = M <= 2 && w->rows_pad / 128 >= 600;
    if (impl == 0 && M >= tc_min_m && !(tc_min_m == 0 && tall_matvec) && qb_gemm_tc_supported(w, M))
        return qb_launch_gemm_tc(ctx, w, q, d, M, part, S);
    return qb_launch_gemm_dp4a(ctx, w, q, d, M, part, S);
}

extern "C" int qb_q8_gemm_partials(qb_ctx *ctx, const qb_weight *w, const int8_t *q_dev, const float *d_dev, uint32_t M,
                                   float *part_dev, uint32_t ksplit, int impl) {
    QB_REQUIRE(ctx && w && q_dev && d_dev && part_dev, "qb_q8_gemm_partials: null argument");
    const uint32_t S = ksplit ? ksplit : qb_ksplit(w->rows, w->cols);
    return qb_launch_gemm(ctx, w, q_dev, d_dev, M, part_dev, S, impl);
}

extern "C" int qb_q8_0_matmul(qb_ctx *ctx, const qb_weight *w, const float *x_dev, uint32_t M, uint32_t x_stride,
                              float *y_dev, uint32_t y_stride, uint32_t ksplit, int impl) {
    QB_REQUIRE(ctx && w && x_dev && y_dev && M > 0, "qb_q8_0_matmul: bad arguments");
    QB_REQUIRE(x_stride >= w->cols && y_stride >= w->rows, "qb_q8_0_matmul: strides smaller than the matrix");
    const uint32_t S = ksplit ? ksplit : qb_ksplit(w->rows, w->cols);
    const uint32_t K = w->cols, N = w->rows, ld = qb_act_ld(M);
    const size_t qbytes = ((size_t)M * K + 255) & ~(size_t)255;
    const size_t dbytes = (((size_t)(K / 32) * ld * 4) + 255) & ~(size_t)255;
    const size_t pbytes = (size_t)S * M * N * 4;
    void *scr = nullptr;
    QB_TRY(qb_ctx_scratch(ctx, qbytes + dbytes + pbytes, &scr));
    int8_t *q = (int8_t *)scr;
    float *d = (float *)((uint8_t *)scr + qbytes);
    float *part = (float *)((uint8_t *)scr + qbytes + dbytes);
    QB_TRY(qb_quantize_act(ctx, x_dev, M, K, x_stride, q, d));
    if (S == 1 && y_stride == N) return qb_launch_gemm(ctx, w, q, d, M, y_dev, 1, impl);
    QB_TRY(qb_launch_gemm(ctx, w, q, d, M, part, S, impl));
    return qb_launch_reduce_parts(ctx, part, S, M, N, y_dev, y_stride);
}

extern "C" int qb_q8_block_dots(qb_ctx *ctx, const qb_weight *w, const int8_t *q_dev, uint32_t M, int32_t *out_dev) {
    QB_REQUIRE(ctx && w && q_dev && out_dev, "qb_q8_block_dots: null argument");
    const uint64_t total = (uint64_t)w->rows * (w->cols / 32);
    block_dots_kernel<<<(uint32_t)((total + 255) / 256), 256, 0, ctx->stream>>>(w->rec, w->cols, w->rows, q_dev, M, out_dev);
    QB_LAUNCHED(ctx, "block_dots_kernel");
    return QB_OK;
}

// ---- matmul for callers that must not allocate ---------------------------------------------------
// qb_q8_0_matmul keeps its work area (int8 activations, their scales, the K-segment partial sums) in a
// context buffer that grows with cudaMalloc.  Some hosts cannot afford that: an inference server whose own
// arena already owns every byte of the device (cudaMalloc would fail or fragment it), or a decode loop in
// which the implicit device-wide synchronisation of cudaMalloc / cudaFree is not acceptable.  This variant
// needs no allocation at all: its work area is the fixed array below, part of the library image, so every
// GPU that loads the library holds these QB_NOALLOC_SCRATCH_BYTES until the process exits.
static const size_t QB_NOALLOC_SCRATCH_BYTES = (size_t)8 << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[QB_NOALLOC_SCRATCH_BYTES];

// Device address of the array for the current device.  The symbol name is only a host-side handle: the
// address a kernel may use comes from cudaGetSymbolAddress, once per device, with that device current.
static int noalloc_scratch_ptr(qb_ctx *ctx, unsigned char **out) {
    static unsigned char *ptrs[64] = {nullptr};
    static std::mutex lock;
    QB_REQUIRE(ctx->device >= 0 && ctx->device < 64, "no-alloc matmul: device ordinal %d out of range", ctx->device);
    std::lock_guard<std::mutex> guard(lock);
    if (!ptrs[ctx->device]) {
        QB_CUDA(cudaSetDevice(ctx->device));
        void *p = nullptr;
        QB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        QB_REQUIRE(p != nullptr, "no-alloc matmul: cudaGetSymbolAddress returned a null address");
        ptrs[ctx->device] = (unsigned char *)p;
    }
    *out = ptrs[ctx->device];
    return QB_OK;
}

extern "C" int qb_q8_0_matmul_noalloc(qb_ctx *ctx, const qb_weight *w, const float *x_dev, uint32_t M, uint32_t x_stride,
                                      float *y_dev, uint32_t y_stride, uint32_t ksplit) {
    QB_REQUIRE(ctx && w && x_dev && y_dev && M > 0, "qb_q8_0_matmul_noalloc: bad arguments");
    QB_REQUIRE(x_stride >= w->cols && y_stride >= w->rows, "qb_q8_0_matmul_noalloc: strides smaller than the matrix");
    const uint32_t S = ksplit ? ksplit : qb_ksplit(w->rows, w->cols);
    const uint32_t K = w->cols, N = w->rows, ld = qb_act_ld(M);
    const bool direct = S == 1 && y_stride == N;                    // a single segment is written straight to y
    const size_t qbytes = ((size_t)M * K + 255) & ~(size_t)255;
    const size_t dbytes = (((size_t)(K / 32) * ld * 4) + 255) & ~(size_t)255;
    const size_t pbytes = direct ? 0 : (size_t)S * M * N * 4;
    if (qbytes + dbytes + pbytes > QB_NOALLOC_SCRATCH_BYTES)
        return qb_fail(QB_ERR_CAPACITY,
                       "qb_q8_0_matmul_noalloc: M=%u rows of a %ux%u weight with %u K segments need %zu bytes of work area, "
                       "the built-in area holds %zu; use qb_q8_0_matmul", M, N, K, S, qbytes + dbytes + pbytes,
                       QB_NOALLOC_SCRATCH_BYTES);
    unsigned char *scr = nullptr;
    QB_TRY(noalloc_scratch_ptr(ctx, &scr));
    int8_t *q = (int8_t *)scr;
    float *d = (float *)(scr + qbytes);
    float *part = (float *)(scr + qbytes + dbytes);
    // the array keeps whatever the previous call left: the scale rows have padding columns the quantiser
    // does not write, so that region starts from zero on every call
    QB_CUDA(cudaMemsetAsync(d, 0, dbytes, ctx->stream));
    QB_TRY(qb_quantize_act(ctx, x_dev, M, K, x_stride, q, d));
    if (direct) return qb_launch_gemm_dp4a(ctx, w, q, d, M, y_dev, 1);
    QB_TRY(qb_launch_gemm_dp4a(ctx, w, q, d, M, part, S));
    return qb_launch_reduce_parts(ctx, part, S, M, N, y_dev, y_stride);
}
