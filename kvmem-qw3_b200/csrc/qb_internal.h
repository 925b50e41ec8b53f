// Internal declarations shared by the CUDA translation units of libqw3b200.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <tuple>
#include <vector>

#include "../../include/qw3b200.h"
#include "../../include/qw3b200_synth.h"

// ---- error convention: thread-local message, integer status ------------------------------
int qb_fail(int code, const char *fmt, ...);
#define QB_CUDA(expr)                                                                              \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return qb_fail(QB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),   \
                           __FILE__, __LINE__);                                                    \
    } while (0)
#define QB_REQUIRE(cond, ...)                                                                      \
    do {                                                                                           \
        if (!(cond)) return qb_fail(QB_ERR_INVALID, __VA_ARGS__);                                  \
    } while (0)
#define QB_TRY(expr)                                                                               \
    do {                                                                                           \
        int _s = (expr);                                                                           \
        if (_s != QB_OK) return _s;                                                                \
    } while (0)
// Counts a kernel launch and checks the launch status.
#define QB_LAUNCHED(ctx, name)                                                                     \
    do {                                                                                           \
        (ctx)->launches++;                                                                         \
        if ((ctx)->trace_on) qb_trace_mark(ctx, name);                                             \
        cudaError_t _e = cudaGetLastError();                                                       \
        if (_e != cudaSuccess)                                                                     \
            return qb_fail(QB_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e));  \
    } while (0)

// Programmatic dependent launch: every kernel of the step is launched with stream serialisation relaxed,
// announces its own dependents at once and then waits for the complete preceding grid (memory flushed), so
// scheduling and launch latency of kernel N+1 overlap the tail of kernel N; semantics stay those of a stream.
#define QB_PDL_ENTER()                                                           \
    do {                                                                         \
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");          \
        asm volatile("griddepcontrol.wait;" ::: "memory");                       \
    } while (0)
template <typename K, typename... Args>
inline cudaError_t qb_launch_pdl(cudaStream_t stream, K kernel, dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

struct qb_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    int64_t launches = 0;
    float *normal_table_dev = nullptr;     // 65536-entry inverse-normal table for seeded weights
    void *flush_buf = nullptr;             // > L2 bytes, written by qb_flush_l2
    size_t flush_bytes = 0;
    int *err_flag_dev = nullptr;           // set by kernels whose bounded waits ran out
    // optional launch trace (qb_trace_*): one event after every launch, durations = event deltas
    bool trace_on = false;
    std::vector<cudaEvent_t> trace_ev;
    std::vector<const char *> trace_names;
    size_t trace_used = 0;
    // optional per-launch timing of the GEMM kernels (qb_prof_*): event pairs + algorithmic bytes
    unsigned long long *tl_dev = nullptr;  // device timeline slots
    uint32_t tl_cap = 0, tl_used = 0;
    std::vector<uint32_t> tl_grid;
    std::vector<double> tl_bytes;          // algorithmic bytes of each recorded launch
    bool prof_on = false;
    std::vector<cudaEvent_t> prof_ev;      // pool, two per recorded launch
    size_t prof_used = 0;
    std::vector<double> prof_bytes;
    // scratch of the op-level entry points (grown on demand)
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    void *scratch2 = nullptr;              // second area for entry points that call another scratch user
    size_t scratch2_bytes = 0;
};
int qb_ctx_scratch(qb_ctx *ctx, size_t bytes, void **out);
int qb_ctx_scratch2(qb_ctx *ctx, size_t bytes, void **out);
void qb_trace_mark(qb_ctx *ctx, const char *name);
// Device timeline (qb_debug_timeline_*): while enabled every tensor-core GEMM launch gets a slot of
// QB_TL_CTAS x 4 words; CTA b stores {entry, dependency wait passed, exit} in nanoseconds of the global
// timer and its SM id.  Returns null when disabled or full.
static const uint32_t QB_TL_CTAS = 320;
unsigned long long *qb_timeline_slot(qb_ctx *ctx, uint32_t grid, double bytes);
#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long qb_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#endif

// ---- Q8_0 weight in device layout ----------------------------------------------------------
// The matrix is cut into records of 128 rows x 128 columns (4 Q8_0 blocks per row), stored row-tile
// major: record (tile, chunk) at rec + (tile * (cols/128) + chunk) * QB_REC_BYTES.  A record is what
// one pipeline stage of the GEMM kernels consumes, so a stage is ONE contiguous 17 KB read:
//   bytes [0, 16384)       the int8 quants as the 128-byte-swizzled shared-memory image the tensor
//                          cores read: 16-byte piece p of row r at r*128 + ((p ^ (r & 7)) << 4)
//   bytes [16384, 17408)   fp16 scales [4 blocks][128 rows]
// Rows are padded to a multiple of 128 with zeros.  34 bytes per 32 weights, as in the GGUF file.
// A view shares storage with its parent.
static const uint32_t QB_REC_Q_BYTES = 16384, QB_REC_BYTES = 17408;
struct qb_weight {
    uint32_t rows = 0, cols = 0, rows_pad = 0;
    uint8_t *rec = nullptr;
    bool owns = false;
};
__host__ __device__ inline size_t qb_rec_offset(uint32_t cols, uint32_t row, uint32_t chunk) {
    return ((size_t)(row >> 7) * (cols >> 7) + chunk) * QB_REC_BYTES;
}
// byte offset of quant (row, col) and of the scale of (row, block kb) inside the weight
__host__ __device__ inline size_t qb_q_offset(uint32_t cols, uint32_t row, uint32_t col) {
    const uint32_t r = row & 127, within = col & 127, p = within >> 4;
    return qb_rec_offset(cols, row, col >> 7) + r * 128 + ((p ^ (r & 7)) << 4) + (within & 15);
}
__host__ __device__ inline size_t qb_d_offset(uint32_t cols, uint32_t row, uint32_t kb) {
    return qb_rec_offset(cols, row, kb >> 2) + QB_REC_Q_BYTES + ((kb & 3) * 128 + (row & 127)) * 2;
}
int qb_weight_alloc(qb_ctx *ctx, uint32_t rows, uint32_t cols, qb_weight **out);
int qb_weight_fill_synth(qb_ctx *ctx, qb_weight *w, uint32_t row_off, uint32_t rows, uint64_t seed,
                         uint32_t tensor_id, float sigma, uint32_t ileave = 0);
int qb_weight_fill_synth_window(qb_ctx *ctx, qb_weight *w, uint32_t row_off, uint32_t rows, uint64_t seed, uint32_t tensor_id, float sigma,
                                uint32_t ileave, uint32_t src_row0, uint32_t src_nb, uint32_t src_kb0);
int qb_weight_fill_upload(qb_ctx *ctx, qb_weight *w, uint32_t row_off, uint32_t rows, const void *host_blocks,
                          uint32_t ileave = 0);
// rows [row_off, row_off+rows) of w as a weight of its own (row_off multiple of 128).
int qb_weight_view(qb_ctx *ctx, const qb_weight *w, uint32_t row_off, uint32_t rows, qb_weight *out);

// ---- TMA tensor maps -----------------------------------------------------------------------
// 2-D row-major tensor map: inner extent `inner` elements, `outer` rows, row pitch `pitch_bytes`.
int qb_make_tmap_2d(CUtensorMap *map, CUtensorMapDataType dt, uint32_t elem_bytes, const void *base,
                    uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner,
                    uint32_t box_outer, CUtensorMapSwizzle swz);

// ---- quantised activations -----------------------------------------------------------------
// q: int8 [M][K] (row pitch q_pitch bytes); d: float [K/32][ld], ld = round_up(M, 4).
static inline uint32_t qb_act_ld(uint32_t M) { return (M + 3u) & ~3u; }

// x (+ optional residual / split partials) -> optional h_out -> optional RMSNorm -> int8 + scales.
#ifdef __CUDACC__
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
// silu(gate) * up (silu_mul_kernel src/kernels_cuda.cu:1894-1903)
__device__ __forceinline__ float qb_swiglu(float g, float u) { return __fdiv_rn(g, 1.0f + expf(-g)) * u; }
#endif

// Sum of the S split partials of one GEMM output element, ascending (the order of the split reduction).
__device__ __forceinline__ float qb_ldsum(const float *p, size_t idx, uint32_t S, size_t pstride) {
    const float p0 = p[idx];
    const float p1 = S > 1 ? p[idx + pstride] : 0.0f;      // both loads in flight before the add
    float v = S > 1 ? p0 + p1 : p0;
    for (uint32_t s = 2; s < S; ++s) v += p[idx + s * pstride];
    return v;
}

struct NormQuantArgs {
    const float *x = nullptr;        // [M][x_stride] or null (treated as zero)
    uint32_t x_stride = 0;
    const int32_t *row_map = nullptr;  // source row of x for output row m (null = identity)
    const float *parts = nullptr;    // [S][M][part_ld] partial sums added in ascending s, or null
    uint32_t S = 0;
    uint32_t part_ld = 0;            // = n of the GEMM that produced them
    float *h_out = nullptr;          // [M][h_stride] receives x + sum(parts), may alias x; or null
    uint32_t h_stride = 0;
    const float *w = nullptr;        // RMSNorm gain [n]; null = no normalisation
    float eps = 0.f;
    uint32_t n = 0;                  // row length, multiple of 32
    int8_t *q = nullptr;             // [M][q_pitch] written at column q_col_off
    uint32_t q_pitch = 0, q_col_off = 0;
    float *d = nullptr;              // [..][d_ld] written from block row d_kb_off
    uint32_t d_ld = 0, d_kb_off = 0;
    float *normed_out = nullptr;     // optional fp32 copy of the normalised row [M][n]
    uint32_t M = 0;
};
int qb_launch_norm_quant(qb_ctx *ctx, const NormQuantArgs &a);

// gate/up fp32 [M][2F] (gate cols [0,F), up cols [F,2F)) -> silu(gate)*up -> int8 + scales.  gu may hold S split
// partials pstride floats apart (summed ascending on read).
int qb_launch_swiglu_quant(qb_ctx *ctx, const float *gu, uint32_t gu_stride, uint32_t M, uint32_t F, int8_t *q,
                           uint32_t q_pitch, float *d, uint32_t d_ld, uint32_t S = 1, size_t pstride = 0, uint32_t ileave = 0);

// ---- GEMM ----------------------------------------------------------------------------------
// part[s][m][n] for s < S; activations q [M][K] pitch K, d [K/32][ld].
int qb_launch_gemm(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part,
                   uint32_t S, int impl);
int qb_launch_gemm_dp4a(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part,
                        uint32_t S);
// Optional fan-out of the tensor-core GEMM's epilogue for the tensor-parallel FFN: every partial sum goes to
// n destinations (this GPU's and its peers' receive areas, same [s][m][n] indexing as `part`), and once a CTA's
// stores are fenced system-wide it adds 1 to each destination's arrival counter.
struct QbGemmPush {
    float *dst[8] = {};
    unsigned int *counter[8] = {};
    uint32_t n = 0;
};
// Optional fused SwiGLU of the tensor-core GEMM (M <= 16, one K segment, weight = [gate; up] interleaved in groups
// of 64 rows): instead of the fp32 products the epilogue writes int8(silu(gate) * up) and its block scales, the
// quantised input of the down projection.
struct QbGemmSwiglu {
    int8_t *q = nullptr;             // [M][q_pitch]
    float *d = nullptr;              // [F/32][d_ld]
    uint32_t q_pitch = 0, d_ld = 0;
};
int qb_launch_gemm_tc(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part,
                      uint32_t S, const QbGemmPush *push = nullptr, uint32_t *grid_out = nullptr,
                      const QbGemmSwiglu *swiglu = nullptr);
bool qb_gemm_tc_supported(const qb_weight *w, uint32_t M);
// hq/hd = quantise(silu(gate) * up) of x W^T for a fused, 64-row-interleaved [gate; up] weight.  Few rows and one K
// segment: one launch (the GEMM epilogue does it); otherwise GEMM (into act, or split partials into parts) and the
// SwiGLU kernel.  mode: 0 = as described, 1 = always two launches, 2 = one launch or fail.
int qb_ffn_gate_up_swiglu(qb_ctx *ctx, const qb_weight *w, const int8_t *xq, const float *xd, uint32_t M, float *act, float *parts,
                          size_t parts_floats, int8_t *hq, uint32_t hq_pitch, float *hd, uint32_t hd_ld, int gemm_impl, int mode);
uint32_t qb_ksplit(uint32_t N, uint32_t K);
// Row order of a tensor-parallel group's gate/up shards: 0 = [gate; up] (the op-level entry points), 64 = the model's
// interleaved order.
void qb_tp_group_set_ileave(qb_tp_group *g, uint32_t ileave);
// y[m][n] = sum_s part[s][m][n] (ascending s).
int qb_launch_reduce_parts(qb_ctx *ctx, const float *part, uint32_t S, uint32_t M, uint32_t N, float *y,
                           uint32_t y_stride);

// ---- misc ops used by the engine -----------------------------------------------------------
int qb_launch_get_rows(qb_ctx *ctx, const qb_weight *w, const int32_t *ids_dev, uint32_t n, float *out,
                       uint32_t out_stride);
int qb_launch_argmax_partial(qb_ctx *ctx, const float *x, uint32_t M, uint32_t n, uint32_t stride, float *pval,
                             int32_t *pidx, uint32_t nblk);
static const uint32_t QB_ARGMAX_BLOCKS = 64;
int qb_launch_sample_rows(qb_ctx *ctx, const float *logits, uint32_t rows, uint32_t V, uint32_t stride, const int32_t *draft,
                          uint32_t K1, const double *u_acc, const double *u_res, float temp, float top_p, int32_t top_k,
                          float min_p, int32_t *token, int32_t *accepted, float *p_draft, float *pval, int32_t *pidx,
                          uint32_t nblk, float presence, float repetition, const uint32_t *seen, uint32_t seen_words,
                          const int32_t *chain_limit = nullptr, int32_t eos = -1);

// Attention over the paged cache.  Rows are grouped per sequence: sequence s owns rows
// [s*R, (s+1)*R), R = rows / n_seqs, at positions seq_pos[s] .. seq_pos[s]+R-1 (seq_pos on the device).
struct AttnArgs {
    float *qkv = nullptr; uint32_t rows = 0, row_stride = 0;   // rows [q(+gate) | k | v]
    uint32_t in_S = 1; size_t in_pstride = 0;                  // qkv holds in_S split partials, in_pstride floats apart
                                                               // (summed ascending on read; q is finalised in partial 0)
    uint32_t n_heads = 0, n_kv = 0, hd = 0, rope_dim = 0; float eps = 0.f;
    const float *q_norm_w = nullptr, *k_norm_w = nullptr, *inv_freq = nullptr;
    const int32_t *page_table = nullptr;
    uint32_t pt_stride = 0, page_size = 0;
    __half *k_cache = nullptr, *v_cache = nullptr;
    uint32_t max_pos = 0;            // upper bound of any row position (sizes the split grid)
    float *part_acc = nullptr, *part_ml = nullptr;   // split partials
    bool kv_only = false;            // prepare: skip the q heads
    bool no_gate = false;            // merge: leave the output ungated (attention_decode + a separate apply_attn_gate)
    uint32_t split_keys = 0;         // keys per split: 0 = the library default (256, QW3B200_ATTN_SPLIT); a batch sets its own
    int *err_flag = nullptr;         // an append to a page-table entry < 0 is skipped and recorded here (3002)
    bool ingest = false;             // rows of a prompt chunk: always the mma.sync shapes, whose rows do not depend on the chunking
    bool prefer_tc = true;           // decode / verify rows on the tensor-memory kernel where it applies (a batch decides once, by its capacity)
};
// Decode / verify rows on tcgen05 (attention_tc.cu): same partials as attn_split_kernel, merged by the same kernel.
bool qb_attn_tc_supports(const AttnArgs &a);
int qb_attn_tc_launch(qb_ctx *ctx, const AttnArgs &a, const int32_t *seq_pos, uint32_t R, uint32_t n_seqs, uint32_t max_splits);
int qb_attn_prepare(qb_ctx *ctx, const AttnArgs &a, const int32_t *seq_pos, uint32_t n_seqs);
// split partials, then merge + gate; out fp32 [rows][n_heads*hd] and/or int8 (q8 [rows][q_pitch], d [.][d_ld]).
int qb_attn_run(qb_ctx *ctx, const AttnArgs &a, const int32_t *seq_pos, uint32_t n_seqs, float *out, int8_t *q8,
                uint32_t q_pitch, float *d, uint32_t d_ld);
size_t qb_attention_scratch_floats(uint32_t rows, uint32_t n_heads, uint32_t hd, uint32_t max_pos,
                                   size_t *ml_floats, uint32_t split = 0);
static const uint32_t QB_ATTN_SPLIT = 256;   // default keys per split (four 64-key tiles), fixed absolute boundaries; a batch may name 128

struct DnArgs {
    const float *proj = nullptr; uint32_t proj_stride = 0;   // rows [qkv | z | alpha | beta]
    uint32_t proj_S = 1; size_t proj_pstride = 0;            // proj holds proj_S split partials, summed ascending on read
    uint32_t n_seqs = 0, rows_per_seq = 0;                   // rows of sequence s: [s*rows_per_seq, ...)
    const float *conv_w = nullptr, *ssm_a = nullptr, *dt_bias = nullptr, *norm_w = nullptr;
    uint32_t nk = 0, nv = 0, hd = 0; float eps = 0.f;
    float *state = nullptr, *conv = nullptr;                 // [n_seqs][n_slots][...]
    float *conv_out = nullptr;                               // new conv state (same layout), a buffer other than conv
    uint32_t n_slots = 0;
    const int32_t *slot_in = nullptr;                        // [n_seqs] device
    int write_all = 0;
    int8_t *q8 = nullptr; uint32_t q_pitch = 0; float *d = nullptr; uint32_t d_ld = 0;   // quantised gated core
    float *core_out = nullptr;                               // optional fp32 gated core
};
int qb_launch_deltanet(qb_ctx *ctx, const DnArgs &a);
