// Gated full attention over a paged fp16 KV cache for the decode / draft / (k+1)-row verify step.
//
// Replaces, for this path, rmsnorm_per_head_batch + rope_partial_batch + kv_append_batch_paged_device
// (src/kernels_cuda.cu:4622-4645, 4697-4799, 8921-8969) and the paged decode attention the
// reference reaches through attention_decode_batch_paged_gated_device (src/kernels_cuda.cu:20187-20358;
// math as in src/fattn_vec_decode.cu:118-124, 156-233; gate src/kernels_cuda.cu:9448-9465).
//
// Rows come in groups: sequence s owns rows [s*R, (s+1)*R) at positions seq_pos[s] .. seq_pos[s]+R-1.
// All query rows of a group that share a KV head are processed by one CTA in ONE pass over that
// head's keys (the reference re-reads the cache once per row).  The key range is cut at fixed
// absolute boundaries (QB_ATTN_SPLIT keys) and tiles (64 keys) and the split partials are merged in
// ascending order, so a row's result does not depend on how many other rows are in the launch.
#include "qb_internal.h"

namespace {

constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = 8;
constexpr int TK = 64;          // keys per tile
constexpr int QR = 4;           // query rows per CTA

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

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

// ---- per-head RMSNorm + partial RoPE + paged K/V append --------------------------------------
// grid (rows, units): units = q heads, then k heads, then v heads.  blockDim = head_dim.
__global__ void qk_norm_rope_append_kernel(AttnArgs a, const int32_t *__restrict__ seq_pos, uint32_t R, uint32_t unit0) {
    QB_PDL_ENTER();
    extern __shared__ float buf[];
    __shared__ float red[8];
    const uint32_t row = blockIdx.x, unit = blockIdx.y + unit0, i = threadIdx.x, hd = a.hd;
    const uint32_t seq = row / R;
    const int pos = seq_pos[seq] + (int)(row % R);
    float *rowp = a.qkv + (size_t)row * a.row_stride;
    const uint32_t kvd = a.n_kv * hd;
    float *base;
    const float *w = nullptr;
    int kind;   // 0 q, 1 k, 2 v
    if (unit < a.n_heads) { base = rowp + (size_t)unit * 2 * hd; w = a.q_norm_w; kind = 0; }
    else if (unit < a.n_heads + a.n_kv) { base = rowp + (size_t)a.n_heads * 2 * hd + (size_t)(unit - a.n_heads) * hd; w = a.k_norm_w; kind = 1; }
    else { base = rowp + (size_t)a.n_heads * 2 * hd + kvd + (size_t)(unit - a.n_heads - a.n_kv) * hd; kind = 2; }
    float v = qb_ldsum(base, i, a.in_S, a.in_pstride);
    if (kind != 2) {
        float ss = warp_sum(v * v);
        if ((i & 31) == 0) red[i >> 5] = ss;
        __syncthreads();
        float tot = 0.0f;
        for (uint32_t k = 0; k < hd / 32; ++k) tot += red[k];
        v = v * rsqrtf(tot / (float)hd + a.eps) * w[i];
        buf[i] = v;
        __syncthreads();
        const uint32_t half = a.rope_dim / 2;
        if (i < a.rope_dim) {
            const uint32_t f = i < half ? i : i - half;
            float s, c;
            sincosf((float)pos * a.inv_freq[f], &s, &c);
            const float x0 = buf[f], x1 = buf[f + half];
            v = i < half ? x0 * c - x1 * s : x0 * s + x1 * c;
        }
    }
    if (kind == 0) { base[i] = v; return; }
    const uint32_t pg = (uint32_t)pos / a.page_size;
    const size_t slot = (size_t)a.page_table[(size_t)seq * a.pt_stride + pg] * a.page_size + (uint32_t)pos % a.page_size;
    const uint32_t h = kind == 1 ? unit - a.n_heads : unit - a.n_heads - a.n_kv;
    __half *dst = (kind == 1 ? a.k_cache : a.v_cache) + (slot * a.n_kv + h) * hd;
    dst[i] = __float2half_rn(v);
}

// ---- split attention ---------------------------------------------------------------------------
template <int HD>
struct AttSmem {
    static constexpr int ROW = HD * 2 + 16;                 // bytes per key row (padded)
    static constexpr int KV_TILE = TK * ROW;
    static constexpr int STAGE = 2 * KV_TILE;               // K then V
    static constexpr int Q_BYTES = 32 * HD * 4;             // up to 32 queries
    static constexpr int P_BYTES = 32 * TK * 4;
    static constexpr int TOTAL = 2 * STAGE + Q_BYTES + P_BYTES;
};

// grid (max_splits, n_kv, n_seqs * ceil(R/QR)).  QPW = queries per warp (QR*G <= 8*QPW).
template <int HD, int QPW>
__global__ void __launch_bounds__(ATT_THREADS) attn_split_kernel(AttnArgs a, const int32_t *__restrict__ seq_pos, uint32_t R,
                                                                 uint32_t max_splits) {
    QB_PDL_ENTER();
    using L = AttSmem<HD>;
    extern __shared__ __align__(16) uint8_t smem[];
    float *Qs = reinterpret_cast<float *>(smem + 2 * L::STAGE);
    float *Ps = reinterpret_cast<float *>(smem + 2 * L::STAGE + L::Q_BYTES);
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t split = blockIdx.x, kvh = blockIdx.y;
    const uint32_t chunks = (R + QR - 1) / QR;
    const uint32_t seq = blockIdx.z / chunks, chunk = blockIdx.z % chunks;
    const uint32_t r_begin = chunk * QR, r_count = min((uint32_t)QR, R - r_begin);
    const uint32_t G = a.n_heads / a.n_kv;
    const uint32_t NQ = r_count * G;
    const int base_pos = seq_pos[seq] + (int)r_begin;            // position of the chunk's first row
    const int last_key = base_pos + (int)r_count - 1;            // highest key index any row here sees
    const int k_begin = (int)(split * QB_ATTN_SPLIT);
    if (k_begin > last_key) return;
    const int k_end = min(k_begin + (int)QB_ATTN_SPLIT, last_key + 1);
    const int n_tiles = (k_end - k_begin + TK - 1) / TK;
    const float scale = rsqrtf((float)HD);
    const int32_t *pt = a.page_table + (size_t)seq * a.pt_stride;

    // stage the queries (scaled): query index qi = r_local * G + g, head = kvh*G + g
    for (uint32_t idx = tid; idx < NQ * HD; idx += ATT_THREADS) {
        const uint32_t qi = idx / HD, dd = idx % HD;
        const uint32_t rl = qi / G, g = qi % G;
        const size_t row = (size_t)seq * R + r_begin + rl;
        Qs[qi * HD + dd] = a.qkv[row * a.row_stride + (size_t)(kvh * G + g) * 2 * HD + dd] * scale;
    }

    auto load_tile = [&](int tile, int slot) {
        uint8_t *ks = smem + slot * L::STAGE, *vs = ks + L::KV_TILE;
        constexpr int CH = HD * 2 / 16;                          // 16-byte chunks per key row
        for (int c = tid; c < TK * CH; c += ATT_THREADS) {
            const int t = c / CH, p = c % CH;
            const int key = k_begin + tile * TK + t;
            const bool valid = key < k_end;
            size_t off = 0;
            if (valid) {
                const size_t slot_i = (size_t)pt[key / (int)a.page_size] * a.page_size + key % (int)a.page_size;
                off = (slot_i * a.n_kv + kvh) * HD;
            }
            cp_async16(ks + t * L::ROW + p * 16, a.k_cache + off + p * 8, valid);
            cp_async16(vs + t * L::ROW + p * 16, a.v_cache + off + p * 8, valid);
        }
    };

    constexpr int DPL = HD / 32;                                 // output dims per lane
    float acc[QPW][DPL];
    float m_run[QPW], l_run[QPW];
#pragma unroll
    for (int j = 0; j < QPW; ++j) {
        m_run[j] = -INFINITY; l_run[j] = 0.0f;
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[j][e] = 0.0f;
    }

    load_tile(0, 0);
    cp_async_commit();
    for (int tile = 0; tile < n_tiles; ++tile) {
        if (tile + 1 < n_tiles) load_tile(tile + 1, (tile + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint8_t *ks = smem + (tile & 1) * L::STAGE, *vs = ks + L::KV_TILE;
        const int key0 = k_begin + tile * TK;

        // scores: lane handles keys lane and lane+32 of the tile
        float s0[QPW], s1[QPW];
#pragma unroll
        for (int j = 0; j < QPW; ++j) { s0[j] = 0.0f; s1[j] = 0.0f; }
        const uint8_t *k0p = ks + lane * L::ROW, *k1p = ks + (lane + 32) * L::ROW;
#pragma unroll 4
        for (int c = 0; c < HD / 8; ++c) {
            const uint4 ka = *reinterpret_cast<const uint4 *>(k0p + c * 16);
            const uint4 kb = *reinterpret_cast<const uint4 *>(k1p + c * 16);
            float fa[8], fb[8];
            {
                const __half2 *ha = reinterpret_cast<const __half2 *>(&ka), *hb = reinterpret_cast<const __half2 *>(&kb);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 x = __half22float2(ha[e]), y = __half22float2(hb[e]);
                    fa[2 * e] = x.x; fa[2 * e + 1] = x.y; fb[2 * e] = y.x; fb[2 * e + 1] = y.y;
                }
            }
#pragma unroll
            for (int j = 0; j < QPW; ++j) {
                const uint32_t qi = warp + j * ATT_WARPS;
                if (qi < NQ) {
                    const float4 qa = *reinterpret_cast<const float4 *>(Qs + qi * HD + c * 8);
                    const float4 qb = *reinterpret_cast<const float4 *>(Qs + qi * HD + c * 8 + 4);
                    s0[j] += qa.x * fa[0] + qa.y * fa[1] + qa.z * fa[2] + qa.w * fa[3] + qb.x * fa[4] + qb.y * fa[5] + qb.z * fa[6] + qb.w * fa[7];
                    s1[j] += qa.x * fb[0] + qa.y * fb[1] + qa.z * fb[2] + qa.w * fb[3] + qb.x * fb[4] + qb.y * fb[5] + qb.z * fb[6] + qb.w * fb[7];
                }
            }
        }
        // online softmax per query, probabilities to shared memory
#pragma unroll
        for (int j = 0; j < QPW; ++j) {
            const uint32_t qi = warp + j * ATT_WARPS;
            if (qi >= NQ) continue;
            const int qpos = base_pos + (int)(qi / G);
            const int ka_i = key0 + (int)lane, kb_i = ka_i + 32;
            const float a0 = (ka_i <= qpos && ka_i < k_end) ? s0[j] : -INFINITY;
            const float a1 = (kb_i <= qpos && kb_i < k_end) ? s1[j] : -INFINITY;
            const float m_new = fmaxf(m_run[j], warp_max(fmaxf(a0, a1)));
            float p0 = 0.0f, p1 = 0.0f, corr = 1.0f;
            if (m_new != -INFINITY) {
                p0 = expf(a0 - m_new);
                p1 = expf(a1 - m_new);
                corr = expf(m_run[j] - m_new);
            }
            l_run[j] = l_run[j] * corr + warp_sum(p0 + p1);
            m_run[j] = m_new;
#pragma unroll
            for (int e = 0; e < DPL; ++e) acc[j][e] *= corr;
            Ps[qi * TK + lane] = p0;
            Ps[qi * TK + lane + 32] = p1;
        }
        __syncwarp();
        // P x V: lane owns dims [lane*DPL, lane*DPL + DPL)
        for (int t = 0; t < TK; ++t) {
            float vv[DPL];
            const __half *vp = reinterpret_cast<const __half *>(vs + t * L::ROW) + lane * DPL;
            if constexpr (DPL == 8) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(vp);
                const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h2[e]); vv[2 * e] = f.x; vv[2 * e + 1] = f.y; }
            } else if constexpr (DPL == 4) {
                const uint2 raw = *reinterpret_cast<const uint2 *>(vp);
                const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
                for (int e = 0; e < 2; ++e) { const float2 f = __half22float2(h2[e]); vv[2 * e] = f.x; vv[2 * e + 1] = f.y; }
            } else {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(vp));
                vv[0] = f.x; vv[1] = f.y;
            }
#pragma unroll
            for (int j = 0; j < QPW; ++j) {
                const uint32_t qi = warp + j * ATT_WARPS;
                if (qi < NQ) {
                    const float p = Ps[qi * TK + t];
#pragma unroll
                    for (int e = 0; e < DPL; ++e) acc[j][e] = fmaf(p, vv[e], acc[j][e]);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int j = 0; j < QPW; ++j) {
        const uint32_t qi = warp + j * ATT_WARPS;
        if (qi >= NQ) continue;
        const size_t row = (size_t)seq * R + r_begin + qi / G;
        const uint32_t head = kvh * G + qi % G;
        const size_t pidx = (row * a.n_heads + head) * max_splits + split;
#pragma unroll
        for (int e = 0; e < DPL; ++e) a.part_acc[pidx * HD + lane * DPL + e] = acc[j][e];
        if (lane == 0) { a.part_ml[pidx * 2] = m_run[j]; a.part_ml[pidx * 2 + 1] = l_run[j]; }
    }
}

// Merge split partials in ascending order, apply the sigmoid gate, write fp32 and/or int8.
// grid (rows, n_heads), blockDim = HD.
__global__ void attn_merge_kernel(AttnArgs a, const int32_t *__restrict__ seq_pos, uint32_t R, uint32_t max_splits,
                                  float *out, int8_t *q8, uint32_t q_pitch, float *dsc, uint32_t d_ld) {
    QB_PDL_ENTER();
    __shared__ float wsplit[256];
    __shared__ float red_m[8];
    const uint32_t row = blockIdx.x, head = blockIdx.y, i = threadIdx.x, hd = a.hd, lane = i & 31;
    const int pos = seq_pos[row / R] + (int)(row % R);
    const uint32_t nsplit = ((uint32_t)pos + QB_ATTN_SPLIT) / QB_ATTN_SPLIT;
    const size_t p0 = ((size_t)row * a.n_heads + head) * max_splits;
    // block-wide maximum of the split maxima (all loads in flight together)
    float mx = -INFINITY;
    for (uint32_t s = i; s < nsplit; s += hd) mx = fmaxf(mx, a.part_ml[(p0 + s) * 2]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red_m[i >> 5] = mx;
    __syncthreads();
    mx = red_m[0];
    for (uint32_t k = 1; k < hd / 32; ++k) mx = fmaxf(mx, red_m[k]);
    // splits in ascending order, 256 at a time: weights computed in parallel, then every thread walks them
    float num = 0.0f, den = 0.0f;
    for (uint32_t s0 = 0; s0 < nsplit; s0 += 256) {
        const uint32_t cnt = min(256u, nsplit - s0);
        __syncthreads();
        for (uint32_t s = i; s < cnt; s += hd) wsplit[s] = expf(a.part_ml[(p0 + s0 + s) * 2] - mx);
        __syncthreads();
        const float *acc = a.part_acc + (p0 + s0) * hd + i;
        const float *ml = a.part_ml + (p0 + s0) * 2 + 1;
        uint32_t s = 0;
        for (; s + 8 <= cnt; s += 8) {
            float va[8], vl[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) { va[u] = acc[(size_t)(s + u) * hd]; vl[u] = ml[(s + u) * 2]; }
#pragma unroll
            for (int u = 0; u < 8; ++u) { num = fmaf(va[u], wsplit[s + u], num); den = fmaf(vl[u], wsplit[s + u], den); }
        }
        for (; s < cnt; ++s) { num = fmaf(acc[(size_t)s * hd], wsplit[s], num); den = fmaf(ml[s * 2], wsplit[s], den); }
    }
    const float gate = qb_ldsum(a.qkv, (size_t)row * a.row_stride + (size_t)head * 2 * hd + hd + i, a.in_S, a.in_pstride);
    const float o = __fdiv_rn(num, den) * __fdiv_rn(1.0f, 1.0f + expf(-gate));
    const uint32_t col = head * hd + i;
    if (out) out[(size_t)row * a.n_heads * hd + col] = o;
    if (q8) {
        float amax = fabsf(o);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const float d_inv = (amax == 0.0f) ? 0.0f : __fdiv_rn(127.0f, amax);
        q8[(size_t)row * q_pitch + col] = (int8_t)((amax == 0.0f) ? 0 : __float2int_rn(__fmul_rn(o, d_inv)));
        if (lane == 0) dsc[(size_t)(col / 32) * d_ld + row] = (amax == 0.0f) ? 0.0f : __fdiv_rn(1.0f, d_inv);
    }
}

template <int HD, int QPW>
int launch_split(qb_ctx *ctx, const AttnArgs &a, const int32_t *seq_pos, uint32_t R, uint32_t n_seqs, uint32_t max_splits) {
    using L = AttSmem<HD>;
    static bool attr = false;
    if (!attr) {
        QB_CUDA(cudaFuncSetAttribute(attn_split_kernel<HD, QPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        attr = true;
    }
    dim3 grid(max_splits, a.n_kv, n_seqs * ((R + QR - 1) / QR));
    QB_CUDA(qb_launch_pdl(ctx->stream, attn_split_kernel<HD, QPW>, dim3(grid), dim3(ATT_THREADS), (size_t)(L::TOTAL), a, seq_pos, R, max_splits));
    QB_LAUNCHED(ctx, "attn_split_kernel");
    return QB_OK;
}

}  // namespace

static uint32_t max_splits_for(uint32_t max_pos) { return max_pos / QB_ATTN_SPLIT + 1; }

size_t qb_attention_scratch_floats(uint32_t rows, uint32_t n_heads, uint32_t hd, uint32_t max_pos, size_t *ml_floats) {
    const size_t ms = max_splits_for(max_pos);
    if (ml_floats) *ml_floats = (size_t)rows * n_heads * ms * 2;
    return (size_t)rows * n_heads * ms * hd;
}

int qb_attn_prepare(qb_ctx *ctx, const AttnArgs &a, const int32_t *seq_pos, uint32_t n_seqs) {
    QB_REQUIRE(a.rows % n_seqs == 0, "attention: rows %u not a multiple of sequences %u", a.rows, n_seqs);
    QB_REQUIRE(a.hd == 64 || a.hd == 128 || a.hd == 256, "attention: head_dim %u unsupported (64/128/256)", a.hd);
    QB_REQUIRE(a.rope_dim <= a.hd && a.rope_dim % 2 == 0, "attention: bad rope_dim %u", a.rope_dim);
    const uint32_t R = a.rows / n_seqs;
    const uint32_t unit0 = a.kv_only ? a.n_heads : 0;
    dim3 grid(a.rows, a.n_heads + 2 * a.n_kv - unit0);
    QB_CUDA(qb_launch_pdl(ctx->stream, qk_norm_rope_append_kernel, dim3(grid), dim3(a.hd), (size_t)(a.hd * sizeof(float)), a, seq_pos, R, unit0));
    QB_LAUNCHED(ctx, "qk_norm_rope_append_kernel");
    return QB_OK;
}

int qb_attn_run(qb_ctx *ctx, const AttnArgs &a, const int32_t *seq_pos, uint32_t n_seqs, float *out, int8_t *q8,
                uint32_t q_pitch, float *d, uint32_t d_ld) {
    QB_REQUIRE(a.rows % n_seqs == 0, "attention: rows %u not a multiple of sequences %u", a.rows, n_seqs);
    const uint32_t R = a.rows / n_seqs;
    const uint32_t G = a.n_heads / a.n_kv;
    QB_REQUIRE(G * a.n_kv == a.n_heads && G <= 8, "attention: GQA group %u unsupported (<= 8)", G);
    const uint32_t ms = max_splits_for(a.max_pos);
    const uint32_t nq = std::min<uint32_t>(R, QR) * G;
    const uint32_t qpw = (nq + ATT_WARPS - 1) / ATT_WARPS;
    int st = QB_OK;
#define QB_ATT_CASE(HD_, QPW_) st = launch_split<HD_, QPW_>(ctx, a, seq_pos, R, n_seqs, ms)
    if (a.hd == 256) { if (qpw <= 1) QB_ATT_CASE(256, 1); else if (qpw <= 2) QB_ATT_CASE(256, 2); else if (qpw == 3) QB_ATT_CASE(256, 3); else QB_ATT_CASE(256, 4); }
    else if (a.hd == 128) { if (qpw <= 1) QB_ATT_CASE(128, 1); else if (qpw <= 2) QB_ATT_CASE(128, 2); else if (qpw == 3) QB_ATT_CASE(128, 3); else QB_ATT_CASE(128, 4); }
    else if (a.hd == 64) { if (qpw <= 1) QB_ATT_CASE(64, 1); else if (qpw <= 2) QB_ATT_CASE(64, 2); else if (qpw == 3) QB_ATT_CASE(64, 3); else QB_ATT_CASE(64, 4); }
    else return qb_fail(QB_ERR_UNSUPPORTED, "attention: head_dim %u unsupported", a.hd);
#undef QB_ATT_CASE
    QB_TRY(st);
    dim3 grid(a.rows, a.n_heads);
    QB_CUDA(qb_launch_pdl(ctx->stream, attn_merge_kernel, dim3(grid), dim3(a.hd), (size_t)(0), a, seq_pos, R, ms, out, q8, q_pitch, d, d_ld));
    QB_LAUNCHED(ctx, "attn_merge_kernel");
    return QB_OK;
}
