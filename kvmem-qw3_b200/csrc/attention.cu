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
// absolute boundaries (QB_ATTN_SPLIT keys) and tiles (64 keys), the tiles of a split are folded in ascending
// order and the split partials merged in ascending order, so a row's result does not depend on how many other
// rows are in the launch.
#include "qb_internal.h"

#include <cstdlib>

namespace {

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
    const int32_t page = a.page_table[(size_t)seq * a.pt_stride + pg];
    if (page < 0) {                                     // no page assigned (pooled page tables): recorded, not dereferenced
        if (i == 0 && a.err_flag) atomicExch(a.err_flag, 3002);
        return;
    }
    const size_t slot = (size_t)page * a.page_size + (uint32_t)pos % a.page_size;
    const uint32_t h = kind == 1 ? unit - a.n_heads : unit - a.n_heads - a.n_kv;
    __half *dst = (kind == 1 ? a.k_cache : a.v_cache) + (slot * a.n_kv + h) * hd;
    dst[i] = __float2half_rn(v);
}

// ---- split attention ---------------------------------------------------------------------------
// One CTA = a run of splits (a.split_keys keys each: 256 = 4 tiles of 64 by default, 128 in batches that name it) of one KV
// head for up to 16 * MT queries (query rows
// x GQA group).  Tensor-core math on fp16 operands with fp32 accumulation (mma.sync m16n8k16; the kernel streams
// the cache once and is bound by HBM, not by the tensor pipe): S = Q K^T with Q (scaled, fp16) as A fragments,
// P = exp(S - m) written to shared memory as fp16, O += P V with V read through ldmatrix.trans.  Warp w = (h, j),
// h < MT, j < JW: query rows [16h, 16h+16), keys [j*64/JW, (j+1)*64/JW) of the tile for S and output dims
// [j*HD/JW, (j+1)*HD/JW) for O.  The running maximum of a row is shared by the JW warps that hold it (one exchange
// per tile through shared memory); row sums are kept per group of 8 keys and added in key order at the end.
// Two shapes of the same arithmetic: MT = 2 for decode and verify rows (<= 4 rows x GQA group: 8 key slices per
// tile, Q fragments in registers, 3 K/V stages) and MT = 4 for prompt chunks (64 queries per CTA, so a chunk reads
// its K/V a quarter as often; 2 stages).  A query row gets the same bits from either: the same MMA chains per
// output element (even and odd 16-deep steps of Q K^T in two accumulators, then added), the same 8-key groups of
// row sums in the same order, the same tile and split order.
constexpr uint32_t QB_ATTN_RUN_PAGES = 128;                  // pages a CTA's run of splits may touch (first slot of each kept in shared memory)
template <int HD, int MT>
struct AttSmem {
    static constexpr int NQ = 16 * MT;                      // queries per CTA
    static constexpr int ROWB = HD * 2 + 16;                // bytes per key / query row (padded: conflict-free ldmatrix)
    static constexpr int KV_TILE = TK * ROWB;
    static constexpr int STAGE = 2 * KV_TILE;               // K then V
    static constexpr int NSTAGE = MT > 2 ? 2 : 3;
    static constexpr int Q_OFF = NSTAGE * STAGE;
    static constexpr int Q_BYTES = NQ * ROWB;
    static constexpr int P_ROWB = TK * 2 + 16;
    static constexpr int P_OFF = Q_OFF + Q_BYTES;
    static constexpr int P_BYTES = NQ * P_ROWB;
    static constexpr int RED_OFF = P_OFF + P_BYTES;         // float [8 key groups][NQ rows]
    static constexpr int TOTAL = RED_OFF + 8 * NQ * 4;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (ceil(max_splits / spc), n_kv, n_seqs * ceil(R / qr)), qr = query rows per CTA.  A CTA walks a run of `spc`
// consecutive splits of its KV head: the K/V tiles of the whole run go through one continuous load pipeline and the
// queries are staged once, but every split still gets its own (max, sum, accumulator) triple written to its own partial
// slot, so the result does not depend on spc (the launcher picks it from the grid size alone: about one wave of CTAs at
// long contexts).
template <int HD, int JW, int MT>
__global__ void __launch_bounds__(32 * JW * MT) attn_split_kernel(AttnArgs a, const int32_t *__restrict__ seq_pos, uint32_t R,
                                                                      uint32_t max_splits, uint32_t spc, uint32_t qr) {
    QB_PDL_ENTER();
    using L = AttSmem<HD, MT>;
    constexpr int THREADS = 32 * JW * MT, WARPS = JW * MT;       // JW warps share a 16-query m-tile
    constexpr int NQM = L::NQ;
    constexpr int KW = TK / JW, NTS = KW / 8;                    // keys (8-key n-tiles) of a tile per warp
    constexpr int DW = HD / JW;                                  // output dims per warp
    constexpr bool QREG = MT <= 2;                               // Q fragments live in registers (else re-read per step)
    constexpr int D = L::NSTAGE - 1;                             // tiles in flight ahead of the one being used
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    float *red = reinterpret_cast<float *>(smem + L::RED_OFF);
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t h = warp % MT, j = warp / MT;                 // query m-tile, key / output-dim slice
    const uint32_t g4 = lane >> 2, t4 = lane & 3;                // accumulator row / column pair of this lane
    const uint32_t split0 = blockIdx.x * spc, kvh = blockIdx.y;  // first split of this CTA's run
    const uint32_t chunks = (R + qr - 1) / qr;
    const uint32_t seq = blockIdx.z / chunks, chunk = blockIdx.z % chunks;
    const uint32_t r_begin = chunk * qr, r_count = min(qr, R - r_begin);
    const uint32_t G = a.n_heads / a.n_kv;
    const uint32_t NQ = r_count * G;
    const int base_pos = seq_pos[seq] + (int)r_begin;            // position of the chunk's first row
    const int last_key = base_pos + (int)r_count - 1;            // highest key index any row here sees
    const int k_begin = (int)(split0 * a.split_keys);
    if (k_begin > last_key) return;
    const int k_end = min(k_begin + (int)(spc * a.split_keys), last_key + 1);
    const int n_tiles = (k_end - k_begin + TK - 1) / TK;
    const int tps = (int)a.split_keys / TK;                      // tiles per split
    const float scale = rsqrtf((float)HD);
    const int32_t *pt = a.page_table + (size_t)seq * a.pt_stride;
    const bool active = h * 16 < NQ;                             // this warp's query rows exist

    // a thread copies one 16-byte column of every (THREADS / CH)-th key row: one page-table lookup per row, no
    // division when the page size is a power of two
    const uint32_t psz = a.page_size;
    const bool pow2 = (psz & (psz - 1)) == 0;
    const int psh = __ffs((int)psz) - 1;
    // first slot of every page the run touches, looked up once (the tile loop then reads shared memory only)
    __shared__ int page_slot[QB_ATTN_RUN_PAGES];
    {
        const uint32_t pg0 = pow2 ? (uint32_t)k_begin >> psh : (uint32_t)k_begin / psz;
        const uint32_t pg1 = pow2 ? (uint32_t)(k_end - 1) >> psh : (uint32_t)(k_end - 1) / psz;
        for (uint32_t i = tid; i <= pg1 - pg0 && i < QB_ATTN_RUN_PAGES; i += THREADS) page_slot[i] = pt[pg0 + i] * (int)psz;
        __syncthreads();
    }
    const uint32_t pg_first = pow2 ? (uint32_t)k_begin >> psh : (uint32_t)k_begin / psz;
    auto load_tile = [&](int tile, int slot) {
        uint8_t *ks = smem + slot * L::STAGE, *vs = ks + L::KV_TILE;
        constexpr int CH = HD * 2 / 16;                          // 16-byte chunks per key row
        constexpr int RPP = THREADS / CH;                        // rows per pass
        const int p = tid % CH;
#pragma unroll
        for (int t = tid / CH; t < TK; t += RPP) {
            const int key = k_begin + tile * TK + t;
            const bool valid = key < k_end;
            size_t off = 0;
            if (valid) {
                const uint32_t pg = pow2 ? (uint32_t)key >> psh : (uint32_t)key / psz;
                const uint32_t in_pg = (uint32_t)key - pg * psz;
                off = ((size_t)(page_slot[pg - pg_first] + (int)in_pg) * a.n_kv + kvh) * HD;
            }
            cp_async16(ks + t * L::ROWB + p * 16, a.k_cache + off + p * 8, valid);
            cp_async16(vs + t * L::ROWB + p * 16, a.v_cache + off + p * 8, valid);
        }
    };
#pragma unroll
    for (int d = 0; d < D; ++d) {
        if (d < n_tiles) load_tile(d, d);
        cp_async_commit();
    }

    // stage the queries (scaled, fp16): query index qi = r_local * G + g, head = kvh*G + g; missing rows are zero
    for (uint32_t qi = warp; qi < (uint32_t)NQM; qi += WARPS) {
        const uint32_t rl = qi / G, gq = qi - rl * G;
        const float *src = a.qkv + ((size_t)seq * R + r_begin + rl) * a.row_stride + (size_t)(kvh * G + gq) * 2 * HD;
#pragma unroll
        for (uint32_t dd = lane * 2; dd < HD; dd += 64) {
            __half2 v = __floats2half2_rn(0.0f, 0.0f);
            if (qi < NQ) {
                const float2 f = *reinterpret_cast<const float2 *>(src + dd);
                v = __floats2half2_rn(f.x * scale, f.y * scale);
            }
            *reinterpret_cast<__half2 *>(smem + L::Q_OFF + qi * L::ROWB + dd * 2) = v;
        }
    }
    __syncthreads();
    const uint32_t qaddr = smem_base + L::Q_OFF + (h * 16 + (lane & 15)) * L::ROWB + ((lane >> 4) * 8) * 2;
    uint32_t qf[QREG ? HD / 16 : 1][4];
    if constexpr (QREG) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) ldsm_x4(qf[ks], qaddr + ks * 32);
    }
    auto q_frag = [&](int ks, uint32_t (&q)[4]) {
        if constexpr (QREG) { q[0] = qf[ks][0]; q[1] = qf[ks][1]; q[2] = qf[ks][2]; q[3] = qf[ks][3]; }
        else ldsm_x4(q, qaddr + ks * 32);
    };

    constexpr int NT_O = DW / 8;                                 // 8-wide output tiles per warp
    float o[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY};                     // rows g4 and g4 + 8 of the m-tile
    float l_run[2][NTS];                                         // row sums per 8-key group of this warp
#pragma unroll
    for (int nt = 0; nt < NTS; ++nt) l_run[0][nt] = l_run[1][nt] = 0.0f;
    // positions of this lane's two query rows (rows past NQ get -1: everything masked)
    int qpos[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const uint32_t qi = h * 16 + g4 + 8 * e;
        qpos[e] = qi < NQ ? base_pos + (int)(qi / G) : -1;
    }

    for (int tile = 0; tile < n_tiles; ++tile) {
        cp_async_wait<D - 1>();
        __syncthreads();                                         // tile landed; everyone is done with tile - 1
        if (tile + D < n_tiles) load_tile(tile + D, (tile + D) % L::NSTAGE);
        cp_async_commit();
        if (tile % tps == 0 && tile > 0) {                       // a new split of the run: fresh running state
#pragma unroll
            for (int n = 0; n < NT_O; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
            m_run[0] = m_run[1] = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < NTS; ++nt) l_run[0][nt] = l_run[1][nt] = 0.0f;
        }
        const uint32_t ks_base = smem_base + (tile % L::NSTAGE) * L::STAGE, vs_base = ks_base + L::KV_TILE;
        const int key0 = k_begin + tile * TK + (int)j * KW;     // first key of this warp's KW

        // S = Q K^T for 16 queries x KW keys: even and odd 16-deep steps in two accumulators (half the dependent
        // chain), added at the end -- the same two chains in every shape of the kernel
        float sc[NTS][4];
#pragma unroll
        for (int nt = 0; nt < NTS; ++nt) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.0f; }
        if (active) {
            if constexpr (NTS >= 2) {
#pragma unroll
                for (int np = 0; np < NTS / 2; ++np) {
                    float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                    const uint32_t kaddr = ks_base + (j * KW + np * 16 + (lane & 7) + ((lane >> 4) << 3)) * L::ROWB + (((lane >> 3) & 1) * 8) * 2;
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ks += 2) {
                        uint32_t b[4], q[4];
                        q_frag(ks, q);
                        ldsm_x4(b, kaddr + ks * 32);
                        mma_f16(sc[2 * np], q, b[0], b[1]);
                        mma_f16(sc[2 * np + 1], q, b[2], b[3]);
                        q_frag(ks + 1, q);
                        ldsm_x4(b, kaddr + (ks + 1) * 32);
                        mma_f16(s2[0], q, b[0], b[1]);
                        mma_f16(s2[1], q, b[2], b[3]);
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) { sc[2 * np][c] += s2[0][c]; sc[2 * np + 1][c] += s2[1][c]; }
                }
            } else {
                // one 8-key n-tile: an x4 load covers two k-steps (d 0-7, 8-15, 16-23, 24-31)
                const uint32_t kaddr = ks_base + (j * KW + (lane & 7)) * L::ROWB + ((lane >> 3) * 8) * 2;
                float s2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks += 2) {
                    uint32_t b[4], q[4];
                    ldsm_x4(b, kaddr + ks * 32);
                    q_frag(ks, q);
                    mma_f16(sc[0], q, b[0], b[1]);
                    q_frag(ks + 1, q);
                    mma_f16(s2, q, b[2], b[3]);
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) sc[0][c] += s2[c];
            }
        }
        // causal mask + this warp's row maxima
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < NTS; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = key0 + nt * 8 + (int)t4 * 2 + (c & 1), e = c >> 1;
                if (!(key <= qpos[e] && key < k_end)) sc[nt][c] = -INFINITY;
                mx[e] = fmaxf(mx[e], sc[nt][c]);
            }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
            if (t4 == 0) red[j * NQM + h * 16 + g4 + 8 * e] = mx[e];
        }
        __syncthreads();
        float corr[2];
        uint32_t pk[NTS][2];                                     // P as fp16 pairs: [nt][row e]
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint32_t r = h * 16 + g4 + 8 * e;
            float m_tile = red[r];
#pragma unroll
            for (int w = 1; w < JW; ++w) m_tile = fmaxf(m_tile, red[w * NQM + r]);
            const float m_new = fmaxf(m_run[e], m_tile);
            corr[e] = 1.0f;
            if (m_new != -INFINITY) corr[e] = __expf(m_run[e] - m_new);
#pragma unroll
            for (int nt = 0; nt < NTS; ++nt) {
                float p0 = 0.0f, p1 = 0.0f;
                if (m_new != -INFINITY) { p0 = __expf(sc[nt][2 * e] - m_new); p1 = __expf(sc[nt][2 * e + 1] - m_new); }
                const __half2 hp = __floats2half2_rn(p0, p1);
                // the row sum uses the rounded probabilities, the values the tensor cores multiply with V
                const float2 fp = __half22float2(hp);
                l_run[e][nt] = l_run[e][nt] * corr[e] + (0.0f + (fp.x + fp.y));
                pk[nt][e] = *reinterpret_cast<const uint32_t *>(&hp);
            }
            m_run[e] = m_new;
        }
#pragma unroll
        for (int nt = 0; nt < NTS; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e)
                *reinterpret_cast<uint32_t *>(smem + L::P_OFF + (h * 16 + g4 + 8 * e) * L::P_ROWB + (j * KW + nt * 8 + t4 * 2) * 2) = pk[nt][e];
#pragma unroll
        for (int n = 0; n < NT_O; ++n) { o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1]; }
        __syncthreads();
        // O += P V for 16 queries x DW dims over the tile's 64 keys
        if (active) {
#pragma unroll
            for (int kk = 0; kk < TK / 16; ++kk) {
                uint32_t pa[4];
                ldsm_x4(pa, smem_base + L::P_OFF + (h * 16 + (lane & 15)) * L::P_ROWB + (kk * 16 + (lane >> 4) * 8) * 2);
                const uint32_t vaddr = vs_base + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * L::ROWB + (j * DW + (lane >> 4) * 8) * 2;
#pragma unroll
                for (int n2 = 0; n2 < NT_O / 2; ++n2) {
                    uint32_t b[4];
                    ldsm_x4_trans(b, vaddr + n2 * 32);
                    mma_f16(o[2 * n2], pa, b[0], b[1]);
                    mma_f16(o[2 * n2 + 1], pa, b[2], b[3]);
                }
            }
        }
        if (tile % tps != tps - 1 && tile != n_tiles - 1) continue;
        // the split is complete: row sums (quad first, then the 8-key groups of a row in key order) and its partial
        const uint32_t split = split0 + (uint32_t)(tile / tps);
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
            for (int nt = 0; nt < NTS; ++nt) {
                float l = l_run[e][nt];
                l += __shfl_xor_sync(0xffffffffu, l, 1);
                l += __shfl_xor_sync(0xffffffffu, l, 2);
                if (t4 == 0) red[(j * NTS + nt) * NQM + h * 16 + g4 + 8 * e] = l;
            }
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint32_t qi = h * 16 + g4 + 8 * e;
            if (qi >= NQ) continue;
            const size_t row = (size_t)seq * R + r_begin + qi / G;
            const uint32_t head = kvh * G + qi % G;
            const size_t pidx = (row * a.n_heads + head) * max_splits + split;
            float *dst = a.part_acc + pidx * HD + j * DW + t4 * 2;
#pragma unroll
            for (int n = 0; n < NT_O; ++n) *reinterpret_cast<float2 *>(dst + n * 8) = make_float2(o[n][2 * e], o[n][2 * e + 1]);
            if (j == 0 && t4 == 0) {
                a.part_ml[pidx * 2] = m_run[e];
                float l = red[qi];
#pragma unroll
                for (int w = 1; w < TK / 8; ++w) l += red[w * NQM + qi];
                a.part_ml[pidx * 2 + 1] = l;
            }
        }
    }
    cp_async_wait<0>();
}

// Merge split partials, apply the sigmoid gate, write fp32 and/or int8.  The splits are folded in blocks of 16 (absolute
// indices): within a block in ascending order, then the block sums in ascending order -- an order that depends on the
// row's own split count only, so a row's bits do not depend on the launch it is in, and that lets the NG thread groups
// of a CTA fold different blocks at the same time (at 32 K context a row has 129 splits; one group walking them all
// was a 36 us chain of dependent loads).  Up to 16 splits (contexts below 4096) it is the plain ascending sum.
// grid (rows, n_heads), block (hd, NG); dynamic shared memory: [nb_max][hd + 1] floats.
constexpr uint32_t MERGE_BLOCK = 16;
__global__ void __launch_bounds__(1024) attn_merge_kernel(AttnArgs a, const int32_t *__restrict__ seq_pos, uint32_t R, uint32_t max_splits,
                                                          float *out, int8_t *q8, uint32_t q_pitch, float *dsc, uint32_t d_ld) {
    QB_PDL_ENTER();
    extern __shared__ float blk[];                                       // [block][hd] numerators, then [block] denominators
    __shared__ float wsplit[1024], lsplit[1024];                         // weight and row sum of every split of a pass
    __shared__ float red_m[32];
    const uint32_t row = blockIdx.x, head = blockIdx.y, i = threadIdx.x, g = threadIdx.y, NG = blockDim.y, hd = a.hd, lane = i & 31;
    const uint32_t tid = g * hd + i, nthreads = hd * NG;
    const int pos = seq_pos[row / R] + (int)(row % R);
    const uint32_t nsplit = ((uint32_t)pos + a.split_keys) / a.split_keys;
    const uint32_t nb = (nsplit + MERGE_BLOCK - 1) / MERGE_BLOCK;
    const size_t p0 = ((size_t)row * a.n_heads + head) * max_splits;
    float *blk_den = blk + (size_t)nb * hd;
    // block-wide maximum of the split maxima (all loads in flight together)
    float mx = -INFINITY;
    for (uint32_t s = tid; s < nsplit; s += nthreads) mx = fmaxf(mx, a.part_ml[(p0 + s) * 2]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((tid & 31) == 0) red_m[tid >> 5] = mx;
    __syncthreads();
    mx = red_m[0];
    for (uint32_t k = 1; k < nthreads / 32; ++k) mx = fmaxf(mx, red_m[k]);
    // 1024 splits at a time: weights computed by everybody, then group g folds the blocks b = g, g + NG, ...
    for (uint32_t s0 = 0; s0 < nsplit; s0 += 1024) {
        const uint32_t cnt = min(1024u, nsplit - s0);
        __syncthreads();
        for (uint32_t s = tid; s < cnt; s += nthreads) {
            const float2 ml = *reinterpret_cast<const float2 *>(a.part_ml + (p0 + s0 + s) * 2);
            wsplit[s] = expf(ml.x - mx);
            lsplit[s] = ml.y;
        }
        __syncthreads();
        for (uint32_t bl = g; bl * MERGE_BLOCK < cnt; bl += NG) {
            const uint32_t sb = bl * MERGE_BLOCK, n = min(MERGE_BLOCK, cnt - sb);
            const float *acc = a.part_acc + (p0 + s0 + sb) * hd + i;
            float va[MERGE_BLOCK];
#pragma unroll
            for (uint32_t u = 0; u < MERGE_BLOCK; ++u) va[u] = u < n ? acc[(size_t)u * hd] : 0.0f;       // all in flight together
            float num = 0.0f, den = 0.0f;
#pragma unroll
            for (uint32_t u = 0; u < MERGE_BLOCK; ++u)
                if (u < n) { num = fmaf(va[u], wsplit[sb + u], num); den = fmaf(lsplit[sb + u], wsplit[sb + u], den); }
            const uint32_t b_abs = s0 / MERGE_BLOCK + bl;
            blk[(size_t)b_abs * hd + i] = num;
            if (i == 0) blk_den[b_abs] = den;
        }
    }
    __syncthreads();
    if (g != 0) return;
    float num = 0.0f, den = 0.0f;
    for (uint32_t bq = 0; bq < nb; ++bq) { num += blk[(size_t)bq * hd + i]; den += blk_den[bq]; }
    float o = __fdiv_rn(num, den);
    if (!a.no_gate) {
        const float gate = qb_ldsum(a.qkv, (size_t)row * a.row_stride + (size_t)head * 2 * hd + hd + i, a.in_S, a.in_pstride);
        o *= __fdiv_rn(1.0f, 1.0f + expf(-gate));
    }
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

// One place for the merge launch: NG thread groups by the host's bound of the split count (the result does not depend on NG).
static int launch_merge(qb_ctx *ctx, const AttnArgs &aa, const int32_t *seq_pos, uint32_t R, uint32_t ms, float *out, int8_t *q8,
                        uint32_t q_pitch, float *d, uint32_t d_ld) {
    const uint32_t nb_max = (ms + MERGE_BLOCK - 1) / MERGE_BLOCK;
    const uint32_t ng = std::max(1u, std::min(std::min(nb_max, 1024u / aa.hd), 8u));
    const size_t smem = (size_t)nb_max * (aa.hd + 1) * sizeof(float);
    QB_REQUIRE(smem <= 200 * 1024, "attention: %u splits exceed the merge kernel's shared memory", ms);
    if (smem > 48 * 1024) QB_CUDA(cudaFuncSetAttribute(attn_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(aa.rows, aa.n_heads), block(aa.hd, ng);
    QB_CUDA(qb_launch_pdl(ctx->stream, attn_merge_kernel, dim3(grid), dim3(block), smem, aa, seq_pos, R, ms, out, q8, q_pitch, d, d_ld));
    QB_LAUNCHED(ctx, "attn_merge_kernel");
    return QB_OK;
}

template <int HD, int JW, int MT>
int launch_split(qb_ctx *ctx, const AttnArgs &a, const int32_t *seq_pos, uint32_t R, uint32_t n_seqs, uint32_t max_splits) {
    using L = AttSmem<HD, MT>;
    // the attribute belongs to the current device: set on every launch (a process may drive several GPUs)
    QB_CUDA(cudaFuncSetAttribute((attn_split_kernel<HD, JW, MT>), cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    const uint32_t G = a.n_heads / a.n_kv;
    const uint32_t qr = std::max(1u, (uint32_t)L::NQ / G);          // query rows per CTA
    // splits per CTA: 1 while the grid fits one wave of CTAs (one per SM), else as many as bring it back to about one
    // wave, at most what the per-CTA page list holds
    const uint32_t zdim = n_seqs * ((R + qr - 1) / qr);
    const uint32_t cap = std::max(1u, std::min(8u, QB_ATTN_RUN_PAGES / std::max(1u, a.split_keys / a.page_size)));
    const uint32_t ctas = max_splits * a.n_kv * zdim;
    const uint32_t spc = std::min(cap, std::max(1u, (ctas + (uint32_t)ctx->sm_count - 1) / (uint32_t)ctx->sm_count));
    dim3 grid((max_splits + spc - 1) / spc, a.n_kv, zdim);
    QB_CUDA(qb_launch_pdl(ctx->stream, (attn_split_kernel<HD, JW, MT>), dim3(grid), dim3(32 * JW * MT), (size_t)(L::TOTAL), a, seq_pos, R, max_splits, spc, qr));
    QB_LAUNCHED(ctx, "attn_split_kernel");
    return QB_OK;
}

}  // namespace

// Keys per split: a fixed number (absolute boundaries), so a row's result never depends on the launch it is in.
static uint32_t split_keys() {
    static const uint32_t v = [] {
        const char *e = getenv("QW3B200_ATTN_SPLIT");
        const uint32_t n = e ? (uint32_t)atoi(e) : QB_ATTN_SPLIT;
        return (n >= 64 && n % 64 == 0) ? n : QB_ATTN_SPLIT;
    }();
    return v;
}
static uint32_t max_splits_for(uint32_t max_pos, uint32_t split) { return max_pos / split + 1; }

size_t qb_attention_scratch_floats(uint32_t rows, uint32_t n_heads, uint32_t hd, uint32_t max_pos, size_t *ml_floats, uint32_t split) {
    const size_t ms = max_splits_for(max_pos, split ? split : split_keys());
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
    AttnArgs aa = a;
    if (aa.split_keys == 0) aa.split_keys = split_keys();       // a batch names its own (a multiple of 64); the op-level calls take the default
    const uint32_t ms = max_splits_for(a.max_pos, aa.split_keys);
    QB_REQUIRE(aa.split_keys / a.page_size <= QB_ATTN_RUN_PAGES, "attention: a split of %u keys spans more than %u pages of %u", aa.split_keys, QB_ATTN_RUN_PAGES, a.page_size);
    QB_REQUIRE(((uintptr_t)a.qkv & 7) == 0 && a.row_stride % 2 == 0, "attention: q rows must be 8-byte aligned");
    int st = QB_OK;
    // decode and verify rows (a handful per sequence) run on the tensor-memory kernel; QW3B200_ATTN_TC=0 keeps them on
    // the mma.sync shapes (the two differ in the last bits, so rows of prompt chunks never take it: a request's bits
    // must not depend on how its prompt was cut; for the same reason a batch fixes a.prefer_tc once, from its capacity,
    // never from the positions of a call)
    const char *tc_env = getenv("QW3B200_ATTN_TC");                  // read per call: tests switch it
    const bool tc_on = !(tc_env && tc_env[0] == '0');
    if (tc_on && a.prefer_tc && !a.ingest && R <= 8 && qb_attn_tc_supports(aa)) {
        QB_TRY(qb_attn_tc_launch(ctx, aa, seq_pos, R, n_seqs, ms));
        return launch_merge(ctx, aa, seq_pos, R, ms, out, q8, q_pitch, d, d_ld);
    }
    // prompt chunks (many rows per sequence) take the 64-query shape: a quarter of the passes over the cache
    const bool wide = R * G > 64;
    if (a.hd == 256) st = wide ? launch_split<256, 4, 4>(ctx, aa, seq_pos, R, n_seqs, ms) : launch_split<256, 8, 2>(ctx, aa, seq_pos, R, n_seqs, ms);
    else if (a.hd == 128) st = wide ? launch_split<128, 4, 4>(ctx, aa, seq_pos, R, n_seqs, ms) : launch_split<128, 8, 2>(ctx, aa, seq_pos, R, n_seqs, ms);
    else if (a.hd == 64) st = wide ? launch_split<64, 4, 4>(ctx, aa, seq_pos, R, n_seqs, ms) : launch_split<64, 4, 2>(ctx, aa, seq_pos, R, n_seqs, ms);
    else return qb_fail(QB_ERR_UNSUPPORTED, "attention: head_dim %u unsupported", a.hd);
    QB_TRY(st);
    return launch_merge(ctx, aa, seq_pos, R, ms, out, q8, q_pitch, d, d_ld);
}
