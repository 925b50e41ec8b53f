// Split attention for decode and verify rows on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor
// memory, K/V tiles by TMA): the same split partials as attn_split_kernel (attention.cu) -- per (row, head, split) the
// maximum, the sum of the fp16-rounded probabilities and the unnormalised fp32 accumulator -- merged by the same
// attn_merge_kernel.  Replaces FlashInfer's batch decode on the reference's paged path (src/kernels_cuda.cu:20187-20358;
// math of src/fattn_vec_decode.cu:118-124, 156-233).
//
// Why the shape is transposed.  A KV head serves at most 32 queries here (<= 4 verify rows x GQA group <= 8), far fewer
// than the 128 rows an MMA wants, while the keys are plenty.  So the KEYS are the M dimension:
//     S^T [128 keys x 32 queries]  = K_tile [128 x HD]      . Q^T       (A = K, K-major as it lies in the cache; B = Q)
//     O^T [HD dims  x 32 queries] += V_tile^T [HD x 128 keys] . P^T     (A = V, "MN-major": the cache rows as they lie)
// Nothing is padded but the query count, and the softmax needs no rescaling of O: a split (256 keys = two tiles) has
// both of its score tiles in tensor memory before the exponentials are taken, so its maximum is exact and its O is
// accumulated once; splits are combined by the merge kernel as before.  A key's 32 scores sit in one TMEM lane = one
// thread; column maxima and sums cross the 128 lanes by a halving exchange (16 shuffles) and one shared-memory step.
//
// One CTA walks a run of consecutive splits of one KV head.  Warp 0 issues the TMA loads (one 64-dim x 16-key box per
// lane: a page's rows of one 128-byte column), warp 1 issues the MMAs and owns the tensor memory, warps 2-9 are the
// softmax threads (two warps per TMEM lane quarter, 16 of the 32 query columns each: with four warps the 64 exponentials
// per thread ran as one latency-bound chain, 4.3 us per split against 1.9 us) and afterwards write the accumulator of the
// split out (O is double-buffered in tensor memory, so the next split's score MMAs do not wait for that).  K/V tiles go through a ring of six 32 KB units (two
// 128-byte columns of a tile each: the score MMAs consume K column pair by column pair as it arrives, the P.V MMAs one
// 128-dim half of V at a time) in the order K0 K1 V0 V1 of every split; a unit is released by the tcgen05.commit of the
// MMAs that read it.  Every wait is bounded (error flag, no trap).  No multicast: the tensor maps cover this GPU's
// cache only.
#include "qb_internal.h"
#include "tc_common.cuh"

#include <cuda_fp16.h>
#include <map>
#include <mutex>
#include <tuple>

using namespace qbtc;

namespace {

constexpr int ATC_NQ = 32;              // queries per CTA (MMA N)
constexpr int ATC_TILE = 128;           // keys per MMA tile (MMA M)
constexpr int ATC_THREADS = 320;

template <int HD>
struct AtcCfg {
    static constexpr int UNIT_BYTES = 2 * ATC_TILE * 128;       // a ring unit: two 128-byte columns of a 128-key tile (32 KB)
    static constexpr int UPT = HD / 128;                        // units per tile of K or of V
    static constexpr int NST = 6;                               // ring units (192 KB)
    static constexpr int Q_OFF = NST * UNIT_BYTES;
    static constexpr int Q_BYTES = ATC_NQ * HD * 2;             // [HD / 64][32 queries][128 B]
    static constexpr int P_OFF = Q_OFF + Q_BYTES;
    static constexpr int P_BYTES = 2 * 2 * ATC_NQ * 128;        // [2 tiles][2 key blocks of 64][32 queries][128 B]
    static constexpr int MISC_OFF = P_OFF + P_BYTES;
    static constexpr int MISC_BYTES = 2048;
    static constexpr int TOTAL = MISC_OFF + MISC_BYTES + 1024;  // + slack for the 1024-byte alignment
    static constexpr uint32_t TMEM_COLS = 256;                  // S^T: 2 x 32 columns at 0; O^T: (HD / 128) x 32 columns at 64 and at 128
};


// MN-major operand with the 128-byte swizzle (V^T: 64 dims per 128-byte row, one row per key): 64-dim blocks are
// `lbo` bytes apart, 8-key groups 1024 bytes.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t lbo) {
    uint64_t d = (uint64_t)((addr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D[tmem] (+)= A[smem] * B[smem], fp16 x fp16 -> fp32.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void named_barrier_256() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
// tcgen05.wait::ld naming the registers of an earlier load: what consumes them is ordered after the wait by a data dependency.
__device__ __forceinline__ void tmem_wait_dep(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                   "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :: "memory");
}
// Bounded wait of a warp that is not on the critical path (loader, write-out, the softmax threads between splits): it
// sleeps between polls, so that its polling does not take issue slots from the warps of its scheduler that do the work.
__device__ __forceinline__ bool mbar_wait_idle(uint32_t bar, uint32_t parity, volatile int *abort_flag, uint32_t ns) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
        __nanosleep(ns);
    }
    *abort_flag = 1;
    return false;
}

// Reduction of 16 per-lane values across the 32 lanes of a warp: afterwards lanes j and j + 16 hold op over all lanes of
// value j (8 + 4 + 2 + 1 exchanges and one across the halves; a fixed tree, so the result depends on the inputs alone).
template <bool MAX>
__device__ __forceinline__ float lane_transpose_reduce16(float (&v)[16], uint32_t lane) {
#pragma unroll
    for (int off = 8, n = 16; off >= 1; off >>= 1, n >>= 1) {
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float keep = up ? v[i + n / 2] : v[i];
            const float send = up ? v[i] : v[i + n / 2];
            const float got = __shfl_xor_sync(0xffffffffu, send, off);
            v[i] = MAX ? fmaxf(keep, got) : keep + got;
        }
    }
    const float other = __shfl_xor_sync(0xffffffffu, v[0], 16);
    return MAX ? fmaxf(v[0], other) : v[0] + other;
}
// grid (ceil(max_splits / spc), n_kv, n_seqs * ceil(R / qr)); 320 threads.
template <int HD>
__global__ void __launch_bounds__(ATC_THREADS, 1)
attn_tc_kernel(AttnArgs a, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
               const int32_t *__restrict__ seq_pos, uint32_t R, uint32_t max_splits, uint32_t spc, uint32_t qr) {
    using C = AtcCfg<HD>;
    constexpr uint32_t NST = C::NST, UPT = C::UPT;
    // programmatic dependent launch: announce the dependents at once; everything that needs nothing of the preceding
    // kernel (barriers, tensor memory, the tensor maps' first fetch) is set up before this kernel waits for it
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *misc = smem + C::MISC_OFF;
    // barriers: full[NST], empty[NST], s_full, p_ready, o_full[2], o_free[2]
    const uint32_t bar_full = smem_u32(misc), bar_empty = bar_full + 8 * NST;
    const uint32_t bar_sfull = bar_empty + 8 * NST, bar_pready = bar_sfull + 8, bar_ofull = bar_pready + 8, bar_ofree = bar_ofull + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(misc + 192);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(misc + 196);
    int *qpos = reinterpret_cast<int *>(misc + 256);                    // [32]
    float *red = reinterpret_cast<float *>(misc + 512);                  // [32 queries][4 warps]: per-warp maxima, later sums
    uint32_t *qidx = reinterpret_cast<uint32_t *>(misc + 1280);          // [32] (row * n_heads + head) of query q
    int *page_slot = reinterpret_cast<int *>(misc + 1536);               // [128]

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (uint32_t i = 0; i < NST; ++i) { mbar_init(bar_full + 8 * i, 1); mbar_init(bar_empty + 8 * i, 1); }
        mbar_init(bar_sfull, 1);
        mbar_init(bar_pready, 256);
        for (uint32_t i = 0; i < 2; ++i) { mbar_init(bar_ofull + 8 * i, 1); mbar_init(bar_ofree + 8 * i, 256); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    __syncthreads();                                                     // barriers initialised before warp 0 loads against them
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t split0 = blockIdx.x * spc, kvh = blockIdx.y;
    const uint32_t chunks = (R + qr - 1) / qr;
    const uint32_t seq = blockIdx.z / chunks, chunk = blockIdx.z % chunks;
    const uint32_t r_begin = chunk * qr, r_count = min(qr, R - r_begin);
    const uint32_t G = a.n_heads / a.n_kv;
    const uint32_t NQ = r_count * G;
    const int base_pos = seq_pos[seq] + (int)r_begin;
    const int last_key = base_pos + (int)r_count - 1;
    const int k_begin = (int)(split0 * a.split_keys);
    if (k_begin > last_key) {                                            // nothing to do (uniform per CTA): give the tensor memory back
        tc_fence_before();
        __syncthreads();
        if (warp == 1) {
            tc_fence_after();
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(*tmem_slot), "r"(C::TMEM_COLS) : "memory");
        }
        return;
    }
    const int k_end = min(k_begin + (int)(spc * a.split_keys), last_key + 1);
    const uint32_t n_splits = (uint32_t)(k_end - k_begin + (int)a.split_keys - 1) / a.split_keys;
    const int32_t *pt = a.page_table + (size_t)seq * a.pt_stride;
    const int pg_last = (k_end - 1) >> 4;                                // pages are 16 keys (checked by the launcher)
    const int pg_first = k_begin >> 4;

    // tiles of split s: 1 or 2 (the last split of a sequence may stop inside its first tile)
    auto tiles_of = [&](uint32_t s) -> uint32_t {
        const int kb = k_begin + (int)(s * a.split_keys);
        return (k_end - kb) > ATC_TILE ? 2u : 1u;
    };
    // The loader's cursor over the units of the run: per split K0 [K1] V0 [V1], a tile being UPT units.
    struct Cursor { uint32_t s, item, n_items; };
    auto cur_start = [&]() { Cursor c; c.s = 0; c.item = 0; c.n_items = 2 * tiles_of(0) * UPT; return c; };
    auto cur_next = [&](Cursor &c) {
        if (++c.item >= c.n_items) { ++c.s; c.item = 0; c.n_items = c.s < n_splits ? 2 * tiles_of(c.s) * UPT : 0; }
    };
    auto load_unit = [&](const Cursor &c, uint32_t st) {                 // whole warp 0
        const uint32_t nt = c.n_items / (2 * UPT);
        const uint32_t tile_item = c.item / UPT, u = c.item % UPT, t = tile_item % nt;
        const bool is_v = tile_item >= nt;
        const uint32_t full = bar_full + 8 * st;
        if (lane == 0) mbar_expect_tx(full, C::UNIT_BYTES);
        __syncwarp();
        const int key0 = k_begin + (int)(c.s * a.split_keys) + (int)t * ATC_TILE;
        if (lane < 16) {
            const uint32_t pg_in = lane >> 1, cb = lane & 1;                    // page of the tile, column block of the unit
            // pages past the last key of the run are not looked up: the last valid page is loaded again (finite values,
            // masked by the softmax)
            const int pg = min((key0 >> 4) + (int)pg_in, pg_last);
            const uint32_t dst = smem_u32(smem + (size_t)st * C::UNIT_BYTES) + cb * (ATC_TILE * 128) + pg_in * 2048;
            tma_load_2d(dst, is_v ? &map_v : &map_k, (int)(kvh * HD + (u * 2 + cb) * 64), page_slot[pg - pg_first], full);
        }
    };
    Cursor lc = cur_start();
    uint32_t l_git = 0;
    if (warp == 0) {
        // barriers, the run's page slots (8 splits x 16 pages at most) and the first ring-full of loads, before the rest of
        // the CTA has staged the queries and allocated tensor memory
        for (int i = (int)lane; i <= pg_last - pg_first && i < 128; i += 32) page_slot[i] = pt[pg_first + i] * 16;
        __syncwarp();
        for (; l_git < NST && lc.s < n_splits; ++l_git, cur_next(lc)) load_unit(lc, l_git);
    }
    if (tid < ATC_NQ) {
        qpos[tid] = tid < NQ ? base_pos + (int)(tid / G) : -1;
        qidx[tid] = (uint32_t)(((size_t)seq * R + r_begin + tid / G) * a.n_heads + kvh * G + tid % G);
    }
    // the queries, scaled, fp16, in the K-major swizzled operand layout: [HD / 64][32 rows][128 B], 16-byte chunk c of row q
    // stored at chunk c ^ (q % 8); rows past the last query are zero
    {
        const float scale = rsqrtf((float)HD);
        for (uint32_t i = tid; i < ATC_NQ * (HD / 8); i += ATC_THREADS) {
            const uint32_t q = i / (HD / 8), c8 = i % (HD / 8);        // 8 consecutive dims
            uint4 packed = make_uint4(0u, 0u, 0u, 0u);
            if (q < NQ) {
                const uint32_t rl = q / G, gq = q - rl * G;
                const float *src = a.qkv + ((size_t)seq * R + r_begin + rl) * a.row_stride + (size_t)(kvh * G + gq) * 2 * HD + c8 * 8;
                const float4 f0 = *reinterpret_cast<const float4 *>(src), f1 = *reinterpret_cast<const float4 *>(src + 4);
                const __half2 h0 = __floats2half2_rn(f0.x * scale, f0.y * scale), h1 = __floats2half2_rn(f0.z * scale, f0.w * scale);
                const __half2 h2 = __floats2half2_rn(f1.x * scale, f1.y * scale), h3 = __floats2half2_rn(f1.z * scale, f1.w * scale);
                packed = make_uint4(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1),
                                    *reinterpret_cast<const uint32_t *>(&h2), *reinterpret_cast<const uint32_t *>(&h3));
            }
            const uint32_t ka = c8 / 8, ch = c8 % 8;
            *reinterpret_cast<uint4 *>(smem + C::Q_OFF + ka * (ATC_NQ * 128) + q * 128 + ((ch ^ (q & 7)) * 16)) = packed;
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");        // the MMAs read Q through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 64;      // O buffer b at tmem_o + 64 * b

    if (warp == 0) {
        // ---- loader: the rest of the units, each into the ring unit its predecessor of NST units ago has left ----
        for (; lc.s < n_splits; ++l_git, cur_next(lc)) {
            const uint32_t st = l_git % NST, ph = (l_git / NST) & 1;
            if (!__all_sync(0xffffffffu, mbar_wait_idle(bar_empty + 8 * st, ph ^ 1, abort_flag, 100))) break;
            load_unit(lc, st);
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            // instruction descriptors: D fp32, A and B fp16, N = 32, M = 128; the P.V form reads A MN-major
            constexpr uint32_t idesc_qk = (1u << 4) | ((uint32_t)(ATC_NQ >> 3) << 17) | ((128u >> 4) << 24);
            constexpr uint32_t idesc_pv = idesc_qk | (1u << 15);
            const uint32_t q_addr = smem_u32(smem + C::Q_OFF), p_addr = smem_u32(smem + C::P_OFF);
            uint32_t git = 0;
            bool ok = true;
            for (uint32_t s = 0; s < n_splits && ok; ++s) {
                const uint32_t nt = tiles_of(s), sph = s & 1, ob = s & 1, oph = (s >> 1) & 1;
                // (S is free: the softmax threads read the previous split's scores before they released its P)
                for (uint32_t t = 0; t < nt && ok; ++t)
                    for (uint32_t u = 0; u < UPT; ++u, ++git) {                       // unit u: dims [128 u, 128 u + 128) of the keys
                        const uint32_t st = git % NST, ph = (git / NST) & 1;
                        if (!mbar_wait(bar_full + 8 * st, ph, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t k_addr = smem_u32(smem + (size_t)st * C::UNIT_BYTES);
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks)
                            tc_mma_f16(tmem_s + t * ATC_NQ, smem_desc_sw128(k_addr + (ks / 4) * (ATC_TILE * 128) + (ks % 4) * 32),
                                       smem_desc_sw128(q_addr + (u * 2 + ks / 4) * (ATC_NQ * 128) + (ks % 4) * 32), idesc_qk, (u > 0 || ks > 0) ? 1u : 0u);
                        tc_commit(bar_empty + 8 * st);
                    }
                if (!ok) break;
                tc_commit(bar_sfull);
                if (!mbar_wait(bar_pready, sph, abort_flag)) break;
                if (!mbar_wait(bar_ofree + 8 * ob, oph ^ 1, abort_flag)) break;       // this O buffer has been written out
                tc_fence_after();
                for (uint32_t t = 0; t < nt && ok; ++t)
                    for (uint32_t u = 0; u < UPT; ++u, ++git) {                       // unit u: output dims [128 u, 128 u + 128)
                        const uint32_t st = git % NST, ph = (git / NST) & 1;
                        if (!mbar_wait(bar_full + 8 * st, ph, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t v_addr = smem_u32(smem + (size_t)st * C::UNIT_BYTES);
#pragma unroll
                        for (int ks = 0; ks < ATC_TILE / 16; ++ks)
                            tc_mma_f16(tmem_o + ob * 64 + u * ATC_NQ, smem_desc_mn_sw128(v_addr + ks * 2048, ATC_TILE * 128),
                                       smem_desc_sw128(p_addr + t * (2 * ATC_NQ * 128) + (ks / 4) * (ATC_NQ * 128) + (ks % 4) * 32),
                                       idesc_pv, (t > 0 || ks > 0) ? 1u : 0u);
                        tc_commit(bar_empty + 8 * st);
                    }
                if (!ok) break;
                tc_commit(bar_ofull + 8 * ob);
            }
        }
    } else {
        // ---- softmax and write-out: 8 warps, two per TMEM lane quarter.  For the softmax a thread is key row `r` of a tile
        // (= TMEM lane r) and owns 16 of the 32 query columns; for the write-out it is output dim r of one 128-dim half. ----
        const uint32_t quarter = warp & 3, half = (warp - 2) >> 2, r = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32u) << 16;
        const uint32_t q0 = half * 16;                                   // first query column of this thread
        const float4 *red4 = reinterpret_cast<const float4 *>(red);
        uint8_t *prow = smem + C::P_OFF + (r >> 6) * (ATC_NQ * 128) + (r & 7) * 2;
        const uint32_t ch = (r & 63) >> 3;
        bool ok = true;
        for (uint32_t s = 0; s < n_splits && ok; ++s) {
            const uint32_t nt = tiles_of(s), sph = s & 1, ob = s & 1, oph = (s >> 1) & 1, split = split0 + s;
            const int kb = k_begin + (int)(s * a.split_keys);
            if (!__all_sync(0xffffffffu, mbar_wait_idle(bar_sfull, sph, abort_flag, 50))) { ok = false; break; }
            tc_fence_after();
            uint32_t raw0[16], raw1[16];
            tmem_ld16(tmem_s + lane_addr + q0, raw0);
            if (nt > 1) tmem_ld16(tmem_s + lane_addr + ATC_NQ + q0, raw1);   // warp-uniform
            tmem_wait_dep(raw0);
            if (nt > 1) tmem_wait_dep(raw1);
            float s0[16], s1[16], mx[16];
            // a split that lies before every query position needs no mask (the zero rows past the last query score 0 against
            // everything: harmless, never written out)
            if (kb + 2 * ATC_TILE <= min(base_pos + 1, k_end)) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    s0[j] = __uint_as_float(raw0[j]);
                    s1[j] = __uint_as_float(raw1[j]);
                    mx[j] = fmaxf(s0[j], s1[j]);
                }
            } else {
                const int key_a = kb + (int)r, key_b = key_a + ATC_TILE;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int qp = qpos[q0 + j];
                    s0[j] = (key_a <= qp && key_a < k_end) ? __uint_as_float(raw0[j]) : -INFINITY;
                    s1[j] = (nt > 1 && key_b <= qp && key_b < k_end) ? __uint_as_float(raw1[j]) : -INFINITY;
                    mx[j] = fmaxf(s0[j], s1[j]);
                }
            }
            const float wmax = lane_transpose_reduce16<true>(mx, lane);   // lanes j and j + 16: maximum of query q0 + j over this warp's keys
            if (lane < 16) red[(q0 + lane) * 4 + quarter] = wmax;
            named_barrier_256();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float4 m4 = red4[q0 + j];
                mx[j] = fmaxf(fmaxf(m4.x, m4.y), fmaxf(m4.z, m4.w));
            }
            // (s0 then holds the packed pair of probabilities, s1 the row-sum contribution)
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float m = mx[j];
                float p0 = 0.0f, p1 = 0.0f;
                if (m != -INFINITY) { p0 = __expf(s0[j] - m); p1 = __expf(s1[j] - m); }
                const __half2 hp = __floats2half2_rn(p0, p1);
                // the row sum uses the rounded probabilities, the values the tensor cores multiply with V
                const float2 fp = __half22float2(hp);
                s1[j] = fp.x + fp.y;
                s0[j] = __uint_as_float(*reinterpret_cast<const uint32_t *>(&hp));
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t q = q0 + j, off = q * 128 + ((ch ^ (q & 7)) * 16);
                const uint32_t bits = __float_as_uint(s0[j]);
                *reinterpret_cast<uint16_t *>(prow + off) = (uint16_t)(bits & 0xffffu);
                *reinterpret_cast<uint16_t *>(prow + 2 * ATC_NQ * 128 + off) = (uint16_t)(bits >> 16);     // second tile (zeros when absent)
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");                    // P is read through the async proxy
            mbar_arrive(bar_pready);
            // off the critical path: the split's (max, sum) per query ...
            const float4 mm = red4[q0 + (lane & 15)];
            const float m_mine = fmaxf(fmaxf(mm.x, mm.y), fmaxf(mm.z, mm.w));
            const float wsum = lane_transpose_reduce16<false>(s1, lane);
            named_barrier_256();                                          // everybody has read the maxima
            if (lane < 16) red[(q0 + lane) * 4 + quarter] = wsum;
            named_barrier_256();
            if (quarter == 0 && lane < 16 && q0 + lane < NQ) {
                const size_t pidx = (size_t)qidx[q0 + lane] * max_splits + split;
                const float4 l4 = red4[q0 + lane];
                a.part_ml[pidx * 2] = m_mine;
                a.part_ml[pidx * 2 + 1] = ((l4.x + l4.y) + l4.z) + l4.w;
            }
            named_barrier_256();                                          // red may be rewritten by the next split
            // ... and the write-out of the split's accumulator once its P.V products are done
            if (!__all_sync(0xffffffffu, mbar_wait_idle(bar_ofull + 8 * ob, oph, abort_flag, 50))) { ok = false; break; }
            tc_fence_after();
            if (HD == 256) {
                uint32_t o[32];
                tmem_ld32(tmem_o + ob * 64 + lane_addr + half * ATC_NQ, o);
                tmem_ld_wait();
                const uint32_t dim = half * 128 + r;
#pragma unroll
                for (int q = 0; q < 32; ++q)
                    if ((uint32_t)q < NQ) a.part_acc[((size_t)qidx[q] * max_splits + split) * HD + dim] = __uint_as_float(o[q]);
            } else {
                uint32_t o[16];
                tmem_ld16(tmem_o + ob * 64 + lane_addr + q0, o);
                tmem_wait_dep(o);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (q0 + j < NQ) a.part_acc[((size_t)qidx[q0 + j] * max_splits + split) * HD + r] = __uint_as_float(o[j]);
            }
            tc_fence_before();
            mbar_arrive(bar_ofree + 8 * ob);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0 && a.err_flag) atomicExch(a.err_flag, 2000 + (int)(blockIdx.x % 1000));
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);                // let this CTA's copies in flight land
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
    }
}

struct KvMapKey {
    int dev; const void *p; uint32_t hd, n_kv;
    bool operator<(const KvMapKey &o) const { return std::tie(dev, p, hd, n_kv) < std::tie(o.dev, o.p, o.hd, o.n_kv); }
};
std::map<KvMapKey, CUtensorMap> g_kv_maps;
std::mutex g_kv_lock;

// The cache as a 2-D tensor: a slot's n_kv * hd halfs are a row; a box is one 128-byte column of 16 slots (one page).
int kv_map(qb_ctx *ctx, const __half *cache, uint32_t hd, uint32_t n_kv, CUtensorMap *out) {
    std::lock_guard<std::mutex> lock(g_kv_lock);
    if (g_kv_maps.size() > 4096) g_kv_maps.clear();
    const KvMapKey key{ctx->device, cache, hd, n_kv};
    auto it = g_kv_maps.find(key);
    if (it == g_kv_maps.end()) {
        CUtensorMap m;
        // the slot extent only bounds the coordinates TMA accepts; the kernel asks for pages of the page table alone
        QB_TRY(qb_make_tmap_2d(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, cache, (uint64_t)n_kv * hd, 1ull << 30, (uint64_t)n_kv * hd * 2, 64, 16,
                               CU_TENSOR_MAP_SWIZZLE_128B));
        it = g_kv_maps.emplace(key, m).first;
    }
    *out = it->second;
    return QB_OK;
}

template <int HD>
int launch_tc(qb_ctx *ctx, const AttnArgs &a, const int32_t *seq_pos, uint32_t R, uint32_t n_seqs, uint32_t max_splits) {
    using C = AtcCfg<HD>;
    QB_CUDA(cudaFuncSetAttribute(attn_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
    CUtensorMap mk, mv;
    QB_TRY(kv_map(ctx, a.k_cache, a.hd, a.n_kv, &mk));
    QB_TRY(kv_map(ctx, a.v_cache, a.hd, a.n_kv, &mv));
    const uint32_t G = a.n_heads / a.n_kv;
    const uint32_t qr = std::max(1u, (uint32_t)ATC_NQ / G);
    const uint32_t zdim = n_seqs * ((R + qr - 1) / qr);
    const uint32_t ctas = max_splits * a.n_kv * zdim;
    const uint32_t spc = std::min(8u, std::max(1u, (ctas + (uint32_t)ctx->sm_count - 1) / (uint32_t)ctx->sm_count));
    dim3 grid((max_splits + spc - 1) / spc, a.n_kv, zdim);
    QB_CUDA(qb_launch_pdl(ctx->stream, attn_tc_kernel<HD>, dim3(grid), dim3(ATC_THREADS), (size_t)C::TOTAL, a, mk, mv, seq_pos, R, max_splits, spc, qr));
    QB_LAUNCHED(ctx, "attn_tc_kernel");
    return QB_OK;
}

}  // namespace

// Whether the tensor-memory kernel takes this call: 16-key pages, 256-key splits, head size 128 or 256, 16-byte aligned
// cache rows.  Anything else runs attn_split_kernel.
bool qb_attn_tc_supports(const AttnArgs &a) {
    return (a.hd == 256 || a.hd == 128) && a.page_size == 16 && a.split_keys == 256 && a.n_heads / a.n_kv <= 8 &&
           ((uintptr_t)a.k_cache & 15) == 0 && ((uintptr_t)a.v_cache & 15) == 0 && ((uintptr_t)a.qkv & 15) == 0 && a.row_stride % 4 == 0;
}

int qb_attn_tc_launch(qb_ctx *ctx, const AttnArgs &a, const int32_t *seq_pos, uint32_t R, uint32_t n_seqs, uint32_t max_splits) {
    if (a.hd == 256) return launch_tc<256>(ctx, a, seq_pos, R, n_seqs, max_splits);
    return launch_tc<128>(ctx, a, seq_pos, R, n_seqs, max_splits);
}
