// Q8_0 x Q8 product on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// Stands in for the INT8-MMA kernels of the reference (mmq_q8_0_vmed_kernel / mmq_q8_0_v8_kernel,
// src/mmq_q8.cu:1795-2248, mma.sync.m16n8k32.s8) with the same arithmetic per output: the exact int32
// dot of every 32-block, acc = fma(d_w*d_x, float(dot), acc) over the blocks of a K segment in
// ascending order, one partial sum per segment (bit-identical to the CUDA-core kernel of this library).
//
// Shape of the kernel ("swap-AB"): the 128 weight rows of a CTA are the MMA's M dimension, the
// activation rows are its N dimension (16..128), and one tcgen05.mma.kind::i8 (K = 32 bytes) covers
// exactly one Q8_0 block.  Every block therefore gets its OWN accumulator columns in tensor memory
// (never accumulated across blocks), and the epilogue warps drain them and apply the per-block scales
// in order.  The weight record of a stage (quants already in the swizzled operand order + scales)
// arrives as one 17 KB bulk copy, the activation tile and its scales by tensor-map TMA (128-byte
// swizzle), all through one mbarrier pipeline; the kernel is an HBM streaming kernel until the
// activation-row count reaches the hundreds.
//
// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (owns the TMEM allocation), warps 2.. = epilogue
// (TMEM lane quarter = warp % 4; four warps for the small tiles, eight from 32 activation rows on).  Every wait is bounded: when a wait runs out
// the CTA raises the context's error flag, lets its copies land, frees its TMEM and returns.
#include "qb_internal.h"
#include "tc_common.cuh"

#include <mutex>

namespace {
using namespace qbtc;

// MT = activation rows per tile (MMA N).  NLD = accumulator columns the epilogue reads (<= MT).
// A pipeline stage holds one weight record (17 KB, one bulk copy, already the swizzled operand image
// plus its scales), the activation tile (MT x 128 B, tensor-map TMA with the 128-byte swizzle) and
// the activation scales.  TMEM: every stage (MT <= 64) or half stage (MT = 128) has its own slot.
template <int MT, int NLD>
struct TcCfg {
    static constexpr int KPS = MT == 128 ? 2 : 4;              // 32-blocks per TMEM slot
    static constexpr int SPS = 4 / KPS;                        // slots per pipeline stage
    // Small tiles run two CTAs per SM (two independent producer/MMA/epilogue chains per SM: the per-stage
    // handshake chain of one CTA, not the memory system, limits a single chain to ~33 GB/s), so each CTA
    // takes half the tensor memory and half the shared memory.
    static constexpr int CTAS_PER_SM = MT == 16 ? 2 : 1;
    // Second launch bound.  Left unspecified, the compiler keeps several variants at 64 registers with spills inside
    // the drain loop (it assumes more resident CTAs than the shared memory allows); told the real residency it uses
    // 94-168 registers and no spills.  The 32-column variant measured faster with the default, so it keeps it (0).
    static constexpr int MIN_CTAS = MT == 32 ? 0 : CTAS_PER_SM;
    static constexpr int NSLOT = 512 / CTAS_PER_SM / (KPS * MT);
    static constexpr int TMEM_COLS = NSLOT * KPS * MT;
    static constexpr int B_OFF = (int)QB_REC_BYTES;            // 17 * 1024: the activation tile stays 1024-aligned
    static constexpr int B_BYTES = MT * 128;
    static constexpr int XD_OFF = B_OFF + B_BYTES;
    static constexpr int XD_BYTES = 4 * MT * 4;
    static constexpr int TX_BYTES = (int)QB_REC_BYTES + B_BYTES + XD_BYTES;
    static constexpr int STAGE = (XD_OFF + XD_BYTES + 1023) / 1024 * 1024;
    static constexpr int BAR_BYTES = 1024;
    // fused SwiGLU (small tiles only): the up half of a tile's rows hands its sums to the gate half, two buffers
    static constexpr int EX_BYTES = MT == 16 ? 2 * NLD * 64 * 4 : 0;
    static constexpr int NST_FIT = (232448 / CTAS_PER_SM - BAR_BYTES - EX_BYTES - 2048) / STAGE;
    static constexpr int NST = NST_FIT > 8 ? 8 : NST_FIT;
    static constexpr int TOTAL = STAGE * NST + BAR_BYTES + EX_BYTES + 1024;   // + slack to align the base to 1024
    static constexpr int CH = NLD < 16 ? NLD : 16;               // columns per tcgen05.ld
    // Epilogue warps: four for the small tiles (one per TMEM lane quarter); eight from MT = 32 and sixteen at
    // MT = 128 (two / four per quarter, each taking a slice of the activation columns): the drain + rescale of a
    // large tile is bound by instruction issue and dependent latencies, which more warps per scheduler hide.
    static constexpr int EPI_WARPS = MT >= 64 ? 16 : MT >= 32 ? 8 : 4;
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
    static constexpr int NC = NLD / (EPI_WARPS / 4);             // accumulator columns per epilogue thread
};

// Persistent kernel: CTA b works on units b, b + gridDim.x, ...; a unit is (activation tile, K segment,
// 128-row weight tile).  The TMA / MMA / TMEM pipeline keeps running across unit boundaries.
template <int MT, int NLD>
__global__ void __launch_bounds__((TcCfg<MT, NLD>::THREADS), (TcCfg<MT, NLD>::MIN_CTAS))
gemm_tc_kernel(const uint8_t *__restrict__ rec, const __grid_constant__ CUtensorMap map_xq,
               const __grid_constant__ CUtensorMap map_xd, uint32_t K, uint32_t N, uint32_t M, float *__restrict__ part,
               uint32_t S, uint32_t tiles, uint32_t units, int *err_flag, unsigned long long *tl,
               const __grid_constant__ QbGemmPush push, const QbGemmSwiglu swz) {
    using C = TcCfg<MT, NLD>;
    constexpr uint32_t NST = C::NST, NSLOT = C::NSLOT;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *bar_mem = smem + (size_t)C::STAGE * NST;
    // barrier layout: full[NST], empty[NST], tmem_full[NSLOT], tmem_empty[NSLOT]
    const uint32_t bar_full = smem_u32(bar_mem), bar_empty = bar_full + 8 * NST;
    const uint32_t bar_tfull = bar_empty + 8 * NST, bar_tempty = bar_tfull + 8 * NSLOT;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_mem + 8 * (2 * NST + 2 * NSLOT));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar_ex = smem_u32(bar_mem + 512);                  // two "up half stored" barriers (fused SwiGLU)
    float *ex = reinterpret_cast<float *>(bar_mem + C::BAR_BYTES);    // [2][NLD][64]

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nchunks = K / 128;
    constexpr uint32_t tmem_cols = C::TMEM_COLS;

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < NST; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1 + C::EPI_WARPS);   // MMA commit + one lane of every epilogue warp
        }
        for (uint32_t i = 0; i < NSLOT; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, C::EPI_WARPS);
        }
        mbar_init(bar_ex, 2);
        mbar_init(bar_ex + 8, 2);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the consumer of the partials may be scheduled already

    // unit -> (m tile, segment, row tile); consecutive units of a CTA differ in the row tile
    auto decode = [&](uint32_t u, uint32_t &tile, uint32_t &seg, uint32_t &m0, uint32_t &c_begin, uint32_t &n_it) {
        const uint32_t per_m = tiles * S;
        m0 = (u / per_m) * MT;
        const uint32_t rem = u % per_m;
        seg = rem / tiles;
        tile = rem % tiles;
        c_begin = tc_seg_begin(seg, S, nchunks);
        n_it = tc_seg_begin(seg + 1, S, nchunks) - c_begin;
    };

    if (warp == 0) {
        if (lane == 0) {
            // Stage cursor over this CTA's units.  The launch is programmatically serialised behind the kernel
            // that produces the activations: the weight records of the first NST stages (which depend on nothing)
            // are requested at once, then the CTA waits for the preceding grid and only then requests activations.
            struct Cursor { uint32_t u, it, n_it, tile, m0, c_begin; bool valid; };
            auto start = [&](uint32_t u) {
                Cursor c; c.u = u; c.it = 0; c.valid = u < units; c.n_it = 0; c.tile = c.m0 = c.c_begin = 0;
                if (c.valid) { uint32_t seg; decode(u, c.tile, seg, c.m0, c.c_begin, c.n_it); }
                return c;
            };
            auto next = [&](Cursor &c) {
                if (++c.it >= c.n_it) c = start(c.u + gridDim.x);
            };
            auto load_w = [&](const Cursor &c, uint32_t st) {
                const uint32_t base = smem_u32(smem + (size_t)st * C::STAGE), full = bar_full + 8 * st;
                mbar_expect_tx(full, C::TX_BYTES);
                bulk_load(base, rec + ((size_t)c.tile * nchunks + c.c_begin + c.it) * QB_REC_BYTES, QB_REC_BYTES, full);
            };
            auto load_x = [&](const Cursor &c, uint32_t st) {
                const uint32_t base = smem_u32(smem + (size_t)st * C::STAGE), full = bar_full + 8 * st;
                const int k0 = (int)((c.c_begin + c.it) * 128);
                tma_load_2d(base + C::B_OFF, &map_xq, k0, (int)c.m0, full);
                tma_load_2d(base + C::XD_OFF, &map_xd, (int)c.m0, k0 / 32, full);
            };
            if (tl) tl[blockIdx.x * 4 + 0] = qb_globaltimer();
            Cursor head = start(blockIdx.x), c = head;
            uint32_t npre = 0;
            for (; npre < NST && c.valid; ++npre, next(c)) load_w(c, npre);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (tl) tl[blockIdx.x * 4 + 1] = qb_globaltimer();
            c = head;
            for (uint32_t g = 0; g < npre; ++g, next(c)) load_x(c, g);
            for (uint32_t git = npre; c.valid; ++git, next(c)) {
                const uint32_t st = git % NST, ph = (git / NST) & 1;
                if (!mbar_wait(bar_empty + 8 * st, ph ^ 1, abort_flag)) break;
                load_w(c, st);
                load_x(c, st);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N = MT, M = 128
            constexpr uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MT >> 3) << 17) | ((128u >> 4) << 24);
            uint32_t git = 0, j = 0;
            bool ok = true;
            for (uint32_t u = blockIdx.x; u < units && ok; u += gridDim.x) {
                uint32_t tile, seg, m0, c_begin, n_it;
                decode(u, tile, seg, m0, c_begin, n_it);
                for (uint32_t it = 0; it < n_it && ok; ++it, ++git) {
                    const uint32_t st = git % NST, ph = (git / NST) & 1;
                    if (!mbar_wait(bar_full + 8 * st, ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + (size_t)st * C::STAGE), b_addr = a_addr + C::B_OFF;
                    for (int sp = 0; sp < C::SPS; ++sp, ++j) {
                        const uint32_t slot = j % NSLOT, sph = (j / NSLOT) & 1;
                        if (!mbar_wait(bar_tempty + 8 * slot, sph ^ 1, abort_flag)) { ok = false; break; }
                        tc_fence_after();
#pragma unroll
                        for (int kl = 0; kl < C::KPS; ++kl) {
                            const int kb = sp * C::KPS + kl;
                            tc_mma_i8(tmem_base + slot * (C::KPS * MT) + kl * MT, smem_desc_sw128(a_addr + kb * 32),
                                      smem_desc_sw128(b_addr + kb * 32), idesc);
                        }
                        tc_commit(bar_tfull + 8 * slot);
                    }
                    if (ok) tc_commit(bar_empty + 8 * st);
                }
            }
        }
    } else {
        const uint32_t quarter = warp & 3;                     // TMEM lanes [32*quarter, +32)
        const uint32_t r = quarter * 32 + lane;                // weight row inside the tile
        uint32_t git = 0, j = 0;
        bool ok = true;
        for (uint32_t u = blockIdx.x; u < units && ok; u += gridDim.x) {
            uint32_t tile, seg, m0, c_begin, n_it;
            decode(u, tile, seg, m0, c_begin, n_it);
            float acc[C::NC];
#pragma unroll
            for (int i = 0; i < C::NC; ++i) acc[i] = 0.0f;
            if constexpr (NLD <= 16) {
                // Small activation tiles (the HBM-bound regime): the scales of a stage are copied to registers
                // as soon as the stage has landed and the stage is released at once, one stage ahead of the
                // TMEM work, so the producer never waits for the accumulator drain.
                float dw_n[4], dx_n[4][NLD];
                auto fetch_scales = [&](uint32_t g) -> bool {
                    const uint32_t st = g % NST, ph = (g / NST) & 1;
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * st, ph, abort_flag))) return false;
                    const uint8_t *stage = smem + (size_t)st * C::STAGE;
                    const __half *wd = reinterpret_cast<const __half *>(stage + QB_REC_Q_BYTES);
                    const float *xd = reinterpret_cast<const float *>(stage + C::XD_OFF);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        dw_n[kb] = __half2float(wd[kb * 128 + r]);
#pragma unroll
                        for (int i = 0; i < NLD; ++i) dx_n[kb][i] = xd[kb * MT + i];
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_empty + 8 * st);
                    return true;
                };
                if (n_it > 0 && !fetch_scales(git)) ok = false;
                for (uint32_t it = 0; it < n_it && ok; ++it, ++git, ++j) {
                    float sc[4][NLD];
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb)
#pragma unroll
                        for (int i = 0; i < NLD; ++i) sc[kb][i] = __fmul_rn(dw_n[kb], dx_n[kb][i]);
                    if (it + 1 < n_it && !fetch_scales(git + 1)) { ok = false; break; }
                    const uint32_t slot = j % NSLOT, sph = (j / NSLOT) & 1;      // one slot per stage here
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * slot, sph, abort_flag))) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + slot * (4 * MT);
                    int32_t v[4][NLD];
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) tmem_ld<NLD>(taddr + kb * MT, v[kb]);
                    tmem_ld_wait();
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb)
#pragma unroll
                        for (int i = 0; i < NLD; ++i) acc[i] = __fmaf_rn(sc[kb][i], (float)v[kb][i], acc[i]);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tempty + 8 * slot);
                }
            } else {
                // Large activation tiles: this warp drains columns [c_base, c_base + NC) of its lane quarter.  The
                // TMEM loads are software-pipelined: the next 16 columns are in flight while the current 16 are
                // rescaled.
                constexpr int NC = C::NC, NCH = NC / 16;                // 16-column chunks per 32-block
                const uint32_t c_base = ((warp - 2) >> 2) * NC;
                f32x2 acc2[NC / 2];                                     // column pairs, packed arithmetic
#pragma unroll
                for (int i = 0; i < NC / 2; ++i) acc2[i] = pack2(0.0f, 0.0f);
                for (uint32_t it = 0; it < n_it && ok; ++it, ++git) {
                    // The stage's own barrier is not waited for: the MMAs whose completion the slot barrier reports were
                    // issued after the stage had landed, and a wait that has nothing to wait for still costs this warp a
                    // barrier round trip per stage (the drain is a chain of such latencies).
                    const uint32_t st = git % NST;
                    const uint8_t *stage = smem + (size_t)st * C::STAGE;
                    const __half *wd = reinterpret_cast<const __half *>(stage + QB_REC_Q_BYTES);
                    const float *xd = reinterpret_cast<const float *>(stage + C::XD_OFF) + c_base;
                    for (int sp = 0; sp < C::SPS; ++sp, ++j) {
                        const uint32_t slot = j % NSLOT, sph = (j / NSLOT) & 1;
                        // warp-uniform results: the TMEM loads below are .aligned
                        if (!__all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * slot, sph, abort_flag))) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t tbase = tmem_base + ((quarter * 32u) << 16) + slot * (C::KPS * MT) + c_base;
                        int32_t v[2][16];
                        tmem_ld<16>(tbase, v[0]);
#pragma unroll
                        for (int q = 0; q < C::KPS * NCH; ++q) {
                            const int kl = q / NCH, c0 = (q % NCH) * 16, kb = sp * C::KPS + kl;
                            tmem_ld_wait16(v[q & 1]);
                            if (q + 1 < C::KPS * NCH) tmem_ld<16>(tbase + ((q + 1) / NCH) * MT + ((q + 1) % NCH) * 16, v[(q + 1) & 1]);
                            const float dw = __half2float(wd[kb * 128 + r]);
                            const f32x2 dw2 = pack2(dw, dw);
                            // four scales per shared-memory load, read as the two packed pairs the arithmetic takes (no repacking)
                            const ulonglong2 *xd4 = reinterpret_cast<const ulonglong2 *>(xd + kb * MT + c0);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const ulonglong2 x4 = xd4[i];
                                acc2[c0 / 2 + 2 * i] = fma2(mul2(dw2, x4.x), pack2((float)v[q & 1][4 * i], (float)v[q & 1][4 * i + 1]), acc2[c0 / 2 + 2 * i]);
                                acc2[c0 / 2 + 2 * i + 1] = fma2(mul2(dw2, x4.y), pack2((float)v[q & 1][4 * i + 2], (float)v[q & 1][4 * i + 3]), acc2[c0 / 2 + 2 * i + 1]);
                            }
                        }
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_tempty + 8 * slot);
                    }
                    if (ok) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_empty + 8 * st);
                    }
                }
#pragma unroll
                for (int i = 0; i < NC / 2; ++i) unpack2(acc2[i], acc[2 * i], acc[2 * i + 1]);
            }
            if constexpr (MT == 16) {
                if (swz.q != nullptr) {
                    // fused SwiGLU: rows 64..127 of the tile are the up rows of the hidden indices whose gate rows are
                    // rows 0..63: the up warps hand their sums over, the gate warps finish (a warp = one 32-block)
                    const uint32_t n_unit = (u - blockIdx.x) / gridDim.x, buf = n_unit & 1, exph = (n_unit >> 1) & 1;
                    float *exb = ex + buf * (NLD * 64);
                    if (quarter >= 2) {
                        if (ok) {
#pragma unroll
                            for (int i = 0; i < NLD; ++i) exb[i * 64 + (r - 64)] = acc[i];
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_ex + 8 * buf);          // arrives also when aborting: nobody waits in vain
                    } else {
                        if (!__all_sync(0xffffffffu, mbar_wait(bar_ex + 8 * buf, exph, abort_flag))) ok = false;
                        if (ok) {
                            const uint32_t hidx = tile * 64 + r;               // hidden index of this thread's gate row
#pragma unroll
                            for (int i = 0; i < NLD; ++i) {
                                const uint32_t m = m0 + i;
                                if (m < M)                                       // warp-uniform
                                    quant_block_store(qb_swiglu(acc[i], exb[i * 64 + r]), (int)lane, swz.q + (size_t)m * swz.q_pitch + (hidx & ~31u),
                                                      swz.d + (size_t)(hidx >> 5) * swz.d_ld + m);
                            }
                        }
                    }
                    continue;
                }
            }
            const uint32_t row = tile * 128 + r;
            if (ok && row < N) {
#pragma unroll
                for (int i = 0; i < C::NC; ++i) {
                    const uint32_t m = m0 + (C::EPI_WARPS > 4 ? ((warp - 2) >> 2) * C::NC : 0u) + i;
                    if (m < M) {
                        const size_t o = ((size_t)seg * M + m) * N + row;
                        if (push.n == 0) part[o] = acc[i];
                        else for (uint32_t p = 0; p < push.n; ++p) push.dst[p][o] = acc[i];
                    }
                }
            }
        }
        if (push.n) __threadfence_system();     // this thread's partial sums are visible to every GPU before the CTA signals
    }
    tc_fence_before();
    __syncthreads();
    if (push.n && threadIdx.x == 0) {
        __threadfence_system();
        for (uint32_t p = 0; p < push.n; ++p) atomicAdd_system(push.counter[p], 1u);
    }
    if (tl && threadIdx.x == 0) {
        tl[blockIdx.x * 4 + 2] = qb_globaltimer();
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        tl[blockIdx.x * 4 + 3] = smid;
    }
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(err_flag, 1000 + (int)(blockIdx.x % 1000));
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);      // let this CTA's copies in flight land
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// Tensor maps of the activation buffers, cached per (device, buffer, shape): the engine reuses a handful of buffers,
// the op-level entry points may see many, so the cache is emptied when it grows large.  One lock for both maps.
struct MapKey {
    int dev; const void *p; uint32_t a, b, c;
    bool operator<(const MapKey &o) const { return std::tie(dev, p, a, b, c) < std::tie(o.dev, o.p, o.a, o.b, o.c); }
};
std::map<MapKey, CUtensorMap> g_xq_maps, g_xd_maps;
std::mutex g_map_lock;
constexpr size_t MAP_CACHE_MAX = 4096;

template <int MT, int NLD>
int launch_tc(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part, uint32_t S,
              const QbGemmPush *push, uint32_t *grid_out, const QbGemmSwiglu *swiglu) {
    using C = TcCfg<MT, NLD>;
    // the attribute belongs to the current device: set on every launch (a process may drive several GPUs)
    QB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<MT, NLD>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
    const uint32_t K = w->cols, ld = qb_act_ld(M);
    MapKey kq{ctx->device, q, M, K, (uint32_t)MT}, kd{ctx->device, d, M, K, (uint32_t)MT};
    CUtensorMap map_q, map_d;
    {
        std::lock_guard<std::mutex> lock(g_map_lock);
        if (g_xq_maps.size() > MAP_CACHE_MAX) g_xq_maps.clear();
        if (g_xd_maps.size() > MAP_CACHE_MAX) g_xd_maps.clear();
        auto iq = g_xq_maps.find(kq);
        if (iq == g_xq_maps.end()) {
            CUtensorMap mq;
            QB_TRY(qb_make_tmap_2d(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q, K, M, K, 128, MT, CU_TENSOR_MAP_SWIZZLE_128B));
            iq = g_xq_maps.emplace(kq, mq).first;
        }
        auto id = g_xd_maps.find(kd);
        if (id == g_xd_maps.end()) {
            CUtensorMap md;
            QB_TRY(qb_make_tmap_2d(&md, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, d, ld, K / 32, (uint64_t)ld * 4, MT, 4, CU_TENSOR_MAP_SWIZZLE_NONE));
            id = g_xd_maps.emplace(kd, md).first;
        }
        map_q = iq->second; map_d = id->second;
    }
    const uint32_t tiles = w->rows_pad / 128;
    const uint32_t units = tiles * S * ((M + MT - 1) / MT);
    const uint32_t grid = std::min<uint32_t>(units, (uint32_t)ctx->sm_count * C::CTAS_PER_SM);
    const size_t smem_bytes = C::TOTAL;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start while the previous kernel drains
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    QB_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<MT, NLD>, (const uint8_t *)w->rec, map_q, map_d, K, w->rows, M, part, S,
                               tiles, units, ctx->err_flag_dev, qb_timeline_slot(ctx, grid, (double)w->rows_pad * K / 32.0 * 34.0 + (double)M * K * 1.125 + (double)S * M * w->rows * 4.0), push ? *push : QbGemmPush(),
                               swiglu ? *swiglu : QbGemmSwiglu()));
    if (grid_out) *grid_out = grid;
    QB_LAUNCHED(ctx, "gemm_tc_kernel");
    return QB_OK;
}

}  // namespace

bool qb_gemm_tc_supported(const qb_weight *w, uint32_t M) {
    return w->rec != nullptr && M >= 1 && w->cols % 128 == 0;
}

int qb_launch_gemm_tc(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part, uint32_t S,
                      const QbGemmPush *push, uint32_t *grid_out, const QbGemmSwiglu *swiglu) {
    QB_REQUIRE(!swiglu || (M <= 16 && S == 1 && w->rows % 128 == 0 && w->cols / 128 > 8 && swiglu->q && swiglu->d),
               "gemm: the fused SwiGLU needs M <= 16, one K segment, whole 128-row tiles and K > 1024");
    QB_REQUIRE(M > 0 && S > 0 && S <= w->cols / 128, "gemm: bad M=%u or ksplit=%u", M, S);
    QB_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)d & 15) == 0, "gemm: activation buffers must be 16-byte aligned");
    if (M <= 4) return launch_tc<16, 4>(ctx, w, q, d, M, part, S, push, grid_out, swiglu);
    if (M <= 8) return launch_tc<16, 8>(ctx, w, q, d, M, part, S, push, grid_out, swiglu);
    if (M <= 16) return launch_tc<16, 16>(ctx, w, q, d, M, part, S, push, grid_out, swiglu);
    if (M <= 32) return launch_tc<32, 32>(ctx, w, q, d, M, part, S, push, grid_out, swiglu);
    if (M <= 64) return launch_tc<64, 64>(ctx, w, q, d, M, part, S, push, grid_out, swiglu);
    return launch_tc<128, 128>(ctx, w, q, d, M, part, S, push, grid_out, swiglu);
}
