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
// in order.  Weight bytes, activation bytes and both scale planes arrive by TMA (128-byte swizzle for
// the MMA operands) through an mbarrier pipeline; the kernel is an HBM streaming kernel until the
// activation-row count reaches the hundreds.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (owns the TMEM allocation),
// warps 2..5 = epilogue (TMEM lane quarter = warp % 4).  Every wait is bounded: when a wait runs out
// the CTA raises the context's error flag, lets its copies land, frees its TMEM and returns.
#include "qb_internal.h"

namespace {

constexpr int TC_THREADS = 192;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait; returns false when the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] = A[smem] * B[smem], int8 x int8 -> int32, no accumulation into D.
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}

// K-major operand tile with 128-byte rows and the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = (uint64_t)((addr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;                  // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;       // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                  // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                  // SWIZZLE_128B
    return d;
}

template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, int32_t *r);
template <>
__device__ __forceinline__ void tmem_ld<4>(uint32_t taddr, int32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<8>(uint32_t taddr, int32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, int32_t *r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__host__ __device__ inline uint32_t tc_seg_begin(uint32_t s, uint32_t S, uint32_t nchunks) {
    return (uint32_t)(((uint64_t)s * nchunks) / S);
}

// MT = activation rows per tile (MMA N).  NLD = accumulator columns the epilogue reads (<= MT).
template <int MT, int NLD>
struct TcCfg {
    static constexpr int KPS = MT == 128 ? 2 : 4;              // 32-blocks per TMEM slot
    static constexpr int SPS = 4 / KPS;                        // slots per pipeline stage
    static constexpr int NSLOT = 512 / (KPS * MT);
    static constexpr int NST = MT <= 32 ? 8 : (MT == 64 ? 6 : 5);
    static constexpr int A_BYTES = 128 * 128;
    static constexpr int B_BYTES = MT * 128;
    static constexpr int WD_BYTES = 4 * 128 * 2;
    static constexpr int XD_BYTES = 4 * MT * 4;
    static constexpr int TX_BYTES = A_BYTES + B_BYTES + WD_BYTES + XD_BYTES;
    static constexpr int STAGE = (TX_BYTES + 1023) / 1024 * 1024;
    static constexpr int BAR_BYTES = 1024;
    static constexpr int TOTAL = STAGE * NST + BAR_BYTES + 1024;   // + slack to align the base to 1024
    static constexpr int CH = NLD < 16 ? NLD : 16;               // columns per tcgen05.ld
};

template <int MT, int NLD>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_wq, const __grid_constant__ CUtensorMap map_wd,
               const __grid_constant__ CUtensorMap map_xq, const __grid_constant__ CUtensorMap map_xd,
               uint32_t K, uint32_t N, uint32_t M, float *__restrict__ part, uint32_t S, int *err_flag) {
    using C = TcCfg<MT, NLD>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *bar_mem = smem + (size_t)C::STAGE * C::NST;
    uint64_t *bars = reinterpret_cast<uint64_t *>(bar_mem);
    // barrier layout: full[NST], empty[NST], tmem_full[NSLOT], tmem_empty[NSLOT]
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * C::NST;
    const uint32_t bar_tfull = bar_empty + 8 * C::NST, bar_tempty = bar_tfull + 8 * C::NSLOT;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_mem + 8 * (2 * C::NST + 2 * C::NSLOT));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row0 = blockIdx.x * 128, seg = blockIdx.y, m0 = blockIdx.z * MT;
    const uint32_t nchunks = K / 128;
    const uint32_t c_begin = tc_seg_begin(seg, S, nchunks), n_it = tc_seg_begin(seg + 1, S, nchunks) - c_begin;

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::NST; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1 + 128);        // MMA commit + every epilogue thread
        }
        for (int i = 0; i < C::NSLOT; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 128);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (uint32_t it = 0; it < n_it; ++it) {
                const uint32_t st = it % C::NST, ph = (it / C::NST) & 1;
                if (!mbar_wait(bar_empty + 8 * st, ph ^ 1, abort_flag)) break;
                const uint32_t base = smem_u32(smem + (size_t)st * C::STAGE);
                const uint32_t full = bar_full + 8 * st;
                mbar_expect_tx(full, C::TX_BYTES);
                const int k0 = (int)((c_begin + it) * 128);
                tma_load_2d(base, &map_wq, k0, (int)row0, full);
                tma_load_2d(base + C::A_BYTES, &map_xq, k0, (int)m0, full);
                tma_load_2d(base + C::A_BYTES + C::B_BYTES, &map_wd, (int)row0, k0 / 32, full);
                tma_load_2d(base + C::A_BYTES + C::B_BYTES + C::WD_BYTES, &map_xd, (int)m0, k0 / 32, full);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N = MT, M = 128
            constexpr uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MT >> 3) << 17) | ((128u >> 4) << 24);
            uint32_t j = 0;
            bool ok = true;
            for (uint32_t it = 0; it < n_it && ok; ++it) {
                const uint32_t st = it % C::NST, ph = (it / C::NST) & 1;
                if (!mbar_wait(bar_full + 8 * st, ph, abort_flag)) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + (size_t)st * C::STAGE), b_addr = a_addr + C::A_BYTES;
                for (int sp = 0; sp < C::SPS; ++sp, ++j) {
                    const uint32_t slot = j % C::NSLOT, sph = (j / C::NSLOT) & 1;
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
    } else {
        const uint32_t quarter = warp & 3;                     // TMEM lanes [32*quarter, +32)
        const uint32_t r = quarter * 32 + lane;                // weight row inside the tile
        float acc[NLD];
#pragma unroll
        for (int i = 0; i < NLD; ++i) acc[i] = 0.0f;
        uint32_t j = 0;
        bool ok = true;
        for (uint32_t it = 0; it < n_it && ok; ++it) {
            const uint32_t st = it % C::NST, ph = (it / C::NST) & 1;
            if (!mbar_wait(bar_full + 8 * st, ph, abort_flag)) break;
            const uint8_t *stage = smem + (size_t)st * C::STAGE;
            const __half *wd = reinterpret_cast<const __half *>(stage + C::A_BYTES + C::B_BYTES);
            const float *xd = reinterpret_cast<const float *>(stage + C::A_BYTES + C::B_BYTES + C::WD_BYTES);
            for (int sp = 0; sp < C::SPS; ++sp, ++j) {
                const uint32_t slot = j % C::NSLOT, sph = (j / C::NSLOT) & 1;
                if (!mbar_wait(bar_tfull + 8 * slot, sph, abort_flag)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kl = 0; kl < C::KPS; ++kl) {
                    const int kb = sp * C::KPS + kl;
                    const float dw = __half2float(wd[kb * 128 + r]);
                    const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + slot * (C::KPS * MT) + kl * MT;
#pragma unroll
                    for (int c0 = 0; c0 < NLD; c0 += C::CH) {
                        int32_t v[C::CH];
                        tmem_ld<C::CH>(taddr + c0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < C::CH; ++i)
                            acc[c0 + i] = __fmaf_rn(__fmul_rn(dw, xd[kb * MT + c0 + i]), (float)v[i], acc[c0 + i]);
                    }
                }
                tc_fence_before();
                mbar_arrive(bar_tempty + 8 * slot);
            }
            if (ok) mbar_arrive(bar_empty + 8 * st);
        }
        const uint32_t row = row0 + r;
        if (ok && !*abort_flag && row < N) {
#pragma unroll
            for (int i = 0; i < NLD; ++i) {
                const uint32_t m = m0 + i;
                if (m < M) part[((size_t)seg * M + m) * N + row] = acc[i];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(err_flag, 1000 + (int)(blockIdx.x % 1000));
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);      // let this CTA's copies in flight land
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

struct MapKey {
    const void *p; uint32_t a, b, c;
    bool operator<(const MapKey &o) const { return std::tie(p, a, b, c) < std::tie(o.p, o.a, o.b, o.c); }
};
std::map<MapKey, CUtensorMap> g_xq_maps, g_xd_maps;

template <int MT, int NLD>
int launch_tc(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part, uint32_t S) {
    using C = TcCfg<MT, NLD>;
    static bool attr = false;
    if (!attr) {
        QB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<MT, NLD>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
        attr = true;
    }
    const uint32_t K = w->cols, ld = qb_act_ld(M);
    MapKey kq{q, M, K, (uint32_t)MT}, kd{d, M, K, (uint32_t)MT};
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
    dim3 grid(w->rows_pad / 128, S, (M + MT - 1) / MT);
    gemm_tc_kernel<MT, NLD><<<grid, TC_THREADS, C::TOTAL, ctx->stream>>>(w->map_q, w->map_d, iq->second, id->second, K, w->rows, M,
                                                                        part, S, ctx->err_flag_dev);
    QB_LAUNCHED(ctx, "gemm_tc_kernel");
    return QB_OK;
}

}  // namespace

bool qb_gemm_tc_supported(const qb_weight *w, uint32_t M) {
    return w->has_maps && M >= 1 && w->cols % 128 == 0;
}

int qb_launch_gemm_tc(qb_ctx *ctx, const qb_weight *w, const int8_t *q, const float *d, uint32_t M, float *part, uint32_t S) {
    QB_REQUIRE(M > 0 && S > 0 && S <= w->cols / 128, "gemm: bad M=%u or ksplit=%u", M, S);
    QB_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)d & 15) == 0, "gemm: activation buffers must be 16-byte aligned");
    if (M <= 4) return launch_tc<16, 4>(ctx, w, q, d, M, part, S);
    if (M <= 8) return launch_tc<16, 8>(ctx, w, q, d, M, part, S);
    if (M <= 16) return launch_tc<16, 16>(ctx, w, q, d, M, part, S);
    if (M <= 32) return launch_tc<32, 32>(ctx, w, q, d, M, part, S);
    if (M <= 64) return launch_tc<64, 64>(ctx, w, q, d, M, part, S);
    return launch_tc<128, 128>(ctx, w, q, d, M, part, S);
}
