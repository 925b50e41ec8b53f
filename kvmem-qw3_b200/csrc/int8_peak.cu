// Measured INT8 tensor-core peak: the denominator for any "fraction of the INT8 peak" statement.
//
// One CTA per SM issues tcgen05.mma.kind::i8 (M = 128, N = 256, K = 32) back to back on operand tiles that stay
// in shared memory, alternating between two accumulator halves of tensor memory; nothing is loaded or drained in
// the loop, so the time is the tensor pipe's.  ops = 2 * 128 * 256 * 32 per instruction.
#include "qb_internal.h"

namespace {

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr) {   // K-major, 128-byte rows, 128-byte swizzle
    uint64_t d = (uint64_t)((addr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__global__ void __launch_bounds__(128) int8_peak_kernel(uint32_t iters, int *err_flag) {
    extern __shared__ uint8_t raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    uint8_t *a_tile = smem, *b_tile = smem + 16384;                 // 128 x 128 B and 256 x 128 B
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    for (uint32_t i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem)[i] = 0x01010101u;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_addr(&tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    bool ok = true;
    if (threadIdx.x == 0) {
        // instruction descriptor: D = s32, A = B = signed 8-bit, K-major, N = 256, M = 128
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
        const uint64_t a0 = desc_sw128(smem_addr(a_tile)), b0 = desc_sw128(smem_addr(b_tile));
        for (uint32_t it = 0; it < iters; ++it) {
#pragma unroll
            for (uint32_t kb = 0; kb < 4; ++kb) {
                const uint32_t acc = kb ? 1u : 0u;                      // first K block of an iteration overwrites
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                    ::"r"(tmem + (it & 1) * 256), "l"(a0 + (uint64_t)(kb * 2)), "l"(b0 + (uint64_t)(kb * 2)), "r"(idesc), "r"(acc),
                      "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
            }
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(&bar)) : "memory");
        uint32_t done = 0;
        for (uint32_t i = 0; i < (1u << 26) && !done; ++i)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(smem_addr(&bar)) : "memory");
        if (!done) { atomicExch(err_flag, 3000); ok = false; }
    }
    (void)ok;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
}

}  // namespace

// Runs the peak kernel (iters x 4 instructions per SM) and returns tera-ops per second (2 ops per multiply-add).
extern "C" int qb_debug_int8_mma_peak(qb_ctx *ctx, uint32_t iters, double *tops_out) {
    QB_REQUIRE(ctx && tops_out && iters > 0, "qb_debug_int8_mma_peak: bad arguments");
    const size_t smem = 16384 + 32768 + 1024;
    QB_CUDA(cudaFuncSetAttribute(int8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaEvent_t e0, e1;
    QB_CUDA(cudaEventCreate(&e0));
    QB_CUDA(cudaEventCreate(&e1));
    int8_peak_kernel<<<ctx->sm_count, 128, smem, ctx->stream>>>(iters / 8 + 1, ctx->err_flag_dev);      // warm-up
    QB_CUDA(cudaEventRecord(e0, ctx->stream));
    int8_peak_kernel<<<ctx->sm_count, 128, smem, ctx->stream>>>(iters, ctx->err_flag_dev);
    QB_CUDA(cudaEventRecord(e1, ctx->stream));
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    QB_LAUNCHED(ctx, "int8_peak_kernel");
    float ms = 0.0f;
    QB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *tops_out = 2.0 * 128 * 256 * 32 * 4.0 * iters * ctx->sm_count / (ms * 1e-3) / 1e12;
    return QB_OK;
}
