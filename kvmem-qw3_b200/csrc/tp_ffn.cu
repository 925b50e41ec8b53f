// Tensor-parallel FFN pair: gate/up sharded over the FFN dimension (column-parallel, no exchange, SwiGLU local),
// down sharded over the same dimension as its K (row-parallel), one all-reduce of the [M][n_out] result.
//
// The all-reduce is one-shot over peer memory and fused with the producing GEMM: the epilogue of the down GEMM
// stores every split partial straight into the receive area of every GPU of the group (its own included),
// fences system-wide and bumps an arrival counter on each of them; the reduce kernel of a GPU waits (bounded)
// until all CTAs of all ranks have arrived and adds, in rank order, each rank's sum over its segments, so every
// GPU gets the same bits.  With many rows the S-fold copy of the partials would make the exchange bandwidth
// bound; from QB_TP_FUSED_ROWS rows on, a rank therefore adds its own segments first and pushes one [M][n_out]
// slice (same order of additions, so the result does not depend on which form ran).  Receive areas are
// double-buffered by step parity: a rank can only be one step ahead of a peer, because its next reduce needs
// that peer's next push.
//
// Receive area of one GPU:  [0,256) arrival counters (parity p at byte 128*p), then for parity p
// slot[p] = float [world][S][max_rows][n_out] with S = qb_ksplit_policy(n_out, k_shard); a push of M rows
// uses the first S*M*n_out floats of its rank's region.
#include "qb_internal.h"

struct qb_tp_group {
    uint32_t rank = 0, world = 1, max_rows = 0, n_in = 0, f_shard = 0, n_out = 0, S_dn = 1;
    uint8_t *recv[8] = {};
    uint64_t expected[2] = {0, 0};
    uint32_t step = 0;
    int8_t *xq = nullptr, *hq = nullptr;
    float *xd = nullptr, *hd = nullptr, *gu_parts = nullptr;
    size_t region_floats = 0, slot_floats = 0;
    float *dn_parts = nullptr;           // local split partials of the down GEMM (many-row form)
    uint32_t pushed_S[2] = {1, 1};       // segments per rank in the slot of each parity
    uint32_t gu_ileave = 0;              // row order of the gate/up shard: 0 = [gate; up], 64 = interleaved in groups of 64 (the engine's)
};
void qb_tp_group_set_ileave(qb_tp_group *g, uint32_t ileave) { if (g) g->gu_ileave = ileave; }

namespace {

constexpr uint32_t QB_TP_FUSED_ROWS = 32;       // below: the GEMM epilogue pushes its split partials itself
constexpr uint32_t TP_WAIT_LIMIT = 1u << 20;     // polls of >= 1 us (a system-scope load + 256 ns sleep): a second or so

__global__ void tp_reduce_kernel(const float *__restrict__ slot, const unsigned int *counter, unsigned int expected,
                                 uint32_t world, uint32_t S, uint32_t M, uint32_t N, size_t region_floats, float *y,
                                 uint32_t y_stride, int *err_flag) {
    QB_PDL_ENTER();
    __shared__ int ok;
    if (threadIdx.x == 0) {
        unsigned int seen = 0;
        uint32_t it = 0;
        for (; it < TP_WAIT_LIMIT; ++it) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            if ((int)(seen - expected) >= 0) break;
            __nanosleep(256);
        }
        ok = it < TP_WAIT_LIMIT;
        if (!ok) atomicExch(err_flag, 2000);     // a peer never arrived: report and return, the context stays usable
    }
    __syncthreads();
    if (!ok) return;
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
    if (n >= N) return;
    float acc = 0.0f;
    for (uint32_t r = 0; r < world; ++r) {
        float mine = __ldcg(slot + r * region_floats + (size_t)m * N + n);
        for (uint32_t s = 1; s < S; ++s) mine += __ldcg(slot + r * region_floats + ((size_t)s * M + m) * N + n);
        acc = r == 0 ? mine : acc + mine;
    }
    y[(size_t)m * y_stride + n] = acc;
}

// Many-row form: this rank's sum over its segments goes to every rank's receive area as one slice.
__global__ void tp_local_reduce_push_kernel(const float *__restrict__ part, uint32_t S, uint32_t M, uint32_t N, QbGemmPush push) {
    QB_PDL_ENTER();
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
    if (n < N) {
        float v = part[(size_t)m * N + n];
        for (uint32_t s = 1; s < S; ++s) v += part[((size_t)s * M + m) * N + n];
        for (uint32_t p = 0; p < push.n; ++p) push.dst[p][(size_t)m * N + n] = v;
        __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (uint32_t p = 0; p < push.n; ++p) atomicAdd_system(push.counter[p], 1u);
    }
}

}  // namespace

extern "C" size_t qb_tp_recv_bytes(uint32_t world, uint32_t max_rows, uint32_t n_out, uint32_t k_shard) {
    const size_t region = (size_t)qb_ksplit(n_out, k_shard) * max_rows * n_out;
    return 256 + 2 * (size_t)world * region * sizeof(float);
}

extern "C" int qb_tp_group_create(qb_ctx *ctx, uint32_t rank, uint32_t world, void *const *recv_ptrs, uint32_t max_rows,
                                  uint32_t n_in, uint32_t f_shard, uint32_t n_out, qb_tp_group **out) {
    QB_REQUIRE(ctx && recv_ptrs && out, "qb_tp_group_create: null argument");
    QB_REQUIRE(world >= 1 && world <= 8 && rank < world, "qb_tp_group_create: rank %u of %u (at most 8 ranks)", rank, world);
    QB_REQUIRE(max_rows > 0 && n_in % 128 == 0 && f_shard % 128 == 0 && n_out % 32 == 0,
               "qb_tp_group_create: n_in %u and f_shard %u must be multiples of 128, n_out %u of 32", n_in, f_shard, n_out);
    auto *g = new qb_tp_group;
    g->rank = rank; g->world = world; g->max_rows = max_rows; g->n_in = n_in; g->f_shard = f_shard; g->n_out = n_out;
    g->S_dn = qb_ksplit(n_out, f_shard);
    g->region_floats = (size_t)g->S_dn * max_rows * n_out;
    g->slot_floats = (size_t)world * g->region_floats;
    for (uint32_t r = 0; r < world; ++r) {
        QB_REQUIRE(recv_ptrs[r] && ((uintptr_t)recv_ptrs[r] & 255) == 0, "qb_tp_group_create: receive area %u missing or not 256-byte aligned", r);
        g->recv[r] = (uint8_t *)recv_ptrs[r];
    }
    const uint32_t ld = qb_act_ld(max_rows), S_gu = qb_ksplit(2 * f_shard, n_in);
    QB_CUDA(cudaMalloc(&g->xq, (size_t)max_rows * n_in));
    QB_CUDA(cudaMalloc(&g->xd, (size_t)(n_in / 32) * ld * sizeof(float)));
    QB_CUDA(cudaMalloc(&g->hq, (size_t)max_rows * f_shard));
    QB_CUDA(cudaMalloc(&g->hd, (size_t)(f_shard / 32) * ld * sizeof(float)));
    QB_CUDA(cudaMalloc(&g->gu_parts, (size_t)S_gu * max_rows * 2 * f_shard * sizeof(float)));
    QB_CUDA(cudaMalloc(&g->dn_parts, g->region_floats * sizeof(float)));
    QB_CUDA(cudaMemsetAsync(g->recv[rank], 0, 256, ctx->stream));     // own arrival counters
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    *out = g;
    return QB_OK;
}

extern "C" int qb_tp_group_destroy(qb_ctx *ctx, qb_tp_group *g) {
    if (!g) return QB_OK;
    if (ctx) cudaStreamSynchronize(ctx->stream);
    cudaFree(g->xq); cudaFree(g->xd); cudaFree(g->hq); cudaFree(g->hd); cudaFree(g->gu_parts); cudaFree(g->dn_parts);
    delete g;
    return QB_OK;
}

// quantise x, gate/up shard GEMM, SwiGLU + quantise, down shard GEMM whose epilogue pushes to every rank.
extern "C" int qb_tp_ffn_push(qb_ctx *ctx, qb_tp_group *g, const qb_weight *gate_up, const qb_weight *down, const float *x_dev,
                              uint32_t M) {
    QB_REQUIRE(ctx && g && gate_up && down && x_dev, "qb_tp_ffn_push: null argument");
    QB_REQUIRE(M > 0 && M <= g->max_rows, "qb_tp_ffn_push: %u rows, group sized for %u", M, g->max_rows);
    QB_REQUIRE(gate_up->rows == 2 * g->f_shard && gate_up->cols == g->n_in && down->rows == g->n_out && down->cols == g->f_shard,
               "qb_tp_ffn_push: shard shapes [%u x %u], [%u x %u] do not match the group (n_in %u, f_shard %u, n_out %u)",
               gate_up->rows, gate_up->cols, down->rows, down->cols, g->n_in, g->f_shard, g->n_out);
    QB_REQUIRE(qb_gemm_tc_supported(down, M), "qb_tp_ffn_push: down shard not in the tensor-core record layout");
    const uint32_t ld = qb_act_ld(M);
    NormQuantArgs a;
    a.x = x_dev; a.x_stride = g->n_in; a.n = g->n_in; a.M = M;
    a.q = g->xq; a.q_pitch = g->n_in; a.d = g->xd; a.d_ld = ld;
    QB_TRY(qb_launch_norm_quant(ctx, a));
    const uint32_t S_gu = qb_ksplit(gate_up->rows, gate_up->cols);
    QB_TRY(qb_launch_gemm(ctx, gate_up, g->xq, g->xd, M, g->gu_parts, S_gu, 0));
    QB_TRY(qb_launch_swiglu_quant(ctx, g->gu_parts, 2 * g->f_shard, M, g->f_shard, g->hq, g->f_shard, g->hd, ld, S_gu,
                                  (size_t)M * 2 * g->f_shard, g->gu_ileave));
    const uint32_t par = g->step & 1;
    QbGemmPush push;
    push.n = g->world;
    for (uint32_t r = 0; r < g->world; ++r) {
        push.dst[r] = reinterpret_cast<float *>(g->recv[r] + 256) + par * g->slot_floats + g->rank * g->region_floats;
        push.counter[r] = reinterpret_cast<unsigned int *>(g->recv[r] + 128 * par);
    }
    uint32_t grid = 0;
    if (M < QB_TP_FUSED_ROWS || g->S_dn == 1) {
        QB_TRY(qb_launch_gemm_tc(ctx, down, g->hq, g->hd, M, nullptr, g->S_dn, &push, &grid));
        g->pushed_S[par] = g->S_dn;
    } else {
        QB_TRY(qb_launch_gemm_tc(ctx, down, g->hq, g->hd, M, g->dn_parts, g->S_dn));
        dim3 rg((g->n_out + 255) / 256, M);
        QB_CUDA(qb_launch_pdl(ctx->stream, tp_local_reduce_push_kernel, rg, dim3(256), (size_t)0, (const float *)g->dn_parts, g->S_dn, M,
                              g->n_out, push));
        QB_LAUNCHED(ctx, "tp_local_reduce_push_kernel");
        grid = rg.x * rg.y;
        g->pushed_S[par] = 1;
    }
    g->expected[par] += (uint64_t)g->world * grid;       // every rank launches the same grid for the same M
    return QB_OK;
}

// y[m][n] = sum over ranks (ascending) of each rank's sum over its segments (ascending).
extern "C" int qb_tp_ffn_reduce(qb_ctx *ctx, qb_tp_group *g, uint32_t M, float *y_dev, uint32_t y_stride) {
    QB_REQUIRE(ctx && g && y_dev && M > 0 && M <= g->max_rows && y_stride >= g->n_out, "qb_tp_ffn_reduce: bad arguments");
    const uint32_t par = g->step & 1;
    const float *slot = reinterpret_cast<const float *>(g->recv[g->rank] + 256) + par * g->slot_floats;
    const unsigned int *counter = reinterpret_cast<const unsigned int *>(g->recv[g->rank] + 128 * par);
    dim3 grid((g->n_out + 255) / 256, M);
    QB_CUDA(qb_launch_pdl(ctx->stream, tp_reduce_kernel, grid, dim3(256), (size_t)0, slot, counter, (unsigned int)g->expected[par], g->world,
                          g->pushed_S[par], M, g->n_out, g->region_floats, y_dev, y_stride, ctx->err_flag_dev));
    QB_LAUNCHED(ctx, "tp_reduce_kernel");
    g->step += 1;
    return QB_OK;
}

extern "C" int qb_tp_ffn(qb_ctx *ctx, qb_tp_group *g, const qb_weight *gate_up, const qb_weight *down, const float *x_dev, uint32_t M,
                         float *y_dev, uint32_t y_stride) {
    QB_TRY(qb_tp_ffn_push(ctx, g, gate_up, down, x_dev, M));
    return qb_tp_ffn_reduce(ctx, g, M, y_dev, y_stride);
}

// ---- CUDA IPC helpers: how the ranks (one process per GPU) learn each other's receive areas ---------------
extern "C" int qb_ipc_export(qb_ctx *ctx, const void *dev_ptr, void *handle64) {
    QB_REQUIRE(ctx && dev_ptr && handle64, "qb_ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    QB_CUDA(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(handle64), const_cast<void *>(dev_ptr)));
    return QB_OK;
}

extern "C" int qb_ipc_open(qb_ctx *ctx, const void *handle64, void **dev_ptr_out) {
    QB_REQUIRE(ctx && handle64 && dev_ptr_out, "qb_ipc_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    QB_CUDA(cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
    return QB_OK;
}

extern "C" int qb_ipc_close(qb_ctx *ctx, void *dev_ptr) {
    QB_REQUIRE(ctx && dev_ptr, "qb_ipc_close: null argument");
    QB_CUDA(cudaIpcCloseMemHandle(dev_ptr));
    return QB_OK;
}
