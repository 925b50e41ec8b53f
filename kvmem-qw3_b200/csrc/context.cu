// Context, memory, events and TMA tensor-map encoding of libqw3b200.
#include "qb_internal.h"
#include "page_pool.h"

#include <cudaTypedefs.h>

static thread_local char g_err[512] = "";

int qb_fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

extern "C" const char *qb_last_error(void) { return g_err; }

extern "C" int qb_create(int device, qb_ctx **out) {
    QB_REQUIRE(out != nullptr, "qb_create: out is null");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return qb_fail(QB_ERR_CUDA, "qb_create: no CUDA device (%s); this library has no CPU path",
                       cudaGetErrorString(e));
    QB_REQUIRE(device >= 0 && device < count, "qb_create: device %d out of range (%d devices)", device, count);
    QB_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    QB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return qb_fail(QB_ERR_UNSUPPORTED, "qb_create: device is sm_%d%d, this library is built for sm_100a only",
                       prop.major, prop.minor);
    qb_ctx *ctx = new qb_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    QB_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
    std::vector<float> table(QS_NORMAL_TABLE_SIZE);
    qs_build_normal_table(table.data());
    QB_CUDA(cudaMalloc(&ctx->normal_table_dev, table.size() * sizeof(float)));
    QB_CUDA(cudaMemcpy(ctx->normal_table_dev, table.data(), table.size() * sizeof(float), cudaMemcpyHostToDevice));
    QB_CUDA(cudaMalloc(&ctx->err_flag_dev, sizeof(int)));
    QB_CUDA(cudaMemset(ctx->err_flag_dev, 0, sizeof(int)));
    *out = ctx;
    return QB_OK;
}

extern "C" void qb_destroy(qb_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->normal_table_dev) cudaFree(ctx->normal_table_dev);
    if (ctx->flush_buf) cudaFree(ctx->flush_buf);
    if (ctx->err_flag_dev) cudaFree(ctx->err_flag_dev);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->scratch2) cudaFree(ctx->scratch2);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

extern "C" int qb_synchronize(qb_ctx *ctx) {
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    int flag = 0;
    QB_CUDA(cudaMemcpy(&flag, ctx->err_flag_dev, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag != 0) {
        cudaMemset(ctx->err_flag_dev, 0, sizeof(int));
        return qb_fail(QB_ERR_CUDA, "a kernel recorded an error (code %d: 3001 / 3002 = a K/V append to an unassigned page, skipped; other codes = a bounded wait that ran out)", flag);
    }
    return QB_OK;
}

extern "C" void *qb_stream(qb_ctx *ctx) { return (void *)ctx->stream; }
extern "C" int qb_sm_count(qb_ctx *ctx) { return ctx->sm_count; }
extern "C" int64_t qb_launch_count(qb_ctx *ctx) { return ctx->launches; }

int qb_ctx_scratch(qb_ctx *ctx, size_t bytes, void **out) {
    if (bytes > ctx->scratch_bytes) {
        QB_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->scratch) QB_CUDA(cudaFree(ctx->scratch));
        ctx->scratch = nullptr;
        ctx->scratch_bytes = 0;
        const size_t want = bytes + (bytes >> 2) + (1u << 20);
        QB_CUDA(cudaMalloc(&ctx->scratch, want));
        ctx->scratch_bytes = want;
    }
    *out = ctx->scratch;
    return QB_OK;
}

int qb_ctx_scratch2(qb_ctx *ctx, size_t bytes, void **out) {
    if (bytes > ctx->scratch2_bytes) {
        QB_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->scratch2) QB_CUDA(cudaFree(ctx->scratch2));
        ctx->scratch2 = nullptr;
        ctx->scratch2_bytes = 0;
        const size_t want = bytes + (bytes >> 2) + (1u << 20);
        QB_CUDA(cudaMalloc(&ctx->scratch2, want));
        ctx->scratch2_bytes = want;
    }
    *out = ctx->scratch2;
    return QB_OK;
}

extern "C" int qb_mem_info(qb_ctx *ctx, size_t *free_bytes, size_t *total_bytes) {
    QB_REQUIRE(ctx, "qb_mem_info: null context");
    QB_CUDA(cudaSetDevice(ctx->device));
    size_t f = 0, t = 0;
    QB_CUDA(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return QB_OK;
}

extern "C" int qb_malloc(qb_ctx *ctx, size_t bytes, void **dev_ptr) {
    QB_CUDA(cudaSetDevice(ctx->device));
    QB_CUDA(cudaMalloc(dev_ptr, bytes ? bytes : 16));
    return QB_OK;
}
extern "C" int qb_free(qb_ctx *ctx, void *dev_ptr) {
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    QB_CUDA(cudaFree(dev_ptr));
    return QB_OK;
}
extern "C" int qb_memcpy_h2d(qb_ctx *ctx, void *dst, const void *src, size_t bytes) {
    QB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    return QB_OK;
}
extern "C" int qb_memcpy_d2h(qb_ctx *ctx, void *dst, const void *src, size_t bytes) {
    QB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    return QB_OK;
}
extern "C" int qb_memcpy_d2d(qb_ctx *ctx, void *dst, const void *src, size_t bytes) {
    QB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return QB_OK;
}
extern "C" int qb_memset(qb_ctx *ctx, void *p, int value, size_t bytes) {
    QB_CUDA(cudaMemsetAsync(p, value, bytes, ctx->stream));
    return QB_OK;
}
extern "C" int qb_host_alloc(qb_ctx *ctx, size_t bytes, void **host_ptr) {
    (void)ctx;
    QB_CUDA(cudaHostAlloc(host_ptr, bytes, cudaHostAllocDefault));
    return QB_OK;
}
extern "C" int qb_host_free(qb_ctx *ctx, void *host_ptr) {
    (void)ctx;
    QB_CUDA(cudaFreeHost(host_ptr));
    return QB_OK;
}

extern "C" int qb_event_create(qb_ctx *ctx, void **event) {
    (void)ctx;
    cudaEvent_t ev;
    QB_CUDA(cudaEventCreate(&ev));
    *event = (void *)ev;
    return QB_OK;
}
extern "C" int qb_event_record(qb_ctx *ctx, void *event) {
    QB_CUDA(cudaEventRecord((cudaEvent_t)event, ctx->stream));
    return QB_OK;
}
extern "C" int qb_event_elapsed_ms(qb_ctx *ctx, void *start, void *stop, float *ms) {
    (void)ctx;
    QB_CUDA(cudaEventSynchronize((cudaEvent_t)stop));
    QB_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return QB_OK;
}
extern "C" int qb_event_destroy(qb_ctx *ctx, void *event) {
    (void)ctx;
    QB_CUDA(cudaEventDestroy((cudaEvent_t)event));
    return QB_OK;
}

extern "C" int qb_flush_l2(qb_ctx *ctx) {
    if (!ctx->flush_buf) {
        ctx->flush_bytes = (size_t)256 << 20;   // 2x the 126 MB L2
        QB_CUDA(cudaMalloc(&ctx->flush_buf, ctx->flush_bytes));
    }
    QB_CUDA(cudaMemsetAsync(ctx->flush_buf, 0x5a, ctx->flush_bytes, ctx->stream));
    return QB_OK;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
int qb_make_tmap_2d(CUtensorMap *map, CUtensorMapDataType dt, uint32_t elem_bytes, const void *base,
                    uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner,
                    uint32_t box_outer, CUtensorMapSwizzle swz) {
    static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        QB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !fn)
            return qb_fail(QB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
        encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    }
    QB_REQUIRE(((uintptr_t)base & 15) == 0, "tensor map base not 16-byte aligned");
    QB_REQUIRE((pitch_bytes & 15) == 0, "tensor map pitch %llu not a multiple of 16", (unsigned long long)pitch_bytes);
    QB_REQUIRE(((uint64_t)box_inner * elem_bytes) % 16 == 0, "tensor map box inner extent not a multiple of 16 bytes");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return qb_fail(QB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    (void)elem_bytes;
    return QB_OK;
}

// ---- launch trace: an event after every kernel launch; the time between consecutive events is the
// duration of the kernel launched in between (kernels of one stream run back to back) ----------------
void qb_trace_mark(qb_ctx *ctx, const char *name) {
    if (ctx->trace_used >= ctx->trace_ev.size()) {
        for (int i = 0; i < 1024; ++i) {
            cudaEvent_t e;
            if (cudaEventCreate(&e) != cudaSuccess) return;
            ctx->trace_ev.push_back(e);
        }
    }
    cudaEventRecord(ctx->trace_ev[ctx->trace_used++], ctx->stream);
    ctx->trace_names.push_back(name);
}

// ---- device timeline of the tensor-core GEMM launches ------------------------------------------
unsigned long long *qb_timeline_slot(qb_ctx *ctx, uint32_t grid, double bytes) {
    if (!ctx->tl_dev || ctx->tl_used >= ctx->tl_cap || grid > QB_TL_CTAS) return nullptr;
    ctx->tl_grid.push_back(grid);
    ctx->tl_bytes.push_back(bytes);
    return ctx->tl_dev + (size_t)(ctx->tl_used++) * QB_TL_CTAS * 4;
}

extern "C" int qb_debug_timeline_enable(qb_ctx *ctx, uint32_t max_launches) {
    QB_REQUIRE(ctx, "qb_debug_timeline_enable: null context");
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->tl_dev) { cudaFree(ctx->tl_dev); ctx->tl_dev = nullptr; }
    ctx->tl_cap = ctx->tl_used = 0;
    ctx->tl_grid.clear();
    ctx->tl_bytes.clear();
    if (max_launches) {
        const size_t bytes = (size_t)max_launches * QB_TL_CTAS * 4 * sizeof(unsigned long long);
        QB_CUDA(cudaMalloc(&ctx->tl_dev, bytes));
        QB_CUDA(cudaMemset(ctx->tl_dev, 0, bytes));
        ctx->tl_cap = max_launches;
    }
    return QB_OK;
}

extern "C" int qb_debug_timeline_read(qb_ctx *ctx, uint64_t *out, uint32_t *grids, double *bytes, uint32_t max_launches,
                                      uint32_t *n_out) {
    QB_REQUIRE(ctx && out && grids && bytes && n_out, "qb_debug_timeline_read: null argument");
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    const uint32_t n = std::min(max_launches, ctx->tl_used);
    if (n) QB_CUDA(cudaMemcpy(out, ctx->tl_dev, (size_t)n * QB_TL_CTAS * 4 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    for (uint32_t i = 0; i < n; ++i) { grids[i] = ctx->tl_grid[i]; bytes[i] = ctx->tl_bytes[i]; }
    *n_out = n;
    return QB_OK;
}

extern "C" int qb_trace_enable(qb_ctx *ctx, int on) {
    ctx->trace_on = false;
    ctx->trace_used = 0;
    ctx->trace_names.clear();
    if (on) {
        qb_trace_mark(ctx, "(start)");
        ctx->trace_on = true;
    }
    return QB_OK;
}

// Writes "name\tlaunches\ttotal_us" lines (sorted by launch order of first appearance) into buf.
extern "C" int qb_trace_summary(qb_ctx *ctx, char *buf, size_t buf_bytes) {
    QB_CUDA(cudaStreamSynchronize(ctx->stream));
    std::vector<std::pair<const char *, std::pair<long, double>>> agg;
    for (size_t i = 1; i < ctx->trace_used; ++i) {
        float ms = 0.0f;
        QB_CUDA(cudaEventElapsedTime(&ms, ctx->trace_ev[i - 1], ctx->trace_ev[i]));
        const char *n = ctx->trace_names[i];
        size_t k = 0;
        for (; k < agg.size(); ++k) if (strcmp(agg[k].first, n) == 0) break;
        if (k == agg.size()) agg.push_back({n, {0, 0.0}});
        agg[k].second.first += 1;
        agg[k].second.second += ms * 1e3;
    }
    size_t off = 0;
    for (auto &a : agg) {
        int w = snprintf(buf + off, off < buf_bytes ? buf_bytes - off : 0, "%s\t%ld\t%.2f\n", a.first, a.second.first, a.second.second);
        if (w < 0 || off + (size_t)w >= buf_bytes) break;
        off += (size_t)w;
    }
    if (buf_bytes) buf[std::min(off, buf_bytes - 1)] = 0;
    return QB_OK;
}

// ---- the page pool on its own (host side only; no device needed) -----------------------------------------------------
// For a caller that keeps its own page tables over the op-level entry points (qb_kv_append / qb_attention_paged take
// page indices): the allocator the pooled batches use, GlobalKvPagePool's role (src/qwen_native_backend.cpp:1155-1265).
extern "C" void *qb_page_pool_create(uint32_t total_pages) { return total_pages ? new QbPagePool(total_pages) : nullptr; }
extern "C" void qb_page_pool_destroy(void *pool) { delete (QbPagePool *)pool; }
extern "C" int32_t qb_page_pool_alloc(void *pool) { return pool ? ((QbPagePool *)pool)->alloc() : -1; }
extern "C" int32_t qb_page_pool_share(void *pool, int32_t page) { return pool && ((QbPagePool *)pool)->share(page) ? 1 : 0; }
extern "C" int32_t qb_page_pool_drop(void *pool, int32_t page) { return pool ? ((QbPagePool *)pool)->drop(page) : -1; }
extern "C" uint32_t qb_page_pool_free_count(void *pool) { return pool ? ((QbPagePool *)pool)->free_count() : 0; }
