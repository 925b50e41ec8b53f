// Q8_0 weights in device layout: upload + repack, seeded on-device generation, download, views.
//
// Replaces the CudaWeight Q8_0 constructor of the reference (src/kernels_cuda.cu:1566-1594), which
// repacks GGUF's interleaved 34-byte blocks into per-row [scales | quants].  Here the quants form
// one int8 matrix [rows_pad][cols] (a legal TMA tensor: every row pitch is a multiple of 16 bytes)
// and the scales one fp16 matrix [cols/32][rows_pad] (scales of 128 consecutive rows are
// contiguous, which is what a thread-per-row epilogue reads).  34 bytes per 32 weights, as on disk.
#include "qb_internal.h"

static int make_maps(qb_weight *w) {
    QB_TRY(qb_make_tmap_2d(&w->map_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->q, w->cols, w->rows_pad, w->cols, 128, 128,
                           CU_TENSOR_MAP_SWIZZLE_128B));
    QB_TRY(qb_make_tmap_2d(&w->map_d, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, w->d, w->rows_pad, w->cols / 32,
                           (uint64_t)w->ld * 2, 128, 4, CU_TENSOR_MAP_SWIZZLE_NONE));
    w->has_maps = true;
    return QB_OK;
}

int qb_weight_alloc(qb_ctx *ctx, uint32_t rows, uint32_t cols, qb_weight **out) {
    QB_REQUIRE(rows > 0 && cols > 0 && cols % 128 == 0, "Q8_0 weight: cols=%u must be a positive multiple of 128", cols);
    qb_weight *w = new qb_weight();
    w->rows = rows;
    w->cols = cols;
    w->rows_pad = (rows + 127u) & ~127u;
    w->ld = w->rows_pad;
    w->owns = true;
    QB_CUDA(cudaSetDevice(ctx->device));
    const size_t qbytes = (size_t)w->rows_pad * cols, dbytes = (size_t)(cols / 32) * w->ld * sizeof(__half);
    QB_CUDA(cudaMalloc(&w->q, qbytes));
    QB_CUDA(cudaMalloc(&w->d, dbytes));
    if (w->rows_pad != rows) {
        QB_CUDA(cudaMemsetAsync(w->q, 0, qbytes, ctx->stream));
        QB_CUDA(cudaMemsetAsync(w->d, 0, dbytes, ctx->stream));
    }
    QB_TRY(make_maps(w));
    *out = w;
    return QB_OK;
}

int qb_weight_view(qb_ctx *ctx, const qb_weight *w, uint32_t row_off, uint32_t rows, qb_weight *out) {
    (void)ctx;
    QB_REQUIRE(row_off % 128 == 0 && row_off + rows <= w->rows_pad, "weight view [%u,+%u) not tile aligned / in range",
               row_off, rows);
    *out = qb_weight();
    out->rows = rows;
    out->cols = w->cols;
    out->rows_pad = (rows + 127u) & ~127u;
    QB_REQUIRE(row_off + out->rows_pad <= w->rows_pad, "weight view padding exceeds the parent");
    out->ld = w->ld;
    out->q = w->q + (size_t)row_off * w->cols;
    out->d = w->d + row_off;
    out->owns = false;
    return make_maps(out);
}

extern "C" void qb_weight_free(qb_ctx *ctx, qb_weight *w) {
    if (!w) return;
    if (w->owns) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(w->q);
        cudaFree(w->d);
    }
    delete w;
}
extern "C" uint32_t qb_weight_rows(const qb_weight *w) { return w->rows; }
extern "C" uint32_t qb_weight_cols(const qb_weight *w) { return w->cols; }

// One thread per 32-block.
__global__ void q8_synth_kernel(int8_t *q, __half *d, uint32_t ld, uint32_t cols, uint32_t row_off, uint32_t rows,
                                const float *__restrict__ table, uint64_t seed, uint32_t tensor_id, float sigma) {
    const uint32_t nb = cols / 32;
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (uint64_t)rows * nb) return;
    const uint32_t row = (uint32_t)(b / nb), kb = (uint32_t)(b % nb);
    uint16_t dbits;
    __align__(16) int8_t qq[32];
    qs_synth_q8_0_block(table, seed, tensor_id, b, sigma, &dbits, qq);
    int4 *dst = reinterpret_cast<int4 *>(q + (size_t)(row_off + row) * cols + (size_t)kb * 32);
    dst[0] = reinterpret_cast<const int4 *>(qq)[0];
    dst[1] = reinterpret_cast<const int4 *>(qq)[1];
    reinterpret_cast<uint16_t *>(d)[(size_t)kb * ld + row_off + row] = dbits;
}

int qb_weight_fill_synth(qb_ctx *ctx, qb_weight *w, uint32_t row_off, uint32_t rows, uint64_t seed,
                         uint32_t tensor_id, float sigma) {
    QB_REQUIRE(row_off + rows <= w->rows_pad, "synth fill out of range");
    const uint64_t nblocks = (uint64_t)rows * (w->cols / 32);
    const uint32_t threads = 128;
    const uint64_t grid = (nblocks + threads - 1) / threads;
    QB_REQUIRE(grid < (1ull << 31), "synth fill too large");
    q8_synth_kernel<<<(uint32_t)grid, threads, 0, ctx->stream>>>(w->q, w->d, w->ld, w->cols, row_off, rows,
                                                                ctx->normal_table_dev, seed, tensor_id, sigma);
    QB_LAUNCHED(ctx, "q8_synth_kernel");
    return QB_OK;
}

// GGUF blocks (34 B, row-major block order) of `rows` rows -> device layout at row_off.
__global__ void q8_repack_kernel(int8_t *q, __half *d, uint32_t ld, uint32_t cols, uint32_t row_off, uint32_t rows,
                                 const uint8_t *__restrict__ blocks) {
    const uint32_t nb = cols / 32;
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (uint64_t)rows * nb) return;
    const uint32_t row = (uint32_t)(b / nb), kb = (uint32_t)(b % nb);
    const uint16_t *src = reinterpret_cast<const uint16_t *>(blocks + b * 34);   // 2-byte aligned
    reinterpret_cast<uint16_t *>(d)[(size_t)kb * ld + row_off + row] = src[0];
    uint16_t *dst = reinterpret_cast<uint16_t *>(q + (size_t)(row_off + row) * cols + (size_t)kb * 32);
#pragma unroll
    for (int i = 0; i < 16; ++i) dst[i] = src[1 + i];
}

__global__ void q8_unpack_kernel(const int8_t *q, const __half *d, uint32_t ld, uint32_t cols, uint32_t row_off,
                                 uint32_t rows, uint8_t *blocks) {
    const uint32_t nb = cols / 32;
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (uint64_t)rows * nb) return;
    const uint32_t row = (uint32_t)(b / nb), kb = (uint32_t)(b % nb);
    uint16_t *dst = reinterpret_cast<uint16_t *>(blocks + b * 34);
    dst[0] = reinterpret_cast<const uint16_t *>(d)[(size_t)kb * ld + row_off + row];
    const uint16_t *src = reinterpret_cast<const uint16_t *>(q + (size_t)(row_off + row) * cols + (size_t)kb * 32);
#pragma unroll
    for (int i = 0; i < 16; ++i) dst[1 + i] = src[i];
}

static const size_t STAGE_BYTES = (size_t)64 << 20;

int qb_weight_fill_upload(qb_ctx *ctx, qb_weight *w, uint32_t row_off, uint32_t rows, const void *host_blocks) {
    QB_REQUIRE(host_blocks != nullptr, "weight upload: host pointer is null");
    QB_REQUIRE(row_off + rows <= w->rows_pad, "weight upload out of range");
    const size_t row_bytes = (size_t)(w->cols / 32) * 34;
    const uint32_t rows_per = (uint32_t)std::max<size_t>(1, STAGE_BYTES / row_bytes);
    void *stage = nullptr;
    QB_CUDA(cudaMalloc(&stage, (size_t)std::min(rows_per, rows) * row_bytes));
    for (uint32_t r0 = 0; r0 < rows; r0 += rows_per) {
        const uint32_t nr = std::min(rows_per, rows - r0);
        QB_CUDA(cudaMemcpyAsync(stage, (const uint8_t *)host_blocks + (size_t)r0 * row_bytes, (size_t)nr * row_bytes,
                                cudaMemcpyHostToDevice, ctx->stream));
        const uint64_t nblocks = (uint64_t)nr * (w->cols / 32);
        q8_repack_kernel<<<(uint32_t)((nblocks + 127) / 128), 128, 0, ctx->stream>>>(w->q, w->d, w->ld, w->cols,
                                                                                     row_off + r0, nr, (const uint8_t *)stage);
        QB_LAUNCHED(ctx, "q8_repack_kernel");
        QB_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    QB_CUDA(cudaFree(stage));
    return QB_OK;
}

extern "C" int qb_weight_q8_0(qb_ctx *ctx, const void *host_blocks, uint32_t rows, uint32_t cols, qb_weight **out) {
    QB_REQUIRE(ctx && out, "qb_weight_q8_0: null argument");
    qb_weight *w = nullptr;
    QB_TRY(qb_weight_alloc(ctx, rows, cols, &w));
    int s = qb_weight_fill_upload(ctx, w, 0, rows, host_blocks);
    if (s != QB_OK) { qb_weight_free(ctx, w); return s; }
    *out = w;
    return QB_OK;
}

extern "C" int qb_weight_q8_0_synth(qb_ctx *ctx, uint64_t seed, uint32_t tensor_id, uint32_t rows, uint32_t cols,
                                    float sigma, qb_weight **out) {
    QB_REQUIRE(ctx && out, "qb_weight_q8_0_synth: null argument");
    qb_weight *w = nullptr;
    QB_TRY(qb_weight_alloc(ctx, rows, cols, &w));
    int s = qb_weight_fill_synth(ctx, w, 0, rows, seed, tensor_id, sigma);
    if (s != QB_OK) { qb_weight_free(ctx, w); return s; }
    *out = w;
    return QB_OK;
}

extern "C" int qb_weight_q8_0_download(qb_ctx *ctx, const qb_weight *w, void *host_blocks) {
    const size_t row_bytes = (size_t)(w->cols / 32) * 34;
    const uint32_t rows_per = (uint32_t)std::max<size_t>(1, STAGE_BYTES / row_bytes);
    void *stage = nullptr;
    QB_CUDA(cudaMalloc(&stage, (size_t)std::min(rows_per, w->rows) * row_bytes));
    for (uint32_t r0 = 0; r0 < w->rows; r0 += rows_per) {
        const uint32_t nr = std::min(rows_per, w->rows - r0);
        const uint64_t nblocks = (uint64_t)nr * (w->cols / 32);
        q8_unpack_kernel<<<(uint32_t)((nblocks + 127) / 128), 128, 0, ctx->stream>>>(w->q, w->d, w->ld, w->cols, r0, nr,
                                                                                     (uint8_t *)stage);
        QB_LAUNCHED(ctx, "q8_unpack_kernel");
        QB_CUDA(cudaMemcpyAsync((uint8_t *)host_blocks + (size_t)r0 * row_bytes, stage, (size_t)nr * row_bytes,
                                cudaMemcpyDeviceToHost, ctx->stream));
        QB_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    QB_CUDA(cudaFree(stage));
    return QB_OK;
}

// q8_get_rows_batch_kernel (src/kernels_cuda.cu:2075-2157): out[i][c] = fp16(d) * q.
__global__ void q8_get_rows_kernel(const int8_t *__restrict__ q, const __half *__restrict__ d, uint32_t ld, uint32_t cols,
                                   uint32_t rows, const int32_t *__restrict__ ids, float *out, uint32_t out_stride) {
    const uint32_t i = blockIdx.y;
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    int32_t row = ids[i];
    row = row < 0 ? 0 : (row >= (int32_t)rows ? (int32_t)rows - 1 : row);
    const float dv = __half2float(d[(size_t)(c / 32) * ld + row]);
    out[(size_t)i * out_stride + c] = dv * (float)q[(size_t)row * cols + c];
}

int qb_launch_get_rows(qb_ctx *ctx, const qb_weight *w, const int32_t *ids_dev, uint32_t n, float *out,
                       uint32_t out_stride) {
    if (n == 0) return QB_OK;
    dim3 grid((w->cols + 255) / 256, n);
    q8_get_rows_kernel<<<grid, 256, 0, ctx->stream>>>(w->q, w->d, w->ld, w->cols, w->rows, ids_dev, out, out_stride);
    QB_LAUNCHED(ctx, "q8_get_rows_kernel");
    return QB_OK;
}

extern "C" int qb_q8_0_get_rows(qb_ctx *ctx, const qb_weight *w, const int32_t *ids_dev, uint32_t n, float *out_dev,
                                uint32_t out_stride) {
    QB_REQUIRE(ctx && w && ids_dev && out_dev, "qb_q8_0_get_rows: null argument");
    QB_REQUIRE(out_stride >= w->cols, "qb_q8_0_get_rows: out_stride < cols");
    return qb_launch_get_rows(ctx, w, ids_dev, n, out_dev, out_stride);
}
