// Q8_0 weights in device layout: upload + repack, seeded on-device generation, download, views.
//
// Replaces the CudaWeight Q8_0 constructor of the reference (src/kernels_cuda.cu:1566-1594), which
// repacks GGUF's interleaved 34-byte blocks into per-row [scales | quants].  Here the repack target is
// the record layout described in qb_internal.h: 128 x 128 tiles, each stored as the swizzled
// shared-memory image of its quants followed by its scales, so that one GEMM pipeline stage is one
// contiguous 17 KB bulk copy.  34 bytes per 32 weights, as on disk.
#include "qb_internal.h"

int qb_weight_alloc(qb_ctx *ctx, uint32_t rows, uint32_t cols, qb_weight **out) {
    QB_REQUIRE(rows > 0 && cols > 0 && cols % 128 == 0, "Q8_0 weight: cols=%u must be a positive multiple of 128", cols);
    qb_weight *w = new qb_weight();
    w->rows = rows;
    w->cols = cols;
    w->rows_pad = (rows + 127u) & ~127u;
    w->owns = true;
    QB_CUDA(cudaSetDevice(ctx->device));
    const size_t bytes = (size_t)(w->rows_pad / 128) * (cols / 128) * QB_REC_BYTES;
    QB_CUDA(cudaMalloc(&w->rec, bytes));
    if (w->rows_pad != rows) QB_CUDA(cudaMemsetAsync(w->rec, 0, bytes, ctx->stream));
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
    out->rec = w->rec + qb_rec_offset(w->cols, row_off, 0);
    out->owns = false;
    return QB_OK;
}

extern "C" void qb_weight_free(qb_ctx *ctx, qb_weight *w) {
    if (!w) return;
    if (w->owns) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(w->rec);
    }
    delete w;
}
extern "C" uint32_t qb_weight_rows(const qb_weight *w) { return w->rows; }
extern "C" uint32_t qb_weight_cols(const qb_weight *w) { return w->cols; }

// Row of the device weight that holds row `row` of a tensor placed at row_off.  ileave = 0: row_off + row.
// ileave = 64 (the two halves of a fused [gate; up] weight): the tensor's rows go to every other group of 64
// rows, so each 128-row tile of the fused weight holds 64 gate rows (row_off 0) and the 64 up rows (row_off 64)
// of the same hidden indices.
__device__ __forceinline__ uint32_t q8_dest_row(uint32_t row_off, uint32_t row, uint32_t ileave) {
    return ileave ? row_off + (row / ileave) * 2 * ileave + row % ileave : row_off + row;
}

// One thread per 32-block.
// The weight may be a window of the seeded tensor (a tensor-parallel shard): destination row r, block kb hold the tensor's
// row src_row0 + r, block src_kb0 + kb, the tensor having src_nb blocks per row.
__global__ void q8_synth_kernel(uint8_t *rec, uint32_t cols, uint32_t row_off, uint32_t rows,
                                const float *__restrict__ table, uint64_t seed, uint32_t tensor_id, float sigma, uint32_t ileave,
                                uint32_t src_row0, uint32_t src_nb, uint32_t src_kb0) {
    const uint32_t nb = cols / 32;
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (uint64_t)rows * nb) return;
    const uint32_t kb = (uint32_t)(b % nb);
    const uint32_t row = q8_dest_row(0, (uint32_t)(b / nb), ileave);
    uint16_t dbits;
    __align__(16) int8_t qq[32];
    qs_synth_q8_0_block(table, seed, tensor_id, ((uint64_t)src_row0 + b / nb) * src_nb + src_kb0 + kb, sigma, &dbits, qq);
    *reinterpret_cast<int4 *>(rec + qb_q_offset(cols, row_off + row, kb * 32)) = reinterpret_cast<const int4 *>(qq)[0];
    *reinterpret_cast<int4 *>(rec + qb_q_offset(cols, row_off + row, kb * 32 + 16)) = reinterpret_cast<const int4 *>(qq)[1];
    *reinterpret_cast<uint16_t *>(rec + qb_d_offset(cols, row_off + row, kb)) = dbits;
}

int qb_weight_fill_synth(qb_ctx *ctx, qb_weight *w, uint32_t row_off, uint32_t rows, uint64_t seed,
                         uint32_t tensor_id, float sigma, uint32_t ileave) {
    return qb_weight_fill_synth_window(ctx, w, row_off, rows, seed, tensor_id, sigma, ileave, 0, w->cols / 32, 0);
}

int qb_weight_fill_synth_window(qb_ctx *ctx, qb_weight *w, uint32_t row_off, uint32_t rows, uint64_t seed, uint32_t tensor_id, float sigma,
                                uint32_t ileave, uint32_t src_row0, uint32_t src_nb, uint32_t src_kb0) {
    QB_REQUIRE(ileave ? (rows % ileave == 0 && row_off + 2 * rows - ileave <= w->rows_pad) : row_off + rows <= w->rows_pad,
               "synth fill out of range");
    const uint64_t nblocks = (uint64_t)rows * (w->cols / 32);
    const uint32_t threads = 128;
    const uint64_t grid = (nblocks + threads - 1) / threads;
    QB_REQUIRE(grid < (1ull << 31), "synth fill too large");
    q8_synth_kernel<<<(uint32_t)grid, threads, 0, ctx->stream>>>(w->rec, w->cols, row_off, rows, ctx->normal_table_dev, seed,
                                                                tensor_id, sigma, ileave, src_row0, src_nb, src_kb0);
    QB_LAUNCHED(ctx, "q8_synth_kernel");
    return QB_OK;
}

// GGUF blocks (34 B, row-major block order) of `rows` rows -> device layout at row_off.
__global__ void q8_repack_kernel(uint8_t *rec, uint32_t cols, uint32_t row_off, uint32_t rows,
                                 const uint8_t *__restrict__ blocks, uint32_t row0, uint32_t ileave) {
    const uint32_t nb = cols / 32;
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (uint64_t)rows * nb) return;
    const uint32_t kb = (uint32_t)(b % nb);
    const uint32_t row = q8_dest_row(0, row0 + (uint32_t)(b / nb), ileave);       // row0 = tensor row of the first staged row
    const uint16_t *src = reinterpret_cast<const uint16_t *>(blocks + b * 34);   // 2-byte aligned
    *reinterpret_cast<uint16_t *>(rec + qb_d_offset(cols, row_off + row, kb)) = src[0];
    uint16_t *lo = reinterpret_cast<uint16_t *>(rec + qb_q_offset(cols, row_off + row, kb * 32));
    uint16_t *hi = reinterpret_cast<uint16_t *>(rec + qb_q_offset(cols, row_off + row, kb * 32 + 16));
#pragma unroll
    for (int i = 0; i < 8; ++i) { lo[i] = src[1 + i]; hi[i] = src[9 + i]; }
}

__global__ void q8_unpack_kernel(const uint8_t *rec, uint32_t cols, uint32_t row_off, uint32_t rows, uint8_t *blocks) {
    const uint32_t nb = cols / 32;
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (uint64_t)rows * nb) return;
    const uint32_t row = (uint32_t)(b / nb), kb = (uint32_t)(b % nb);
    uint16_t *dst = reinterpret_cast<uint16_t *>(blocks + b * 34);
    dst[0] = *reinterpret_cast<const uint16_t *>(rec + qb_d_offset(cols, row_off + row, kb));
    const uint16_t *lo = reinterpret_cast<const uint16_t *>(rec + qb_q_offset(cols, row_off + row, kb * 32));
    const uint16_t *hi = reinterpret_cast<const uint16_t *>(rec + qb_q_offset(cols, row_off + row, kb * 32 + 16));
#pragma unroll
    for (int i = 0; i < 8; ++i) { dst[1 + i] = lo[i]; dst[9 + i] = hi[i]; }
}

static const size_t STAGE_BYTES = (size_t)64 << 20;

int qb_weight_fill_upload(qb_ctx *ctx, qb_weight *w, uint32_t row_off, uint32_t rows, const void *host_blocks, uint32_t ileave) {
    QB_REQUIRE(host_blocks != nullptr, "weight upload: host pointer is null");
    QB_REQUIRE(ileave ? (rows % ileave == 0 && row_off + 2 * rows - ileave <= w->rows_pad) : row_off + rows <= w->rows_pad,
               "weight upload out of range");
    const size_t row_bytes = (size_t)(w->cols / 32) * 34;
    const uint32_t rows_per = (uint32_t)std::max<size_t>(1, STAGE_BYTES / row_bytes);
    void *stage = nullptr;
    QB_CUDA(cudaMalloc(&stage, (size_t)std::min(rows_per, rows) * row_bytes));
    for (uint32_t r0 = 0; r0 < rows; r0 += rows_per) {
        const uint32_t nr = std::min(rows_per, rows - r0);
        QB_CUDA(cudaMemcpyAsync(stage, (const uint8_t *)host_blocks + (size_t)r0 * row_bytes, (size_t)nr * row_bytes,
                                cudaMemcpyHostToDevice, ctx->stream));
        const uint64_t nblocks = (uint64_t)nr * (w->cols / 32);
        q8_repack_kernel<<<(uint32_t)((nblocks + 127) / 128), 128, 0, ctx->stream>>>(w->rec, w->cols, row_off, nr,
                                                                                     (const uint8_t *)stage, r0, ileave);
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

// Fused [gate; up] weight of an FFN from the two GGUF tensors, rows interleaved in groups of 64 (see q8_dest_row):
// the layout the fused gate/up + SwiGLU kernel needs (a 128-row tile = 64 gate rows + the matching 64 up rows).
extern "C" int qb_weight_q8_0_gate_up(qb_ctx *ctx, const void *gate_blocks, const void *up_blocks, uint32_t n_ff, uint32_t cols,
                                      qb_weight **out) {
    QB_REQUIRE(ctx && gate_blocks && up_blocks && out, "qb_weight_q8_0_gate_up: null argument");
    QB_REQUIRE(n_ff % 64 == 0, "qb_weight_q8_0_gate_up: FFN dimension %u is not a multiple of 64", n_ff);
    qb_weight *w = nullptr;
    QB_TRY(qb_weight_alloc(ctx, 2 * n_ff, cols, &w));
    int s = qb_weight_fill_upload(ctx, w, 0, n_ff, gate_blocks, 64);
    if (s == QB_OK) s = qb_weight_fill_upload(ctx, w, 64, n_ff, up_blocks, 64);
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
        q8_unpack_kernel<<<(uint32_t)((nblocks + 127) / 128), 128, 0, ctx->stream>>>(w->rec, w->cols, r0, nr, (uint8_t *)stage);
        QB_LAUNCHED(ctx, "q8_unpack_kernel");
        QB_CUDA(cudaMemcpyAsync((uint8_t *)host_blocks + (size_t)r0 * row_bytes, stage, (size_t)nr * row_bytes,
                                cudaMemcpyDeviceToHost, ctx->stream));
        QB_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    QB_CUDA(cudaFree(stage));
    return QB_OK;
}

// q8_get_rows_batch_kernel (src/kernels_cuda.cu:2075-2157): out[i][c] = fp16(d) * q.
__global__ void q8_get_rows_kernel(const uint8_t *__restrict__ rec, uint32_t cols, uint32_t rows,
                                   const int32_t *__restrict__ ids, float *out, uint32_t out_stride) {
    QB_PDL_ENTER();
    const uint32_t i = blockIdx.y;
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    int32_t row = ids[i];
    row = row < 0 ? 0 : (row >= (int32_t)rows ? (int32_t)rows - 1 : row);
    const float dv = __half2float(*reinterpret_cast<const __half *>(rec + qb_d_offset(cols, (uint32_t)row, c / 32)));
    out[(size_t)i * out_stride + c] = dv * (float)*reinterpret_cast<const int8_t *>(rec + qb_q_offset(cols, (uint32_t)row, c));
}

int qb_launch_get_rows(qb_ctx *ctx, const qb_weight *w, const int32_t *ids_dev, uint32_t n, float *out,
                       uint32_t out_stride) {
    if (n == 0) return QB_OK;
    dim3 grid((w->cols + 255) / 256, n);
    QB_CUDA(qb_launch_pdl(ctx->stream, q8_get_rows_kernel, dim3(grid), dim3(256), (size_t)(0), w->rec, w->cols, w->rows, ids_dev, out, out_stride));
    QB_LAUNCHED(ctx, "q8_get_rows_kernel");
    return QB_OK;
}

extern "C" int qb_q8_0_get_rows(qb_ctx *ctx, const qb_weight *w, const int32_t *ids_dev, uint32_t n, float *out_dev,
                                uint32_t out_stride) {
    QB_REQUIRE(ctx && w && ids_dev && out_dev, "qb_q8_0_get_rows: null argument");
    QB_REQUIRE(out_stride >= w->cols, "qb_q8_0_get_rows: out_stride < cols");
    return qb_launch_get_rows(ctx, w, ids_dev, n, out_dev, out_stride);
}
