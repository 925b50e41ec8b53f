// Gated DeltaNet recurrent layer for the decode / verify rows, with per-row state checkpoints.
//
// Replaces DeviceBackend::recurrent_batch for this path (src/kernels_cuda.cu:15053-15608):
//   recurrent_conv_batch_kernel<4> (:3649-3694)   causal conv1d + SiLU with conv-state checkpoints
//   l2_norm_128_qk_batch_kernel (:4122-4156)      L2 norm of the q and k heads
//   prep_g_sigmoid_beta_kernel + gated_delta_net_kernel (src/gated_delta_net.cu:44-177)
//   recurrent_norm_gate_batch_kernel (:4595-4620) RMSNorm(core) * w * SiLU(z)
// ONE launch per layer for any number of sequences (the reference's ragged path loops on the host per
// request).  State lives in slots: [seq][slot][v_head][col][i]; the rows of a step read the slot named by
// slot_in[seq] (a device value written by the accept kernel) and, in checkpoint mode, the state after row t
// goes to slot t, so accepting `a` drafts is "slot_in = a" and nothing is copied.  Without checkpoints only
// the final state is written, to slot 0.
#include "qb_internal.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- one kernel for the whole layer -------------------------------------------------------------------------
// grid (HD/COLS, nv, n_seqs), cluster (HD/COLS, 1, 1), block 512: the CTAs of a cluster share one v head, each owns
// COLS = 32 or 64 state columns (a warp 2 or 4 of them, lanes stripe the k dimension).  Rows are processed in blocks of 4:
//   conv + SiLU of the head's q and k channels (every CTA of the head repeats them: 2*HD cheap channels) and of
//   its own 32 v channels, L2 norm of q and k, all in shared memory;
//   the delta rule for the block's rows on the register-resident state (checkpoints written as it goes);
//   the head-wide mean square of the core output crosses the cluster once per block through distributed shared
//   memory (push + one barrier.cluster); RMSNorm * gain * SiLU(z) and the int8 quantisation of the CTA's 32
//   columns (= one quantisation block).
// The q/k conv windows are read by several CTAs but written by one (v head < nk, column block 0), so the kernel
// reads the conv state from conv and writes it to conv_out (a different buffer: the caller ping-pongs).
// RB = rows per block (one conv / norm phase, one exchange of the head's sums of squares and one norm-gate phase per
// block): 4 for the decode and verify steps, 8 for prompt ingestion, where the per-block costs dominate.  A row's
// arithmetic does not depend on RB.
template <int HD, int CPW, int RB, int MINB>
__global__ void __launch_bounds__(512, MINB) dn_fused_kernel(DnArgs a) {
    constexpr int COLS = 16 * CPW, NCB = HD / COLS, NQB = COLS / 32, RPL = HD / 32, NCH = 2 * HD + COLS;
    static_assert(NCB * NQB * RB <= 32 && NQB * RB <= 16 && 2 * RB <= 32, "row block too large for the warp role mapping");
    constexpr int QK_WARPS = 2 * HD / 32;
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");     // "this CTA runs": awaited before the first push
    QB_PDL_ENTER();
    __shared__ float xs[RB][NCH];
    __shared__ float red[RB][8];
    __shared__ float core_s[RB][COLS];
    __shared__ float gbs[RB][2];
    __shared__ float cl_ss[2][HD / 32][RB];      // sums of squares per 32-column group of the head, by block parity
    const uint32_t cb = blockIdx.x, vh = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t slot = (uint32_t)a.slot_in[seq];        // requested now, first needed after the block inputs
    const uint32_t kh = vh % a.nk;                         // src/gated_delta_net.cu:105
    const uint32_t C = 2 * a.nk * HD + a.nv * HD, vdim = a.nv * HD, R = a.rows_per_seq;
    const size_t ssz = (size_t)a.nv * HD * HD;
    float *state_seq = a.state + (size_t)seq * a.n_slots * ssz;
    const float *conv_in = a.conv + (size_t)seq * a.n_slots * C * 3;
    float *conv_out = a.conv_out + (size_t)seq * a.n_slots * C * 3;

    // thread tid < NCH convolves one channel: a q or k channel of head kh, or one of this CTA's 32 v channels
    const bool has = tid < NCH, is_qk = tid < 2 * HD;
    const uint32_t ch = tid < HD ? kh * HD + tid : tid < 2 * HD ? a.nk * HD + kh * HD + (tid - HD) : 2 * a.nk * HD + vh * HD + cb * COLS + (tid - 2 * HD);
    const bool writes = is_qk ? (vh < a.nk && cb == 0) : true;
    const uint32_t col0 = cb * COLS + warp * CPW;
    const uint32_t ng_t = warp % RB, ng_q = warp / RB;       // norm-gate role of this warp: row of the block, 32-column group

    // The inputs of a row block (projection rows, gate inputs, z) do not depend on the state slot: they are
    // requested first, and the next block's while the current one is processed.
    struct BlockIn { float cur[RB]; float zv, graw; };
    // Ingestion form: every load of a block is issued before the first add (a load-add-load-add chain exposes one memory
    // latency per row); each element still adds its K-segment partials in ascending order.
    auto load_block = [&](uint32_t rb0) {
        BlockIn in;
        const uint32_t nrows = rb0 < R ? min((uint32_t)RB, R - rb0) : 0u;
        const size_t row0 = (size_t)seq * R + rb0;
        if constexpr (RB <= 4) {
            // the step forms (64 registers per thread): element by element
            if (a.proj_S == 2) {                      // the usual split of the input projection: both partials of every row first
                float p1[RB];
#pragma unroll
                for (int t = 0; t < RB; ++t) {
                    const bool on = has && (uint32_t)t < nrows;
                    in.cur[t] = on ? a.proj[(row0 + t) * a.proj_stride + ch] : 0.0f;
                    p1[t] = on ? a.proj[(row0 + t) * a.proj_stride + ch + a.proj_pstride] : 0.0f;
                }
#pragma unroll
                for (int t = 0; t < RB; ++t) in.cur[t] += p1[t];
            } else {
#pragma unroll
                for (int t = 0; t < RB; ++t) {
                    in.cur[t] = 0.0f;
                    if (has && (uint32_t)t < nrows) in.cur[t] = qb_ldsum(a.proj, (row0 + t) * a.proj_stride + ch, a.proj_S, a.proj_pstride);
                }
            }
            in.zv = 0.0f;
            if (ng_q < NQB && ng_t < nrows)
                in.zv = qb_ldsum(a.proj, (row0 + ng_t) * a.proj_stride + C + vh * HD + cb * COLS + ng_q * 32 + lane, a.proj_S, a.proj_pstride);
            in.graw = 0.0f;
            if (warp == 15 && lane < 2 * nrows)      // (row, decay | write strength) of the block: lanes of the last warp
                in.graw = qb_ldsum(a.proj, (row0 + (lane >> 1)) * a.proj_stride + C + vdim + (lane & 1) * a.nv + vh, a.proj_S, a.proj_pstride);
            return in;
        }
        const uint32_t S = a.proj_S;
        const bool two = S > 1;
        const bool hz = ng_q < NQB && ng_t < nrows, hg = warp == 15 && lane < 2 * nrows;
        const size_t iz = (row0 + ng_t) * a.proj_stride + C + vh * HD + cb * COLS + ng_q * 32 + lane;
        const size_t ig = (row0 + (lane >> 1)) * a.proj_stride + C + vdim + (lane & 1) * a.nv + vh;
        float p0[RB], p1[RB];
#pragma unroll
        for (int t = 0; t < RB; ++t) {
            const bool on = has && (uint32_t)t < nrows;
            p0[t] = on ? a.proj[(row0 + t) * a.proj_stride + ch] : 0.0f;
            p1[t] = on && two ? a.proj[(row0 + t) * a.proj_stride + ch + a.proj_pstride] : 0.0f;
        }
        const float z0 = hz ? a.proj[iz] : 0.0f, z1 = hz && two ? a.proj[iz + a.proj_pstride] : 0.0f;
        const float g0 = hg ? a.proj[ig] : 0.0f, g1 = hg && two ? a.proj[ig + a.proj_pstride] : 0.0f;
#pragma unroll
        for (int t = 0; t < RB; ++t) in.cur[t] = two ? p0[t] + p1[t] : p0[t];
        in.zv = two ? z0 + z1 : z0;
        in.graw = two ? g0 + g1 : g0;
        for (uint32_t sg = 2; sg < S; ++sg) {                 // further segments: again all loads, then the adds
            const size_t off = (size_t)sg * a.proj_pstride;
#pragma unroll
            for (int t = 0; t < RB; ++t) p0[t] = has && (uint32_t)t < nrows ? a.proj[(row0 + t) * a.proj_stride + ch + off] : 0.0f;
            const float zs = hz ? a.proj[iz + off] : 0.0f, gs = hg ? a.proj[ig + off] : 0.0f;
#pragma unroll
            for (int t = 0; t < RB; ++t) in.cur[t] += p0[t];
            in.zv += zs;
            in.graw += gs;
        }
        return in;
    };
    BlockIn nxt = load_block(0);
    float w[4] = {0.f, 0.f, 0.f, 0.f};
    if (has) {
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = a.conv_w[(size_t)ch * 4 + k];
    }
    const float oscale = rsqrtf((float)HD);
    const float A = a.ssm_a[vh], bias = a.dt_bias[vh];
    const float nw = ng_q < NQB ? a.norm_w[cb * COLS + ng_q * 32 + lane] : 0.0f;
    uint32_t crank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
    // ... then everything that hangs on the slot: conv window and the warp's state columns
    float st[3] = {0.f, 0.f, 0.f};
    if (has) {
#pragma unroll
        for (int k = 0; k < 3; ++k) st[k] = conv_in[((size_t)slot * C + ch) * 3 + k];
    }
    float s[CPW][RPL];
#pragma unroll
    for (int cc = 0; cc < CPW; ++cc)
#pragma unroll
        for (int r = 0; r < RPL; ++r)
            s[cc][r] = state_seq[(size_t)slot * ssz + ((size_t)vh * HD + col0 + cc) * HD + r * 32 + lane];

    for (uint32_t rb0 = 0, blk = 0; rb0 < R; rb0 += RB, ++blk) {
        const uint32_t nrows = min((uint32_t)RB, R - rb0), par = blk & 1;
        const size_t row0 = (size_t)seq * R + rb0;
        const BlockIn in = nxt;
        nxt = load_block(rb0 + RB);
        const float zv = in.zv;
        float cur[RB];
#pragma unroll
        for (int t = 0; t < RB; ++t) cur[t] = in.cur[t];
        // decay and write strength of the block's rows
        if (warp == 15 && lane < 2 * nrows)
            gbs[lane >> 1][lane & 1] = (lane & 1) == 0 ? expf(log1pf(expf(in.graw + bias)) * A) : __fdiv_rn(1.0f, 1.0f + expf(-in.graw));
        // conv + SiLU, conv-state checkpoints
        float x[RB];
#pragma unroll
        for (int t = 0; t < RB; ++t) {
            x[t] = 0.0f;
            if (has && (uint32_t)t < nrows) {
                float acc = w[3] * cur[t];
#pragma unroll
                for (int k = 0; k < 3; ++k) acc += w[k] * st[k];
                x[t] = __fdiv_rn(acc, 1.0f + expf(-acc));
                st[0] = st[1]; st[1] = st[2]; st[2] = cur[t];
                if (writes && a.write_all && rb0 + t < a.n_slots) {
#pragma unroll
                    for (int k = 0; k < 3; ++k) conv_out[((size_t)(rb0 + t) * C + ch) * 3 + k] = st[k];
                }
            }
            if (warp < QK_WARPS) {                    // warp-uniform: q and k channels only
                const float ss = warp_sum(x[t] * x[t]);
                if (lane == 0) red[t][warp] = ss;
            }
        }
        __syncthreads();
        if (has) {
#pragma unroll
            for (int t = 0; t < RB; ++t) {
                if ((uint32_t)t >= nrows) continue;
                float v = x[t];
                if (is_qk) {
                    const int g0 = tid < HD ? 0 : HD / 32;
                    float tot = 0.0f;
#pragma unroll
                    for (int k = 0; k < HD / 32; ++k) tot += red[t][g0 + k];
                    v *= rsqrtf(tot + a.eps);
                }
                xs[t][tid] = v;
            }
        }
        __syncthreads();
        // delta rule on the block's rows
#pragma unroll 1
        for (uint32_t t = 0; t < nrows; ++t) {
            const float g = gbs[t][0], beta = gbs[t][1];
            float kr[RPL], qr[RPL];
#pragma unroll
            for (int r = 0; r < RPL; ++r) { qr[r] = xs[t][r * 32 + lane]; kr[r] = xs[t][HD + r * 32 + lane]; }
            if constexpr (CPW == 4) {
                // Four columns per warp: their 32-lane sums share their shuffles.  Each exchange step halves the
                // values a lane carries (lanes 16+ keep columns 2 and 3, then lanes with bit 3 the odd one), so a
                // lane ends with the total of one column; every partial sum is the same pair added in the same
                // step as in the plain butterfly, hence the same bits.  The totals come back with four broadcasts.
                const bool hi16 = (lane & 16) != 0, hi8 = (lane & 8) != 0;
                auto sum4 = [&](const float (&v)[4]) -> float {
                    float k0 = hi16 ? v[2] : v[0], k1 = hi16 ? v[3] : v[1];
                    const float s0 = hi16 ? v[0] : v[2], s1 = hi16 ? v[1] : v[3];
                    k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
                    k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
                    float k = hi8 ? k1 : k0;
                    const float sd = hi8 ? k0 : k1;
                    k += __shfl_xor_sync(0xffffffffu, sd, 8);
                    k += __shfl_xor_sync(0xffffffffu, k, 4);
                    k += __shfl_xor_sync(0xffffffffu, k, 2);
                    k += __shfl_xor_sync(0xffffffffu, k, 1);
                    return k;                                  // total of column 2 * hi16 + hi8
                };
                float kvp[4];
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    float kv = 0.0f;
#pragma unroll
                    for (int r = 0; r < RPL; ++r) kv += s[cc][r] * kr[r];
                    kvp[cc] = kv;
                }
                const float kvt = sum4(kvp);
                float atp[4];
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const float kv = __shfl_sync(0xffffffffu, kvt, 8 * (cc & 1) + 16 * (cc >> 1));
                    const float delta = (xs[t][2 * HD + warp * CPW + cc] - g * kv) * beta;
                    float at = 0.0f;
#pragma unroll
                    for (int r = 0; r < RPL; ++r) {
                        s[cc][r] = g * s[cc][r] + kr[r] * delta;
                        at += s[cc][r] * qr[r];
                    }
                    atp[cc] = at;
                    if (a.write_all && rb0 + t < a.n_slots) {
#pragma unroll
                        for (int r = 0; r < RPL; ++r)
                            state_seq[(size_t)(rb0 + t) * ssz + ((size_t)vh * HD + col0 + cc) * HD + r * 32 + lane] = s[cc][r];
                    }
                }
                const float att = sum4(atp);
                if ((lane & 7) == 0) core_s[t][warp * CPW + 2 * (lane >> 4) + ((lane >> 3) & 1)] = att * oscale;
            } else if constexpr (CPW == 2) {
                // two columns per warp: the same sharing, one halving step
                const bool hi16 = (lane & 16) != 0;
                auto sum2 = [&](float v0, float v1) -> float {
                    float k = hi16 ? v1 : v0;
                    const float sd = hi16 ? v0 : v1;
                    k += __shfl_xor_sync(0xffffffffu, sd, 16);
                    k += __shfl_xor_sync(0xffffffffu, k, 8);
                    k += __shfl_xor_sync(0xffffffffu, k, 4);
                    k += __shfl_xor_sync(0xffffffffu, k, 2);
                    k += __shfl_xor_sync(0xffffffffu, k, 1);
                    return k;                                  // total of column hi16
                };
                float kvp[2], atp[2];
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    float kv = 0.0f;
#pragma unroll
                    for (int r = 0; r < RPL; ++r) kv += s[cc][r] * kr[r];
                    kvp[cc] = kv;
                }
                const float kvt = sum2(kvp[0], kvp[1]);
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const float kv = __shfl_sync(0xffffffffu, kvt, 16 * cc);
                    const float delta = (xs[t][2 * HD + warp * CPW + cc] - g * kv) * beta;
                    float at = 0.0f;
#pragma unroll
                    for (int r = 0; r < RPL; ++r) {
                        s[cc][r] = g * s[cc][r] + kr[r] * delta;
                        at += s[cc][r] * qr[r];
                    }
                    atp[cc] = at;
                    if (a.write_all && rb0 + t < a.n_slots) {
#pragma unroll
                        for (int r = 0; r < RPL; ++r)
                            state_seq[(size_t)(rb0 + t) * ssz + ((size_t)vh * HD + col0 + cc) * HD + r * 32 + lane] = s[cc][r];
                    }
                }
                const float att = sum2(atp[0], atp[1]);
                if ((lane & 15) == 0) core_s[t][warp * CPW + (lane >> 4)] = att * oscale;
            } else {
#pragma unroll
            for (int cc = 0; cc < CPW; ++cc) {
                float kv = 0.0f;
#pragma unroll
                for (int r = 0; r < RPL; ++r) kv += s[cc][r] * kr[r];
                kv = warp_sum(kv);
                const float delta = (xs[t][2 * HD + warp * CPW + cc] - g * kv) * beta;
                float at = 0.0f;
#pragma unroll
                for (int r = 0; r < RPL; ++r) {
                    s[cc][r] = g * s[cc][r] + kr[r] * delta;
                    at += s[cc][r] * qr[r];
                }
                at = warp_sum(at);
                if (lane == 0) core_s[t][warp * CPW + cc] = at * oscale;
                if (a.write_all && rb0 + t < a.n_slots) {
#pragma unroll
                    for (int r = 0; r < RPL; ++r)
                        state_seq[(size_t)(rb0 + t) * ssz + ((size_t)vh * HD + col0 + cc) * HD + r * 32 + lane] = s[cc][r];
                }
            }
            }
        }
        __syncthreads();
        // this CTA's part of the head's sum of squares, pushed to every CTA of the cluster
        if (blk == 0) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");      // all CTAs of the cluster run
        if (warp == 0) {
            // one value per (32-column group of this CTA, row); the same grouping whatever COLS is, so the
            // head's sum below adds the same numbers in the same order in both forms of the kernel
            float mine = 0.0f;
#pragma unroll
            for (int q = 0; q < NQB; ++q)
#pragma unroll
                for (int t = 0; t < RB; ++t) {
                    const float v = (uint32_t)t < nrows ? core_s[t][q * 32 + lane] : 0.0f;
                    const float ss = warp_sum(v * v);
                    if ((lane % (NQB * RB)) == (uint32_t)(q * RB + t)) mine = ss;
                }
            if (lane < NCB * NQB * RB) {
                const uint32_t dest = lane / (NQB * RB), q = (lane / RB) % NQB, t = lane % RB;
                uint32_t local = (uint32_t)__cvta_generic_to_shared(&cl_ss[par][crank * NQB + q][t]), remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(dest));
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(mine) : "memory");
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        // RMSNorm * gain * SiLU(z), int8 quantisation: a warp takes (row, 32-column group), lane = column
        if (ng_q < NQB && ng_t < nrows) {
            const uint32_t t = ng_t, col = vh * HD + cb * COLS + ng_q * 32 + lane;
            const size_t row = row0 + t;
            float tot = 0.0f;
#pragma unroll
            for (int r = 0; r < HD / 32; ++r) tot += cl_ss[par][r][t];
            const float o = core_s[t][ng_q * 32 + lane] * rsqrtf(tot / (float)HD + a.eps) * nw * __fdiv_rn(zv, 1.0f + expf(-zv));
            if (a.core_out) a.core_out[row * vdim + col] = o;
            if (a.q8) {
                float amax = fabsf(o);
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
                const float d_inv = (amax == 0.0f) ? 0.0f : __fdiv_rn(127.0f, amax);
                a.q8[row * a.q_pitch + col] = (int8_t)((amax == 0.0f) ? 0 : __float2int_rn(__fmul_rn(o, d_inv)));
                if (lane == 0) a.d[(size_t)(col / 32) * a.d_ld + row] = (amax == 0.0f) ? 0.0f : __fdiv_rn(1.0f, d_inv);
            }
        }
    }
    if (!a.write_all) {
        if (has && writes) {
#pragma unroll
            for (int k = 0; k < 3; ++k) conv_out[(size_t)ch * 3 + k] = st[k];
        }
#pragma unroll
        for (int cc = 0; cc < CPW; ++cc)
#pragma unroll
            for (int r = 0; r < RPL; ++r)
                state_seq[((size_t)vh * HD + col0 + cc) * HD + r * 32 + lane] = s[cc][r];
    }
}

template <int HD, int CPW, int RB, int MINB>
int launch_fused(qb_ctx *ctx, const DnArgs &a) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(HD / (16 * CPW), a.nv, a.n_seqs);
    cfg.blockDim = dim3(512);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = HD / (16 * CPW);
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    QB_CUDA(cudaLaunchKernelEx(&cfg, (dn_fused_kernel<HD, CPW, RB, MINB>), a));
    QB_LAUNCHED(ctx, "dn_fused_kernel");
    return QB_OK;
}

}  // namespace

int qb_launch_deltanet(qb_ctx *ctx, const DnArgs &a) {
    QB_REQUIRE(a.n_seqs > 0 && a.rows_per_seq > 0 && a.n_slots > 0, "deltanet: empty launch");
    QB_REQUIRE(!a.write_all || a.rows_per_seq <= a.n_slots, "deltanet: %u rows need %u checkpoint slots, have %u",
               a.rows_per_seq, a.rows_per_seq, a.n_slots);
    QB_REQUIRE(a.conv_out && a.conv_out != a.conv, "deltanet: the new conv state needs a buffer of its own");
    // one request: 32 state columns per CTA (more CTAs, shortest critical path); several: 64 per CTA (the per-CTA
    // work that does not depend on the column count — the head's q/k conv, the barriers — is paid half as often)
    // prompt ingestion (many rows per sequence): 64 columns per CTA and 8-row blocks
    const bool wide = a.n_seqs > 2, many = a.rows_per_seq >= 16;
    if (a.hd == 128) return many ? launch_fused<128, 4, 8, 1>(ctx, a) : wide ? launch_fused<128, 4, 4, 2>(ctx, a) : launch_fused<128, 2, 4, 2>(ctx, a);
    if (a.hd == 64) return many ? launch_fused<64, 4, 8, 1>(ctx, a) : wide ? launch_fused<64, 4, 4, 2>(ctx, a) : launch_fused<64, 2, 4, 2>(ctx, a);
    return qb_fail(QB_ERR_UNSUPPORTED, "deltanet: head dim %u unsupported (64/128)", a.hd);
}
