// Gated DeltaNet recurrent layer for the decode / verify rows, with per-row state checkpoints.
//
// Replaces DeviceBackend::recurrent_batch for this path (src/kernels_cuda.cu:15053-15608):
//   recurrent_conv_batch_kernel<4> (:3649-3694)   causal conv1d + SiLU with conv-state checkpoints
//   l2_norm_128_qk_batch_kernel (:4122-4156)      L2 norm of the q and k heads
//   prep_g_sigmoid_beta_kernel + gated_delta_net_kernel (src/gated_delta_net.cu:44-177)
//   recurrent_norm_gate_batch_kernel (:4595-4620) RMSNorm(core) * w * SiLU(z)
// Three launches per layer for any number of sequences (the reference's ragged path loops on the
// host per request).  State lives in slots: [seq][slot][v_head][col][i]; the rows of a step read the
// slot named by slot_in[seq] (a device value written by the accept kernel) and, in checkpoint mode,
// the state after row t goes to slot t, so accepting `a` drafts is "slot_in = a" and nothing is
// copied.  Without checkpoints only the final state is written, to slot 0.
#include "qb_internal.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// grid (qkv_dim / HD, n_seqs), block HD: one head-sized chunk of channels, all rows of a sequence.
template <int HD>
__global__ void __launch_bounds__(HD) dn_conv_kernel(DnArgs a) {
    QB_PDL_ENTER();
    __shared__ float red[HD / 32];
    const uint32_t chunk = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x;
    const uint32_t C = 2 * a.nk * HD + a.nv * HD, R = a.rows_per_seq;
    const uint32_t c = chunk * HD + tid;
    const bool is_qk = chunk < 2 * a.nk;
    const uint32_t slot = (uint32_t)a.slot_in[seq];
    float *conv_seq = a.conv + (size_t)seq * a.n_slots * C * 3;
    float st[3], w[4];
#pragma unroll
    for (int k = 0; k < 3; ++k) st[k] = conv_seq[((size_t)slot * C + c) * 3 + k];
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = a.conv_w[(size_t)c * 4 + k];
    float nxt = qb_ldsum(a.proj, (size_t)seq * R * a.proj_stride + c, a.proj_S, a.proj_pstride);
    for (uint32_t t = 0; t < R; ++t) {
        const size_t row = (size_t)seq * R + t;
        const float cur = nxt;
        if (t + 1 < R) nxt = qb_ldsum(a.proj, (row + 1) * a.proj_stride + c, a.proj_S, a.proj_pstride);   // next row's load overlaps this row
        float acc = w[3] * cur;
#pragma unroll
        for (int k = 0; k < 3; ++k) acc += w[k] * st[k];
        float x = __fdiv_rn(acc, 1.0f + expf(-acc));
        st[0] = st[1]; st[1] = st[2]; st[2] = cur;
        if (is_qk) {
            const float ss = warp_sum(x * x);
            __syncthreads();
            if ((tid & 31) == 0) red[tid >> 5] = ss;
            __syncthreads();
            float tot = 0.0f;
#pragma unroll
            for (int k = 0; k < HD / 32; ++k) tot += red[k];
            x *= rsqrtf(tot + a.eps);
        }
        a.xconv[row * C + c] = x;
        if (a.write_all && t < a.n_slots) {
#pragma unroll
            for (int k = 0; k < 3; ++k) conv_seq[((size_t)t * C + c) * 3 + k] = st[k];
        }
    }
    if (!a.write_all) {
#pragma unroll
        for (int k = 0; k < 3; ++k) conv_seq[(size_t)c * 3 + k] = st[k];
    }
}

// grid (nv, HD / 8, n_seqs), block 128: each warp owns 2 state columns, lanes stripe the k-dim.
template <int HD>
__global__ void __launch_bounds__(128) dn_delta_kernel(DnArgs a) {
    QB_PDL_ENTER();
    constexpr int RPL = HD / 32, CPW = 2;
    const uint32_t vh = blockIdx.x, seq = blockIdx.z, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t col0 = blockIdx.y * 8 + warp * CPW;
    const uint32_t kh = vh % a.nk;                        // src/gated_delta_net.cu:105
    const uint32_t C = 2 * a.nk * HD + a.nv * HD, vdim = a.nv * HD, R = a.rows_per_seq;
    const size_t ssz = (size_t)a.nv * HD * HD;
    float *state_seq = a.state + (size_t)seq * a.n_slots * ssz;
    const uint32_t slot = (uint32_t)a.slot_in[seq];
    float s[CPW][RPL];
#pragma unroll
    for (int cc = 0; cc < CPW; ++cc)
#pragma unroll
        for (int r = 0; r < RPL; ++r)
            s[cc][r] = state_seq[(size_t)slot * ssz + ((size_t)vh * HD + col0 + cc) * HD + r * 32 + lane];
    const float oscale = rsqrtf((float)HD);
    const float A = a.ssm_a[vh], bias = a.dt_bias[vh];
    // operands of one row; the next row's are requested before this row's arithmetic
    struct RowIn { float ga, gb, q[RPL], k[RPL], xv[CPW]; };
    auto load_row = [&](uint32_t t) {
        RowIn in;
        const size_t row = (size_t)seq * R + t;
        const float *x = a.xconv + row * C;
        const size_t pr = row * a.proj_stride + C + vdim;
        in.ga = qb_ldsum(a.proj, pr + vh, a.proj_S, a.proj_pstride);
        in.gb = qb_ldsum(a.proj, pr + a.nv + vh, a.proj_S, a.proj_pstride);
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            in.q[r] = x[kh * HD + r * 32 + lane];
            in.k[r] = x[a.nk * HD + kh * HD + r * 32 + lane];
        }
#pragma unroll
        for (int cc = 0; cc < CPW; ++cc) in.xv[cc] = x[2 * a.nk * HD + vh * HD + col0 + cc];
        return in;
    };
    RowIn nxt = load_row(0);
    for (uint32_t t = 0; t < R; ++t) {
        const size_t row = (size_t)seq * R + t;
        const RowIn in = nxt;
        if (t + 1 < R) nxt = load_row(t + 1);
        const float g = expf(log1pf(expf(in.ga + bias)) * A);
        const float beta = __fdiv_rn(1.0f, 1.0f + expf(-in.gb));
        const float *kr = in.k, *qr = in.q;
#pragma unroll
        for (int cc = 0; cc < CPW; ++cc) {
            float kv = 0.0f;
#pragma unroll
            for (int r = 0; r < RPL; ++r) kv += s[cc][r] * kr[r];
            kv = warp_sum(kv);
            const float delta = (in.xv[cc] - g * kv) * beta;
            float at = 0.0f;
#pragma unroll
            for (int r = 0; r < RPL; ++r) {
                s[cc][r] = g * s[cc][r] + kr[r] * delta;
                at += s[cc][r] * qr[r];
            }
            at = warp_sum(at);
            if (lane == 0) a.core[row * vdim + vh * HD + col0 + cc] = at * oscale;
            if (a.write_all && t < a.n_slots) {
#pragma unroll
                for (int r = 0; r < RPL; ++r)
                    state_seq[(size_t)t * ssz + ((size_t)vh * HD + col0 + cc) * HD + r * 32 + lane] = s[cc][r];
            }
        }
    }
    if (!a.write_all) {
#pragma unroll
        for (int cc = 0; cc < CPW; ++cc)
#pragma unroll
            for (int r = 0; r < RPL; ++r)
                state_seq[((size_t)vh * HD + col0 + cc) * HD + r * 32 + lane] = s[cc][r];
    }
}

// grid (rows, nv), block HD.
template <int HD>
__global__ void __launch_bounds__(HD) dn_normgate_kernel(DnArgs a) {
    QB_PDL_ENTER();
    __shared__ float red[HD / 32];
    const uint32_t row = blockIdx.x, vh = blockIdx.y, i = threadIdx.x, lane = i & 31;
    const uint32_t C = 2 * a.nk * HD + a.nv * HD, vdim = a.nv * HD;
    const float v = a.core[(size_t)row * vdim + vh * HD + i];
    const float ss = warp_sum(v * v);
    if (lane == 0) red[i >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int k = 0; k < HD / 32; ++k) tot += red[k];
    const float z = qb_ldsum(a.proj, (size_t)row * a.proj_stride + C + vh * HD + i, a.proj_S, a.proj_pstride);
    const float o = v * rsqrtf(tot / (float)HD + a.eps) * a.norm_w[i] * __fdiv_rn(z, 1.0f + expf(-z));
    const uint32_t col = vh * HD + i;
    if (a.core_out) a.core_out[(size_t)row * vdim + col] = o;
    if (a.q8) {
        float amax = fabsf(o);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const float d_inv = (amax == 0.0f) ? 0.0f : __fdiv_rn(127.0f, amax);
        a.q8[(size_t)row * a.q_pitch + col] = (int8_t)((amax == 0.0f) ? 0 : __float2int_rn(__fmul_rn(o, d_inv)));
        if (lane == 0) a.d[(size_t)(col / 32) * a.d_ld + row] = (amax == 0.0f) ? 0.0f : __fdiv_rn(1.0f, d_inv);
    }
}

template <int HD>
int launch_all(qb_ctx *ctx, const DnArgs &a) {
    const uint32_t C = 2 * a.nk * HD + a.nv * HD;
    QB_CUDA(qb_launch_pdl(ctx->stream, dn_conv_kernel<HD>, dim3(dim3(C / HD, a.n_seqs)), dim3(HD), (size_t)(0), a));
    QB_LAUNCHED(ctx, "dn_conv_kernel");
    QB_CUDA(qb_launch_pdl(ctx->stream, dn_delta_kernel<HD>, dim3(dim3(a.nv, HD / 8, a.n_seqs)), dim3(128), (size_t)(0), a));
    QB_LAUNCHED(ctx, "dn_delta_kernel");
    QB_CUDA(qb_launch_pdl(ctx->stream, dn_normgate_kernel<HD>, dim3(dim3(a.n_seqs * a.rows_per_seq, a.nv)), dim3(HD), (size_t)(0), a));
    QB_LAUNCHED(ctx, "dn_normgate_kernel");
    return QB_OK;
}

}  // namespace

int qb_launch_deltanet(qb_ctx *ctx, const DnArgs &a) {
    QB_REQUIRE(a.n_seqs > 0 && a.rows_per_seq > 0 && a.n_slots > 0, "deltanet: empty launch");
    QB_REQUIRE(!a.write_all || a.rows_per_seq <= a.n_slots, "deltanet: %u rows need %u checkpoint slots, have %u",
               a.rows_per_seq, a.rows_per_seq, a.n_slots);
    if (a.hd == 128) return launch_all<128>(ctx, a);
    if (a.hd == 64) return launch_all<64>(ctx, a);
    return qb_fail(QB_ERR_UNSUPPORTED, "deltanet: head dim %u unsupported (64/128)", a.hd);
}
