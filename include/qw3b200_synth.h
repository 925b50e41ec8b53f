/* Seeded synthetic model data for the qwen35 MTP decode step.
 *
 * There is no model file for this path (weights are random-init from a seed), so
 * the byte recipe for every tensor is defined here once, in plain C that compiles
 * unchanged as host C/C++ and as CUDA device code.  A Q8_0 tensor is defined block
 * by block: block `b` (row-major block index row * (cols/32) + kb) of tensor
 * `tensor_id` is
 *
 *     u[0..31]  = 32 x 16-bit draws from Philox-4x32-10(key = seed, counter = (b, j, tensor_id))
 *     x[t]      = sigma * NORMAL_TABLE[u[t]]          (65536-quantile normal, host-built table)
 *     d         = amax(x) / 127 ;  d_inv = d ? 1/d : 0
 *     stored    = fp16(d), q[t] = clamp(lrint(x[t] * d_inv), -127, 127)
 *
 * which is the host quantiser of the reference's Q8 GEMM parity test
 * (tests/mmq_parity.cu:54-80) applied to N(0, sigma^2) samples.  All arithmetic after the
 * table lookup is single IEEE operations (mul, div, round-to-nearest-even), so host and
 * device produce the same 34 bytes.
 */
#ifndef QW3B200_SYNTH_H
#define QW3B200_SYNTH_H

#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define QS_HD __host__ __device__ static inline
#else
#define QS_HD static inline
#endif

#define QS_NORMAL_TABLE_SIZE 65536

typedef struct { uint32_t v[4]; } qs_u32x4;

QS_HD uint32_t qs_mulhi(uint32_t a, uint32_t b) {
    return (uint32_t)(((uint64_t)a * (uint64_t)b) >> 32);
}

/* Philox-4x32 with 10 rounds (Salmon et al., SC'11). */
QS_HD qs_u32x4 qs_philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                             uint32_t k0, uint32_t k1) {
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = qs_mulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = qs_mulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0;
        const uint32_t n1 = lo1;
        const uint32_t n2 = hi0 ^ c3 ^ k1;
        const uint32_t n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    qs_u32x4 o; o.v[0] = c0; o.v[1] = c1; o.v[2] = c2; o.v[3] = c3;
    return o;
}

/* fp32 -> fp16 bits, round to nearest even, no NaN handling needed (finite inputs). */
QS_HD uint16_t qs_f32_to_f16_bits(float f) {
    union { float f; uint32_t u; } in; in.f = f;
    const uint32_t x = in.u;
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t mant = x & 0x007FFFFFu;
    const int32_t  exp  = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);              /* overflow -> inf */
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;                      /* underflow -> 0 */
        const uint32_t m = mant | 0x00800000u;
        const uint32_t shift = (uint32_t)(14 - exp);
        uint32_t h = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u);
        const uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1u))) h++;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((uint32_t)exp << 10) | (mant >> 13);
    const uint32_t rem = mant & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)(sign | h);
}

QS_HD float qs_f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t mant = h & 0x3FFu;
    union { float f; uint32_t u; } out;
    if (exp == 0) {
        if (mant == 0) { out.u = sign; return out.f; }
        int e = -1;
        do { mant <<= 1; ++e; } while (!(mant & 0x400u));
        mant &= 0x3FFu;
        out.u = sign | ((uint32_t)(127 - 15 - e) << 23) | (mant << 13);
        return out.f;
    }
    if (exp == 31) { out.u = sign | 0x7F800000u | (mant << 13); return out.f; }
    out.u = sign | ((exp - 15 + 127) << 23) | (mant << 13);
    return out.f;
}

/* Writes the 32 samples (already scaled by sigma) of one block. */
QS_HD void qs_block_samples(const float *normal_table, uint64_t seed, uint32_t tensor_id,
                            uint64_t block, float sigma, float *x32) {
    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    for (uint32_t j = 0; j < 4; ++j) {
        const qs_u32x4 r = qs_philox4x32((uint32_t)block, (uint32_t)(block >> 32), j, tensor_id, k0, k1);
        for (int w = 0; w < 4; ++w) {
            x32[j * 8 + w * 2 + 0] = sigma * normal_table[r.v[w] & 0xFFFFu];
            x32[j * 8 + w * 2 + 1] = sigma * normal_table[r.v[w] >> 16];
        }
    }
}

/* Quantises 32 floats to one Q8_0 block: returns the fp16 scale bits, fills q[32]. */
QS_HD uint16_t qs_quantize_q8_0_block(const float *x32, int8_t *q32) {
    float amax = 0.0f;
    for (int t = 0; t < 32; ++t) { const float a = fabsf(x32[t]); amax = a > amax ? a : amax; }
    const float d = amax / 127.0f;
    const float d_inv = (d == 0.0f) ? 0.0f : 1.0f / d;
    for (int t = 0; t < 32; ++t) {
        int qi = (int)rintf(x32[t] * d_inv);
        qi = qi < -127 ? -127 : (qi > 127 ? 127 : qi);
        q32[t] = (int8_t)qi;
    }
    return qs_f32_to_f16_bits(d);
}

/* One synthetic Q8_0 block in GGUF order: out34 = [fp16 d][int8 q x 32]. */
QS_HD void qs_synth_q8_0_block(const float *normal_table, uint64_t seed, uint32_t tensor_id,
                               uint64_t block, float sigma, uint16_t *d_bits, int8_t *q32) {
    float x[32];
    qs_block_samples(normal_table, seed, tensor_id, block, sigma, x);
    *d_bits = qs_quantize_q8_0_block(x, q32);
}

/* Uniform in [0,1) with 24 bits from one Philox word; used for the small fp32 tensors
 * and for token ids, host side only. */
QS_HD uint32_t qs_rand_u32(uint64_t seed, uint32_t stream, uint64_t index) {
    const qs_u32x4 r = qs_philox4x32((uint32_t)index, (uint32_t)(index >> 32), 0x51u, stream,
                                     (uint32_t)seed, (uint32_t)(seed >> 32));
    return r.v[0];
}

/* Host only. Inverse normal CDF (Acklam's rational approximation + one Halley step on erfc). */
static inline double qs_inv_normal_cdf(double p) {
    static const double a[6] = {-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02,
                                1.383577518672690e+02, -3.066479806614716e+01, 2.506628277459239e+00};
    static const double b[5] = {-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02,
                                6.680131188771972e+01, -1.328068155288572e+01};
    static const double c[6] = {-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00,
                                -2.549732539343734e+00, 4.374664141464968e+00, 2.938163982698783e+00};
    static const double d[4] = {7.784695709041462e-03, 3.224671290700398e-01, 2.445134137142996e+00,
                                3.754408661907416e+00};
    double x;
    if (p < 0.02425) {
        const double q = sqrt(-2.0 * log(p));
        x = (((((c[0] * q + c[1]) * q + c[2]) * q + c[3]) * q + c[4]) * q + c[5]) /
            ((((d[0] * q + d[1]) * q + d[2]) * q + d[3]) * q + 1.0);
    } else if (p > 1.0 - 0.02425) {
        const double q = sqrt(-2.0 * log(1.0 - p));
        x = -(((((c[0] * q + c[1]) * q + c[2]) * q + c[3]) * q + c[4]) * q + c[5]) /
            ((((d[0] * q + d[1]) * q + d[2]) * q + d[3]) * q + 1.0);
    } else {
        const double q = p - 0.5, r = q * q;
        x = (((((a[0] * r + a[1]) * r + a[2]) * r + a[3]) * r + a[4]) * r + a[5]) * q /
            (((((b[0] * r + b[1]) * r + b[2]) * r + b[3]) * r + b[4]) * r + 1.0);
    }
    const double e = 0.5 * erfc(-x / 1.4142135623730951) - p;
    const double u = e * 2.5066282746310002 * exp(x * x / 2.0);
    return x - u / (1.0 + x * u / 2.0);
}

/* table[i] = Phi^-1((i + 0.5) / 65536) as fp32. */
static inline void qs_build_normal_table(float *table) {
    for (int i = 0; i < QS_NORMAL_TABLE_SIZE; ++i) {
        table[i] = (float)qs_inv_normal_cdf(((double)i + 0.5) / (double)QS_NORMAL_TABLE_SIZE);
    }
}

#endif /* QW3B200_SYNTH_H */
