/*
 * fomoe_oracle.c -- scalar C restatement of fomoe's routed-expert FFN decode
 * arithmetic (TEST INFRASTRUCTURE ONLY; see fomoe_oracle.h).
 *
 * The reference computes the Q8_K-activation dots with AVX2 intrinsics.  This
 * file restates the same arithmetic lane by lane in scalar C (fmaf where the
 * reference issues an FMA intrinsic), so the result is bit-identical to the
 * compiled reference and does not depend on this file's compiler flags.
 * Build with -ffp-contract=off: every fused operation below is explicit.
 */
#include "fomoe_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---- fp16 -> fp32 : src/quant.c:30-47 (exact IEEE half to float) ---- */
float orc_fp16_to_fp32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal half: man * 2^-24, exactly representable */
            float f = (float)man * 0x1.0p-24f;
            memcpy(&bits, &f, 4);
            bits |= sign;
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

#ifndef ORC_Q8_0_FMA
#define ORC_Q8_0_FMA 0
#endif
#ifndef ORC_MXFP4_FMA
#define ORC_MXFP4_FMA 1
#endif

uint64_t orc_row_bytes(int type, int k) {
    if (type == ORC_TYPE_Q4_K) return (uint64_t)(k / ORC_QK_K) * sizeof(orc_block_q4_K);
    if (type == ORC_TYPE_Q5_K) return (uint64_t)(k / ORC_QK_K) * sizeof(orc_block_q5_K);
    if (type == ORC_TYPE_Q6_K) return (uint64_t)(k / ORC_QK_K) * sizeof(orc_block_q6_K);
    if (type == ORC_TYPE_Q8_0) return (uint64_t)(k / 32) * 34u;
    if (type == ORC_TYPE_MXFP4) return (uint64_t)(k / 32) * 17u;
    return 0;
}

/* ---- 6-bit scale/min unpack : src/quant.c:72-80 ---- */
static void scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* ---- Q4_K dequant : src/quant.c:82-105.  y = (d*sc)*q - (dmin*m). ---- */
void orc_dequantize_row_q4_K(const void *xv, float *y, int64_t k) {
    const orc_block_q4_K *x = (const orc_block_q4_K *)xv;
    int64_t nb = k / ORC_QK_K;
    for (int64_t i = 0; i < nb; i++) {
        float d = orc_fp16_to_fp32(x[i].d);
        float mn = orc_fp16_to_fp32(x[i].dmin);
        const uint8_t *q = x[i].qs;
        for (int c = 0; c < 4; c++) {
            uint8_t sc1, m1, sc2, m2;
            scale_min_k4(2 * c, x[i].scales, &sc1, &m1);
            scale_min_k4(2 * c + 1, x[i].scales, &sc2, &m2);
            float d1 = d * (float)sc1, mm1 = mn * (float)m1;
            float d2 = d * (float)sc2, mm2 = mn * (float)m2;
            for (int l = 0; l < 32; l++) y[l] = d1 * (float)(q[l] & 0xF) - mm1;
            for (int l = 0; l < 32; l++) y[32 + l] = d2 * (float)(q[l] >> 4) - mm2;
            y += 64;
            q += 32;
        }
    }
}

/* ---- Q5_K dequant : src/quant.c:216-247.  The nibble plus 16 where the fifth bit (qh, bit 2c / 2c+1 for the two
 * halves of 64-chunk c) is set.  d*sc*q has at most 22 significant bits, so contraction cannot change the result. ---- */
void orc_dequantize_row_q5_K(const void *xv, float *y, int64_t k) {
    const orc_block_q5_K *x = (const orc_block_q5_K *)xv;
    int64_t nb = k / ORC_QK_K;
    for (int64_t i = 0; i < nb; i++) {
        float d = orc_fp16_to_fp32(x[i].d);
        float mn = orc_fp16_to_fp32(x[i].dmin);
        const uint8_t *q = x[i].qs;
        const uint8_t *qh = x[i].qh;
        for (int c = 0; c < 4; c++) {
            uint8_t sc1, m1, sc2, m2;
            scale_min_k4(2 * c, x[i].scales, &sc1, &m1);
            scale_min_k4(2 * c + 1, x[i].scales, &sc2, &m2);
            float d1 = d * (float)sc1, mm1 = mn * (float)m1;
            float d2 = d * (float)sc2, mm2 = mn * (float)m2;
            for (int l = 0; l < 32; l++) y[l] = d1 * (float)((q[l] & 0xF) + (((qh[l] >> (2 * c)) & 1) ? 16 : 0)) - mm1;
            for (int l = 0; l < 32; l++)
                y[32 + l] = d2 * (float)((q[l] >> 4) + (((qh[l] >> (2 * c + 1)) & 1) ? 16 : 0)) - mm2;
            y += 64;
            q += 32;
        }
    }
}

/* ---- Q5_K x Q8_K : src/quant.c:609-621, a scalar loop in the reference: dequantise the block, then
 * sum += (tmp[j] * y.d) * q8[j] sequentially, one block sum added to the row sum.  The reference build computes
 * the products separately (vectorised) and adds them in order, i.e. no fused multiply-add; ORC_Q5_FMA = 0 is that
 * form and is pinned bit for bit against the compiled reference. ---- */
#ifndef ORC_Q5_FMA
#define ORC_Q5_FMA 0
#endif
float orc_vec_dot_q5_K_q8_K(const void *xv, const void *yv, int nb) {
    const orc_block_q5_K *x = (const orc_block_q5_K *)xv;
    const orc_block_q8_K *y = (const orc_block_q8_K *)yv;
    float sumf = 0.0f;
    float tmp[ORC_QK_K];
    for (int i = 0; i < nb; i++) {
        orc_dequantize_row_q5_K(&x[i], tmp, ORC_QK_K);
        float sum = 0.0f;
        for (int j = 0; j < ORC_QK_K; j++) {
#if ORC_Q5_FMA
            sum = fmaf(tmp[j] * y[i].d, (float)y[i].qs[j], sum);
#else
            sum = sum + tmp[j] * y[i].d * (float)y[i].qs[j];
#endif
        }
        sumf = sumf + sum;
    }
    return sumf;
}

/* ---- Q6_K dequant : src/quant.c:147-175.  y = (d*sc)*q, left to right. ---- */
void orc_dequantize_row_q6_K(const void *xv, float *y, int64_t k) {
    const orc_block_q6_K *x = (const orc_block_q6_K *)xv;
    int64_t nb = k / ORC_QK_K;
    for (int64_t i = 0; i < nb; i++) {
        float d = orc_fp16_to_fp32(x[i].d);
        for (int h = 0; h < 2; h++) {
            const uint8_t *ql = x[i].ql + 64 * h;
            const uint8_t *qh = x[i].qh + 32 * h;
            const int8_t *sc = x[i].scales + 8 * h;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int q1 = (int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                int q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                int q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                int q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                y[l] = d * (float)sc[is + 0] * (float)q1;
                y[l + 32] = d * (float)sc[is + 2] * (float)q2;
                y[l + 64] = d * (float)sc[is + 4] * (float)q3;
                y[l + 96] = d * (float)sc[is + 6] * (float)q4;
            }
            y += 128;
        }
    }
}

/* ---- Q8_K activation quantiser : src/quant.c:343-375 ---- */
void orc_quantize_row_q8_K(const float *x, void *yv, int64_t k) {
    orc_block_q8_K *y = (orc_block_q8_K *)yv;
    int64_t nb = k / ORC_QK_K;
    for (int64_t i = 0; i < nb; i++, x += ORC_QK_K) {
        float amax = 0.0f;
        for (int j = 0; j < ORC_QK_K; j++) {
            float ax = fabsf(x[j]);
            if (ax > amax) amax = ax;
        }
        if (amax == 0.0f) {
            memset(&y[i], 0, sizeof(y[i]));
            continue;
        }
        float iscale = 127.0f / amax;
        for (int j = 0; j < ORC_QK_K; j++) {
            int v = (int)roundf(iscale * x[j]); /* half away from zero */
            if (v > 127) v = 127;
            if (v < -127) v = -127;
            y[i].qs[j] = (int8_t)v;
        }
        for (int j = 0; j < 16; j++) {
            int s = 0;
            for (int l = 0; l < 16; l++) s += y[i].qs[16 * j + l];
            y[i].bsums[j] = (int16_t)s;
        }
        y[i].d = 1.0f / iscale;
    }
}

/* Horizontal sum of 8 float lanes in the order of hsum_float_8, src/quant.c:379-385:
 * r[i] = a[i] + a[i+4]; then (r0 + r2) + (r1 + r3). */
static float hsum8(const float a[8]) {
    float r0 = a[0] + a[4], r1 = a[1] + a[5], r2 = a[2] + a[6], r3 = a[3] + a[7];
    float s0 = r0 + r2, s1 = r1 + r3;
    return s0 + s1;
}

/* ---- Q4_K x Q8_K dot : src/quant.c:405-476.
 * Per block the AVX2 code keeps 8 int32 lanes: lane t holds
 *   sum_j sc_j * sum_{bytes 4t..4t+3 of sub-block j} q4*q8
 * (maddubs pairs adjacent bytes, madd pairs adjacent int16s); then
 *   acc[t]   = fma(y.d*d,      float(lane t), acc[t])
 *   acc_m[p] = fma(-y.d*dmin,  float(m_{2p}*bs_{2p} + m_{2p+1}*bs_{2p+1}), acc_m[p])
 * with bs_j = bsums[2j] + bsums[2j+1]; final hsum8(acc) + ((m0+m2)+(m1+m3)). ---- */
float orc_vec_dot_q4_K_q8_K(const void *xv, const void *yv, int nb) {
    const orc_block_q4_K *x = (const orc_block_q4_K *)xv;
    const orc_block_q8_K *y = (const orc_block_q8_K *)yv;
    float acc[8] = {0}, acc_m[4] = {0};
    for (int i = 0; i < nb; i++) {
        float d = y[i].d * orc_fp16_to_fp32(x[i].d);
        float dmin = -y[i].d * orc_fp16_to_fp32(x[i].dmin);
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; j++) scale_min_k4(j, x[i].scales, &sc[j], &mn[j]);
        for (int p = 0; p < 4; p++) {
            int32_t prod = 0;
            for (int j = 2 * p; j < 2 * p + 2; j++)
                prod += (int32_t)mn[j] * ((int32_t)y[i].bsums[2 * j] + (int32_t)y[i].bsums[2 * j + 1]);
            acc_m[p] = fmaf(dmin, (float)prod, acc_m[p]);
        }
        int32_t lane[8] = {0};
        const uint8_t *q4 = x[i].qs;
        const int8_t *q8 = y[i].qs;
        for (int c = 0; c < 4; c++, q4 += 32, q8 += 64) {
            for (int t = 0; t < 8; t++) {
                int32_t lo = 0, hi = 0;
                for (int b = 4 * t; b < 4 * t + 4; b++) {
                    lo += (int32_t)(q4[b] & 0xF) * q8[b];
                    hi += (int32_t)(q4[b] >> 4) * q8[32 + b];
                }
                lane[t] += (int32_t)sc[2 * c] * lo + (int32_t)sc[2 * c + 1] * hi;
            }
        }
        for (int t = 0; t < 8; t++) acc[t] = fmaf(d, (float)lane[t], acc[t]);
    }
    float m = (acc_m[0] + acc_m[2]) + (acc_m[1] + acc_m[3]);
    return hsum8(acc) + m;
}

/* ---- Q6_K x Q8_K dot : src/quant.c:478-607.
 * 8 int32 lanes per block; for each 32-value sub-block s (value positions
 * 128h+32i .. +31), lane t takes bytes 4t..4t+3 times scale sc[8h+2i+(t>=4)];
 * acc[t] = fma(y.d*d, float(lane t), acc[t]); final hsum8(acc). ---- */
float orc_vec_dot_q6_K_q8_K(const void *xv, const void *yv, int nb) {
    const orc_block_q6_K *x = (const orc_block_q6_K *)xv;
    const orc_block_q8_K *y = (const orc_block_q8_K *)yv;
    float acc[8] = {0};
    for (int i = 0; i < nb; i++) {
        float d = y[i].d * orc_fp16_to_fp32(x[i].d);
        int32_t lane[8] = {0};
        for (int h = 0; h < 2; h++) {
            const uint8_t *ql = x[i].ql + 64 * h;
            const uint8_t *qh = x[i].qh + 32 * h;
            const int8_t *sc = x[i].scales + 8 * h;
            const int8_t *q8 = y[i].qs + 128 * h;
            for (int s = 0; s < 4; s++) {
                for (int t = 0; t < 8; t++) {
                    int32_t p = 0;
                    for (int b = 4 * t; b < 4 * t + 4; b++) {
                        int lo = (s & 1) ? ql[b + 32] : ql[b];
                        lo = (s & 2) ? (lo >> 4) : (lo & 0xF);
                        int q6 = (lo | (((qh[b] >> (2 * s)) & 3) << 4)) - 32;
                        p += q6 * q8[32 * s + b];
                    }
                    lane[t] += p * (int32_t)sc[2 * s + (t >= 4)];
                }
            }
        }
        for (int t = 0; t < 8; t++) acc[t] = fmaf(d, (float)lane[t], acc[t]);
    }
    return hsum8(acc);
}

/* ---- fp32-activation dots: src/quant.c:109-143 (Q4_K), 249-262 (Q5_K), 177-212 (Q6_K).  One sum per block, added
 * to the row sum.  The reference build fuses `sum += w * y` into a multiply-add in the Q4_K loop and not in the
 * other two (their products are computed first, vectorised, and added in order); each form below is pinned bit for
 * bit against the compiled reference. ---- */
static inline float acc_f32(float w, float y, float sum) { return fmaf(w, y, sum); }

float orc_vec_dot_q4_K_f32(const void *xv, const float *y, int64_t n) {
    const orc_block_q4_K *x = (const orc_block_q4_K *)xv;
    int64_t nb = n / ORC_QK_K;
    float sumf = 0.0f;
    for (int64_t i = 0; i < nb; i++) {
        const uint8_t *q = x[i].qs;
        float d = orc_fp16_to_fp32(x[i].d), dmin = orc_fp16_to_fp32(x[i].dmin);
        float sum = 0.0f;
        for (int c = 0; c < 4; c++) {
            uint8_t sc1, m1, sc2, m2;
            scale_min_k4(2 * c, x[i].scales, &sc1, &m1);
            scale_min_k4(2 * c + 1, x[i].scales, &sc2, &m2);
            float d1 = d * (float)sc1, mm1 = dmin * (float)m1, d2 = d * (float)sc2, mm2 = dmin * (float)m2;
            for (int l = 0; l < 32; l++) sum = acc_f32(d1 * (float)(q[l] & 0xF) - mm1, y[64 * c + l], sum);
            for (int l = 0; l < 32; l++) sum = acc_f32(d2 * (float)(q[l] >> 4) - mm2, y[64 * c + 32 + l], sum);
            q += 32;
        }
        sumf = sumf + sum;
        y += ORC_QK_K;
    }
    return sumf;
}

float orc_vec_dot_q5_K_f32(const void *xv, const float *y, int64_t n) {
    const orc_block_q5_K *x = (const orc_block_q5_K *)xv;
    int64_t nb = n / ORC_QK_K;
    float sumf = 0.0f, tmp[ORC_QK_K];
    for (int64_t i = 0; i < nb; i++) {
        orc_dequantize_row_q5_K(&x[i], tmp, ORC_QK_K);
        float sum = 0.0f;
        for (int j = 0; j < ORC_QK_K; j++) sum = sum + tmp[j] * y[i * ORC_QK_K + j];
        sumf = sumf + sum;
    }
    return sumf;
}

float orc_vec_dot_q6_K_f32(const void *xv, const float *y, int64_t n) {
    const orc_block_q6_K *x = (const orc_block_q6_K *)xv;
    int64_t nb = n / ORC_QK_K;
    float sumf = 0.0f;
    for (int64_t i = 0; i < nb; i++) {
        float d = orc_fp16_to_fp32(x[i].d);
        float sum = 0.0f;
        for (int h = 0; h < 2; h++) {
            const uint8_t *ql = x[i].ql + 64 * h, *qh = x[i].qh + 32 * h;
            const int8_t *sc = x[i].scales + 8 * h;
            const float *yp = y + i * ORC_QK_K + 128 * h;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int8_t q1 = (int8_t)((int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32);
                int8_t q2 = (int8_t)((int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
                int8_t q3 = (int8_t)((int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
                int8_t q4 = (int8_t)((int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
                sum = sum + d * (float)sc[is + 0] * (float)q1 * yp[l];
                sum = sum + d * (float)sc[is + 2] * (float)q2 * yp[l + 32];
                sum = sum + d * (float)sc[is + 4] * (float)q3 * yp[l + 64];
                sum = sum + d * (float)sc[is + 6] * (float)q4 * yp[l + 96];
            }
        }
        sumf = sumf + sum;
    }
    return sumf;
}

/* ---- 32-value blocks on fp32 activations: Q8_0 {fp16 d; int8 qs[32]} (include/quant_types.h:41-46) and MXFP4
 * {uint8 e8m0 s; uint8 qs[16]} (48-53).  src/quant.c:266-288 and 290-337: one sum per block, `sumf += scale * sum`.
 * ORC_Q8_0_FMA / ORC_MXFP4_FMA say whether the reference build fuses the multiply-adds of these loops (it does for
 * MXFP4, whose table look-ups keep the loop scalar, and not for Q8_0, whose products are vectorised first); each
 * form is pinned bit for bit against the compiled reference by the tests. ---- */
static const float mxfp4_table[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                      -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
static float e8m0_scale(uint8_t s) { return s == 0xFF ? 0.0f : ldexpf(1.0f, (int)s - 127); }

void orc_dequantize_row_q8_0(const void *xv, float *y, int64_t k) {
    const uint8_t *x = (const uint8_t *)xv;
    for (int64_t i = 0; i < k / 32; i++) {
        uint16_t dh;
        memcpy(&dh, x + 34 * i, 2);
        const float d = orc_fp16_to_fp32(dh);
        for (int j = 0; j < 32; j++) y[32 * i + j] = d * (float)(int8_t)x[34 * i + 2 + j];
    }
}

void orc_dequantize_row_mxfp4(const void *xv, float *y, int64_t k) {
    const uint8_t *x = (const uint8_t *)xv;
    for (int64_t i = 0; i < k / 32; i++) {
        const float scale = e8m0_scale(x[17 * i]);
        for (int j = 0; j < 16; j++) {
            const uint8_t b = x[17 * i + 1 + j];
            y[32 * i + j] = mxfp4_table[b & 0x0F] * scale;
            y[32 * i + j + 16] = mxfp4_table[b >> 4] * scale;
        }
    }
}

float orc_vec_dot_q8_0_f32(const void *xv, const float *y, int64_t n) {
    const uint8_t *x = (const uint8_t *)xv;
    float sumf = 0.0f;
    for (int64_t i = 0; i < n / 32; i++) {
        uint16_t dh;
        memcpy(&dh, x + 34 * i, 2);
        const float d = orc_fp16_to_fp32(dh);
        float sum = 0.0f;
        for (int j = 0; j < 32; j++) {
            const float w = (float)(int8_t)x[34 * i + 2 + j];
#if ORC_Q8_0_FMA
            sum = fmaf(w, y[32 * i + j], sum);
#else
            sum = sum + w * y[32 * i + j];
#endif
        }
#if ORC_Q8_0_FMA
        sumf = fmaf(d, sum, sumf);
#else
        sumf = sumf + d * sum;
#endif
    }
    return sumf;
}

float orc_vec_dot_mxfp4_f32(const void *xv, const float *y, int64_t n) {
    const uint8_t *x = (const uint8_t *)xv;
    float sumf = 0.0f;
    for (int64_t i = 0; i < n / 32; i++) {
        const float scale = e8m0_scale(x[17 * i]);
        float sum = 0.0f;
        for (int j = 0; j < 16; j++) {
            const uint8_t b = x[17 * i + 1 + j];
#if ORC_MXFP4_FMA
            sum = fmaf(mxfp4_table[b & 0x0F], y[32 * i + j], sum);
            sum = fmaf(mxfp4_table[b >> 4], y[32 * i + j + 16], sum);
#else
            sum = sum + mxfp4_table[b & 0x0F] * y[32 * i + j];
            sum = sum + mxfp4_table[b >> 4] * y[32 * i + j + 16];
#endif
        }
#if ORC_MXFP4_FMA
        sumf = fmaf(scale, sum, sumf);
#else
        sumf = sumf + scale * sum;
#endif
    }
    return sumf;
}

static void matvec_f32(float *out, const void *mat, int type, const float *x, int M, int K) {
    uint64_t rb = orc_row_bytes(type, K);
    const uint8_t *m = (const uint8_t *)mat;
    for (int i = 0; i < M; i++) {
        const void *row = m + (uint64_t)i * rb;
        out[i] = type == ORC_TYPE_Q4_K ? orc_vec_dot_q4_K_f32(row, x, K)
               : type == ORC_TYPE_Q5_K ? orc_vec_dot_q5_K_f32(row, x, K)
               : type == ORC_TYPE_Q8_0 ? orc_vec_dot_q8_0_f32(row, x, K)
               : type == ORC_TYPE_MXFP4 ? orc_vec_dot_mxfp4_f32(row, x, K) : orc_vec_dot_q6_K_f32(row, x, K);
    }
}

void orc_mat_vec_mul_f32act(float *out, const void *mat, int type, const float *x, int M, int K) {
    matvec_f32(out, mat, type, x, M, K);
}

/* ---- src/inference.c:361-374: the shared expert on fp32 activations, each matrix with its own type ---- */
void orc_shared_ffn_f32(float *out, const float *h, const void *gate, int gate_type, const void *up, int up_type,
                        const void *down, int down_type, int n_embd, int inter) {
    float *g = (float *)malloc(sizeof(float) * (size_t)inter);
    float *u = (float *)malloc(sizeof(float) * (size_t)inter);
    matvec_f32(g, gate, gate_type, h, inter, n_embd);
    for (int r = 0; r < inter; r++) g[r] = g[r] / (1.0f + expf(-g[r]));
    matvec_f32(u, up, up_type, h, inter, n_embd);
    for (int r = 0; r < inter; r++) g[r] = g[r] * u[r];
    matvec_f32(out, down, down_type, g, n_embd, inter);
    free(g);
    free(u);
}

/* ---- src/inference.c:556-575 (routed experts: silu(gate) * up, down, out += score * down; the reference build
 * fuses that multiply-add) and 361-374, 582-596 (shared expert, added with weight 1) ---- */
void orc_moe_block_f32(float *out, const float *h, const void *const *experts, const float *scores, int k,
                       const void *shared_data, int gate_type, int up_type, int down_type, uint64_t gate_size,
                       uint64_t up_size, int n_embd, int inter) {
    float *g = (float *)malloc(sizeof(float) * (size_t)inter);
    float *u = (float *)malloc(sizeof(float) * (size_t)inter);
    float *dn = (float *)malloc(sizeof(float) * (size_t)n_embd);
    memset(out, 0, sizeof(float) * (size_t)n_embd);
    for (int i = 0; i <= k; i++) {
        const uint8_t *e = (const uint8_t *)(i < k ? experts[i] : shared_data);
        if (!e) break;
        matvec_f32(g, e, gate_type, h, inter, n_embd);
        for (int r = 0; r < inter; r++) g[r] = g[r] / (1.0f + expf(-g[r]));
        matvec_f32(u, e + gate_size, up_type, h, inter, n_embd);
        for (int r = 0; r < inter; r++) g[r] = g[r] * u[r];
        matvec_f32(dn, e + gate_size + up_size, down_type, g, n_embd, inter);
        if (i < k)
            for (int r = 0; r < n_embd; r++) out[r] = fmaf(scores[i], dn[r], out[r]);
        else
            for (int r = 0; r < n_embd; r++) out[r] = out[r] + dn[r];
    }
    free(g);
    free(u);
    free(dn);
}

/* ---- src/cpu_expert.c:52-72 ---- */
void orc_matvec_q8(float *out, const void *mat, int type, const void *q8, int M, int K) {
    int nb = K / ORC_QK_K;
    uint64_t rb = orc_row_bytes(type, K);
    const uint8_t *m = (const uint8_t *)mat;
    for (int i = 0; i < M; i++) {
        if (type == ORC_TYPE_Q4_K) out[i] = orc_vec_dot_q4_K_q8_K(m + (uint64_t)i * rb, q8, nb);
        else if (type == ORC_TYPE_Q5_K) out[i] = orc_vec_dot_q5_K_q8_K(m + (uint64_t)i * rb, q8, nb);
        else out[i] = orc_vec_dot_q6_K_q8_K(m + (uint64_t)i * rb, q8, nb);
    }
}

/* ---- src/cpu_expert.c:75-116.  The final accumulate `partial += score*down`
 * compiles to a fused multiply-add in the reference build (gcc contracts it);
 * ORC_ACCUM_FMA selects that form and is pinned against the compiled reference. ---- */
#ifndef ORC_ACCUM_FMA
#define ORC_ACCUM_FMA 1
#endif
void orc_expert_ffn(float *partial, const void *expert_data, const void *q8_input, float score,
                    int gate_type, int up_type, int down_type, uint64_t gate_size, uint64_t up_size,
                    int n_embd, int inter, float *act_out) {
    const uint8_t *e = (const uint8_t *)expert_data;
    float *g = (float *)malloc(sizeof(float) * (size_t)inter);
    float *u = (float *)malloc(sizeof(float) * (size_t)inter);
    float *dn = (float *)malloc(sizeof(float) * (size_t)n_embd);
    orc_block_q8_K *q8a = (orc_block_q8_K *)malloc(sizeof(orc_block_q8_K) * (size_t)(inter / ORC_QK_K));
    orc_matvec_q8(g, e, gate_type, q8_input, inter, n_embd);
    orc_matvec_q8(u, e + gate_size, up_type, q8_input, inter, n_embd);
    for (int i = 0; i < inter; i++) g[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
    if (act_out) memcpy(act_out, g, sizeof(float) * (size_t)inter);
    orc_quantize_row_q8_K(g, q8a, inter);
    orc_matvec_q8(dn, e + gate_size + up_size, down_type, q8a, n_embd, inter);
    for (int i = 0; i < n_embd; i++) {
#if ORC_ACCUM_FMA
        partial[i] = fmaf(score, dn[i], partial[i]);
#else
        partial[i] = partial[i] + score * dn[i];
#endif
    }
    free(g);
    free(u);
    free(dn);
    free(q8a);
}

/* ---- router ---- */
void orc_router_logits(float *logits, const float *w, const float *h, int n_experts, int n_embd) {
    for (int i = 0; i < n_experts; i++) {
        float sum = 0.0f;
        const float *r = w + (size_t)i * n_embd;
        for (int j = 0; j < n_embd; j++) sum = sum + r[j] * h[j];
        logits[i] = sum;
    }
}

/* ---- scalar gate of the shared expert: src/inference.c:586-590.  (inference.c is not among the reference files
 * that compile on their own, so this one function is checked by reading, not against the compiled reference.) ---- */
float orc_shared_gate(const float *h, const float *w, int n_embd) {
    float dot = 0.0f;
    for (int i = 0; i < n_embd; i++) dot = dot + h[i] * w[i];
    return 1.0f / (1.0f + expf(-dot));
}

void orc_softmax(float *x, int64_t n) {
    float mx = x[0];
    for (int64_t i = 1; i < n; i++)
        if (x[i] > mx) mx = x[i];
    float sum = 0.0f;
    for (int64_t i = 0; i < n; i++) {
        x[i] = expf(x[i] - mx);
        sum += x[i];
    }
    float inv = 1.0f / sum;
    for (int64_t i = 0; i < n; i++) x[i] *= inv;
}

/* Insertion top-k, strict '>' so ties keep the lower index; src/tensor.c:226-252. */
void orc_top_k(const float *x, int64_t n, int k, int *indices, float *values) {
    for (int i = 0; i < k; i++) {
        indices[i] = -1;
        values[i] = -1e30f;
    }
    for (int64_t j = 0; j < n; j++) {
        int pos = k;
        while (pos > 0 && x[j] > values[pos - 1]) pos--;
        if (pos < k) {
            for (int i = k - 1; i > pos; i--) {
                indices[i] = indices[i - 1];
                values[i] = values[i - 1];
            }
            indices[pos] = (int)j;
            values[pos] = x[j];
        }
    }
}

void orc_renorm(float *scores, int k) {
    float s = 0.0f;
    for (int i = 0; i < k; i++) s += scores[i];
    if (s > 0.0f) {
        float inv = 1.0f / s;
        for (int i = 0; i < k; i++) scores[i] *= inv;
    }
}

void orc_rms_norm(float *out, const float *x, const float *w, int64_t n, float eps) {
    float ss = 0.0f;
    for (int64_t i = 0; i < n; i++) ss = fmaf(x[i], x[i], ss); /* contracted in the reference build */
    ss = 1.0f / sqrtf(ss / (float)n + eps);
    for (int64_t i = 0; i < n; i++) out[i] = x[i] * ss * w[i];
}

/* ---- CAR, one residency tier.  src/car.c:36-264 with budgets off. ---- */
static int resident(const uint32_t *mask, int e) { return (mask[e >> 5] >> (e & 31)) & 1u; }

int orc_car(int *ids, float *scores, int k, const float *all_scores, int n_experts,
            const uint32_t *mask, float threshold, int dampen) {
    /* guard: src/gpu_kernels.hip:7170 (threshold > 0) and src/car.c:68 (threshold < 1) */
    if (!(threshold > 0.0f) || threshold >= 1.0f || !mask) return 0;
    int unc[64], n_unc = 0;
    for (int i = 0; i < k; i++) /* classify, ascending list position */
        if (!resident(mask, ids[i])) unc[n_unc++] = i;
    if (n_unc == 0) return 0;

    uint8_t selected[64] = {0}; /* 512 bits, src/car.c:85 */
    for (int i = 0; i < k; i++) selected[ids[i] >> 3] |= (uint8_t)(1 << (ids[i] & 7));

    struct cand {
        int idx, best;
        float best_score, ratio;
    } c[16];
    int nc = 0;
    for (int u = 0; u < n_unc; u++) {
        int idx = unc[u];
        float orig = all_scores[ids[idx]];
        int best = -1;
        float best_score = 0.0f;
        for (int e = 0; e < n_experts; e++) {
            if (selected[e >> 3] & (1 << (e & 7))) continue;
            if (all_scores[e] <= best_score) continue;
            if (resident(mask, e)) {
                best = e;
                best_score = all_scores[e];
            }
        }
        float ratio = (orig > 0.0f) ? best_score / orig : 0.0f;
        if (best >= 0 && ratio >= threshold) {
            c[nc].idx = idx;
            c[nc].best = best;
            c[nc].best_score = best_score;
            c[nc].ratio = ratio;
            nc++;
            selected[best >> 3] |= (uint8_t)(1 << (best & 7)); /* reserved at once */
        }
    }
    for (int i = 1; i < nc; i++) { /* stable insertion sort, ratio descending */
        struct cand t = c[i];
        int j = i - 1;
        while (j >= 0 && c[j].ratio < t.ratio) {
            c[j + 1] = c[j];
            j--;
        }
        c[j + 1] = t;
    }
    for (int i = 0; i < nc; i++) {
        ids[c[i].idx] = c[i].best;
        scores[c[i].idx] = dampen ? scores[c[i].idx] * c[i].ratio : c[i].best_score;
    }
    if (nc > 0 && !dampen) orc_renorm(scores, k);
    return nc;
}

int orc_route(const float *router_w, const float *h, int n_experts, int n_embd, int k,
              const uint32_t *mask, float threshold, int dampen, float *all_scores, int *ids,
              float *scores) {
    orc_router_logits(all_scores, router_w, h, n_experts, n_embd);
    orc_softmax(all_scores, n_experts);
    orc_top_k(all_scores, n_experts, k, ids, scores);
    orc_renorm(scores, k);
    return orc_car(ids, scores, k, all_scores, n_experts, mask, threshold, dampen);
}

void orc_moe_block(float *out, const float *h, const void *const *experts, const float *scores, int k,
                   const void *shared_data, int gate_type, int up_type, int down_type,
                   uint64_t gate_size, uint64_t up_size, int n_embd, int inter) {
    orc_block_q8_K *q8 = (orc_block_q8_K *)malloc(sizeof(orc_block_q8_K) * (size_t)(n_embd / ORC_QK_K));
    orc_quantize_row_q8_K(h, q8, n_embd);
    memset(out, 0, sizeof(float) * (size_t)n_embd);
    for (int i = 0; i < k; i++)
        orc_expert_ffn(out, experts[i], q8, scores[i], gate_type, up_type, down_type, gate_size, up_size,
                       n_embd, inter, NULL);
    if (shared_data) { /* shared expert: own accumulator, weight 1, added after (src/inference.c:595) */
        float *sh = (float *)calloc((size_t)n_embd, sizeof(float));
        orc_expert_ffn(sh, shared_data, q8, 1.0f, gate_type, up_type, down_type, gate_size, up_size,
                       n_embd, inter, NULL);
        for (int i = 0; i < n_embd; i++) out[i] = out[i] + sh[i];
        free(sh);
    }
    free(q8);
}
