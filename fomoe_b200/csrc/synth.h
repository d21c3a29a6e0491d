/*
 * synth.h -- counter-based synthetic weight generator, identical on host and device.
 *
 * The 397B-shape expert table is 234 GB; it cannot cross PCIe for every run, so it is
 * generated on the GPU from a hash of (seed, layer, expert, matrix, block, word).  The
 * host regenerates only the experts a parity check touches.  Every value is produced by
 * integer arithmetic plus at most one IEEE fp32 multiply, so host and device agree bit
 * for bit without relying on libm.
 *
 * Distributions follow the benchmark's synthetic-input description:
 *   Q4_K block: d, dmin = fp16(|z| * 1e-3); the 12 scale bytes and 128 nibble bytes are raw
 *               hash bytes (uniform 6-bit scales/mins, uniform nibbles).
 *   Q5_K block: as Q4_K, the 32 bytes of fifth bits raw hash bytes as well.
 *   Q6_K block: ql, qh raw hash bytes; scales = (byte & 63) - 32; d = fp16(|z| * 1e-3).
 *   fp32 streams (router, hidden, residual, norm weight): mean + std * z.
 * z is an 8-term Irwin-Hall variate (sum of eight 16-bit uniforms, centred and scaled to
 * unit variance): a close stand-in for N(0,1) with support +-4.9 sigma.
 */
#ifndef FOMOE_B200_SYNTH_H
#define FOMOE_B200_SYNTH_H

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define FSYN_HD __host__ __device__ __forceinline__
#else
#define FSYN_HD static inline
#endif

/* matrix / stream selectors */
#define FSYN_M_GATE 0u
#define FSYN_M_UP 1u
#define FSYN_M_DOWN 2u
#define FSYN_M_ROUTER 3u
#define FSYN_M_RESID 4u
#define FSYN_M_NORMW 5u
#define FSYN_M_HIDDEN 6u
#define FSYN_M_SHGATE 7u

FSYN_HD uint64_t fsyn_mix(uint64_t z) {
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

/* One key per (seed, layer, expert, matrix) stream. */
FSYN_HD uint64_t fsyn_key(uint64_t seed, uint32_t layer, uint32_t expert, uint32_t matrix) {
    uint64_t k = fsyn_mix(seed + 0x9E3779B97F4A7C15ull);
    k = fsyn_mix(k ^ ((uint64_t)layer << 40) ^ ((uint64_t)expert << 8) ^ (uint64_t)matrix);
    return k;
}

FSYN_HD uint64_t fsyn_word(uint64_t key, uint64_t idx) {
    return fsyn_mix(key + (idx + 1) * 0x9E3779B97F4A7C15ull);
}

/* 8-term Irwin-Hall variate, unit variance.  sum of 8 u16 has variance 8*(65536^2)/12. */
FSYN_HD float fsyn_normal(uint64_t a, uint64_t b) {
    uint32_t s = (uint32_t)(a & 0xFFFF) + (uint32_t)((a >> 16) & 0xFFFF) + (uint32_t)((a >> 32) & 0xFFFF) +
                 (uint32_t)(a >> 48) + (uint32_t)(b & 0xFFFF) + (uint32_t)((b >> 16) & 0xFFFF) +
                 (uint32_t)((b >> 32) & 0xFFFF) + (uint32_t)(b >> 48);
    int32_t c = (int32_t)s - 4 * 65535; /* exact, |c| < 2^19 */
    return (float)c * 1.86880e-5f;      /* 1 / (65536 * sqrt(8/12)) */
}

/* IEEE fp32 -> fp16, round to nearest even, for finite non-negative inputs below 65504. */
FSYN_HD uint16_t fsyn_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t e = (x >> 23) & 0xFF, m = x & 0x7FFFFF;
    if (e >= 113) { /* normal half */
        uint32_t h = ((e - 112) << 10) | (m >> 13);
        uint32_t rem = m & 0x1FFF;
        if (rem > 0x1000 || (rem == 0x1000 && (h & 1))) h++;
        return (uint16_t)h;
    }
    if (e < 102) return 0; /* below half of the smallest subnormal */
    m |= 0x800000;         /* subnormal half: value = m * 2^(e-150), unit 2^-24 */
    uint32_t shift = 126 - e; /* 14..24 */
    uint32_t h = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) h++;
    return (uint16_t)h;
}

FSYN_HD uint16_t fsyn_scale_f16(uint64_t key, uint64_t widx) {
    float z = fsyn_normal(fsyn_word(key, widx), fsyn_word(key, widx + 1));
    if (z < 0.0f) z = -z;
    return fsyn_f32_to_f16(z * 1.0e-3f);
}

/* Words consumed per block: Q4_K 22 (0-3 d/dmin, 4-5 scales, 6-21 qs); Q6_K 28
 * (0-15 ql, 16-23 qh, 24-25 scales, 26-27 d). */
#define FSYN_Q4K_WORDS 22u
#define FSYN_Q6K_WORDS 28u
#define FSYN_Q5K_WORDS 26u /* 0-3 d/dmin, 4-5 scales, 6-9 qh, 10-25 qs */

/* Writes block `blk` of the stream `key` in ggml Q4_K byte order (144 B) as 36 u32. */
FSYN_HD void fsyn_q4k_block(uint64_t key, uint64_t blk, uint32_t out[36]) {
    uint64_t base = blk * FSYN_Q4K_WORDS;
    uint32_t d = fsyn_scale_f16(key, base + 0), dmin = fsyn_scale_f16(key, base + 2);
    out[0] = d | (dmin << 16);
    uint64_t s0 = fsyn_word(key, base + 4), s1 = fsyn_word(key, base + 5);
    out[1] = (uint32_t)s0;
    out[2] = (uint32_t)(s0 >> 32);
    out[3] = (uint32_t)s1;
    for (int i = 0; i < 16; i++) {
        uint64_t w = fsyn_word(key, base + 6 + i);
        out[4 + 2 * i] = (uint32_t)w;
        out[5 + 2 * i] = (uint32_t)(w >> 32);
    }
}

/* Writes block `blk` in ggml Q5_K byte order (176 B) as 44 u32: d|dmin, scales[12], qh[32], qs[128]. */
FSYN_HD void fsyn_q5k_block(uint64_t key, uint64_t blk, uint32_t out[44]) {
    uint64_t base = blk * FSYN_Q5K_WORDS;
    uint32_t d = fsyn_scale_f16(key, base + 0), dmin = fsyn_scale_f16(key, base + 2);
    out[0] = d | (dmin << 16);
    uint64_t s0 = fsyn_word(key, base + 4), s1 = fsyn_word(key, base + 5);
    out[1] = (uint32_t)s0;
    out[2] = (uint32_t)(s0 >> 32);
    out[3] = (uint32_t)s1;
    for (int i = 0; i < 20; i++) {
        uint64_t w = fsyn_word(key, base + 6 + i);
        out[4 + 2 * i] = (uint32_t)w;
        out[5 + 2 * i] = (uint32_t)(w >> 32);
    }
}

/* Writes block `blk` in ggml Q6_K byte order (210 B): ql u32[32], qh u32[16], scales u32[4], d u16. */
FSYN_HD void fsyn_q6k_block(uint64_t key, uint64_t blk, uint32_t ql[32], uint32_t qh[16], uint32_t sc[4],
                            uint16_t *d) {
    uint64_t base = blk * FSYN_Q6K_WORDS;
    for (int i = 0; i < 16; i++) {
        uint64_t w = fsyn_word(key, base + i);
        ql[2 * i] = (uint32_t)w;
        ql[2 * i + 1] = (uint32_t)(w >> 32);
    }
    for (int i = 0; i < 8; i++) {
        uint64_t w = fsyn_word(key, base + 16 + i);
        qh[2 * i] = (uint32_t)w;
        qh[2 * i + 1] = (uint32_t)(w >> 32);
    }
    for (int i = 0; i < 2; i++) {
        uint64_t w = fsyn_word(key, base + 24 + i);
        /* per byte: (b & 63) - 32 as int8 == (b & 63) ^ 0x20 sign-extended from bit 5 */
        uint64_t v = w & 0x3F3F3F3F3F3F3F3Full;
        uint64_t neg = (~v) & 0x2020202020202020ull; /* bytes with value < 32 become negative */
        v = (v ^ 0x2020202020202020ull) | (neg << 1) | (neg << 2);
        sc[2 * i] = (uint32_t)v;
        sc[2 * i + 1] = (uint32_t)(v >> 32);
    }
    *d = fsyn_scale_f16(key, base + 26);
}

/* fp32 stream element i: mean + std * z. */
FSYN_HD float fsyn_f32(uint64_t key, uint64_t i, float mean, float std) {
    float z = fsyn_normal(fsyn_word(key, 2 * i), fsyn_word(key, 2 * i + 1));
    return fmaf(std, z, mean); /* explicit FMA: same rounding on host and device */
}

#endif
