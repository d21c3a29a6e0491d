/*
 * synth_host.c -- the seeded synthetic-input generator of synth.h as a small host-only library
 * (libfomoe_synth.so, plain C, no CUDA).  It produces the same bytes as the device generator that
 * fills the expert table and as fomoe_b200_synth_matrix / fomoe_b200_synth_f32 of the main library;
 * programs that must not load the CUDA library (the CPU arm of the benchmark) take their inputs here.
 */
#include <stdint.h>
#include <string.h>

#include "layout.h"
#include "synth.h"

void fomoe_synth_matrix(uint64_t seed, int layer, int expert, int matrix, int type, int rows, int cols, void *out) {
    const uint64_t key = fsyn_key(seed, (uint32_t)layer, (uint32_t)expert, (uint32_t)matrix);
    const uint64_t nblk = (uint64_t)rows * (uint64_t)(cols / FB_QK);
    uint8_t *o = (uint8_t *)out;
    for (uint64_t b = 0; b < nblk; b++) {
        if (type == FB_TYPE_Q4_K) {
            uint32_t w[36];
            fsyn_q4k_block(key, b, w);
            memcpy(o + b * FB_Q4K_BLOCK, w, FB_Q4K_BLOCK);
        } else if (type == FB_TYPE_Q5_K) {
            uint32_t w[44];
            fsyn_q5k_block(key, b, w);
            memcpy(o + b * FB_Q5K_BLOCK, w, FB_Q5K_BLOCK);
        } else {
            uint32_t ql[32], qh[16], sc[4];
            uint16_t d;
            fsyn_q6k_block(key, b, ql, qh, sc, &d);
            uint8_t *p = o + b * FB_Q6K_BLOCK;
            memcpy(p, ql, 128);
            memcpy(p + 128, qh, 64);
            memcpy(p + 192, sc, 16);
            memcpy(p + 208, &d, 2);
        }
    }
}

void fomoe_synth_f32(uint64_t seed, int layer, int stream_id, float mean, float std, uint64_t n, float *out) {
    const uint64_t key = fsyn_key(seed, (uint32_t)layer, 0, (uint32_t)stream_id);
    for (uint64_t i = 0; i < n; i++) out[i] = fsyn_f32(key, i, mean, std);
}
