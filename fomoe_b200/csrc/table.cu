/*
 * table.cu -- building and inspecting the HBM-resident expert table.
 *
 * The table replaces the reference's three storage tiers (VRAM LRU, pinned-DRAM LRU, NVMe
 * store: src/expert_cache.c, src/expert_store.c, src/nvme_io.c): every expert of every
 * layer lives in device memory in the lane-striped layout of layout.h, already cut to this
 * rank's tensor-parallel shard.  Kernels here
 *   - generate synthetic experts straight into that layout (synth.h),
 *   - repack ggml-ordered bytes (what the reference's .qmoe records and gpu_expert_ffn
 *     buffers hold) into it, and export it back,
 *   - dequantise a shard to fp32 (bit-exact against src/quant.c:82-105 / 147-175),
 *   - run a single dequant-matvec for the microbenchmark.
 */
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "dots.cuh"
#include "launch.h"
#include "synth.h"

/* local block index -> (group, lane) and the block's index in the full matrix */
__device__ __forceinline__ uint64_t full_block_index(const fb_shard_geom_t &g, int lb) {
    const int lr = lb / g.bpr_local, lc = lb - lr * g.bpr_local;
    return (uint64_t)(g.row0 + lr) * g.bpr_full + (g.b0 + lc);
}

__device__ __forceinline__ void store_q4k(uint8_t *shard, int lb, const uint32_t w[36]) {
    uint4 *grp = reinterpret_cast<uint4 *>(shard + (uint64_t)(lb >> 5) * FB_Q4K_GROUP) + (lb & 31);
#pragma unroll
    for (int k = 0; k < 9; k++) grp[32 * k] = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
}

__device__ __forceinline__ void store_q5k(uint8_t *shard, int lb, const uint32_t w[44]) {
    uint4 *grp = reinterpret_cast<uint4 *>(shard + (uint64_t)(lb >> 5) * FB_Q5K_GROUP) + (lb & 31);
#pragma unroll
    for (int k = 0; k < 11; k++) grp[32 * k] = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
}

__device__ __forceinline__ void store_q6k(uint8_t *shard, int lb, const uint32_t ql[32], const uint32_t qh[16],
                                          const uint32_t sc[4], uint16_t d) {
    uint8_t *gb = shard + (uint64_t)(lb >> 5) * FB_Q6K_GROUP;
    uint4 *grp = reinterpret_cast<uint4 *>(gb) + (lb & 31);
#pragma unroll
    for (int k = 0; k < 8; k++) grp[32 * k] = make_uint4(ql[4 * k], ql[4 * k + 1], ql[4 * k + 2], ql[4 * k + 3]);
#pragma unroll
    for (int k = 0; k < 4; k++)
        grp[32 * (8 + k)] = make_uint4(qh[4 * k], qh[4 * k + 1], qh[4 * k + 2], qh[4 * k + 3]);
    grp[32 * 12] = make_uint4(sc[0], sc[1], sc[2], sc[3]);
    reinterpret_cast<uint16_t *>(gb + FB_Q6K_OFF_D)[lb & 31] = d;
}

/* half super-blocks: w / ql, qh, sc, d are the WHOLE block as generated or read; only half `h` is kept */
__device__ __forceinline__ void store_q4k_half(uint8_t *shard, int lb, const uint32_t w[36], int h) {
    uint4 *grp = reinterpret_cast<uint4 *>(shard + (uint64_t)(lb >> 5) * FB_Q4K_HGROUP) + (lb & 31);
    grp[0] = make_uint4(w[0], w[1], w[2], w[3]);
    const uint32_t *q = w + 4 + 16 * h;
#pragma unroll
    for (int k = 0; k < 4; k++) grp[32 * (k + 1)] = make_uint4(q[4 * k], q[4 * k + 1], q[4 * k + 2], q[4 * k + 3]);
}

__device__ __forceinline__ void store_q5k_half(uint8_t *shard, int lb, const uint32_t w[44], int h) {
    uint4 *grp = reinterpret_cast<uint4 *>(shard + (uint64_t)(lb >> 5) * FB_Q5K_HGROUP) + (lb & 31);
    grp[0] = make_uint4(w[0], w[1], w[2], w[3]);
    grp[32] = make_uint4(w[4], w[5], w[6], w[7]);     /* the fifth-bit field stays whole */
    grp[64] = make_uint4(w[8], w[9], w[10], w[11]);
    const uint32_t *q = w + 12 + 16 * h;
#pragma unroll
    for (int k = 0; k < 4; k++) grp[32 * (k + 3)] = make_uint4(q[4 * k], q[4 * k + 1], q[4 * k + 2], q[4 * k + 3]);
}

__device__ __forceinline__ void store_q6k_half(uint8_t *shard, int lb, const uint32_t ql[32], const uint32_t qh[16],
                                               const uint32_t sc[4], uint16_t d, int h) {
    uint8_t *gb = shard + (uint64_t)(lb >> 5) * FB_Q6K_HGROUP;
    uint4 *grp = reinterpret_cast<uint4 *>(gb) + (lb & 31);
    const uint32_t *l = ql + 16 * h, *q = qh + 8 * h;
#pragma unroll
    for (int k = 0; k < 4; k++) grp[32 * k] = make_uint4(l[4 * k], l[4 * k + 1], l[4 * k + 2], l[4 * k + 3]);
#pragma unroll
    for (int k = 0; k < 2; k++) grp[32 * (4 + k)] = make_uint4(q[4 * k], q[4 * k + 1], q[4 * k + 2], q[4 * k + 3]);
    reinterpret_cast<uint2 *>(gb + FB_Q6K_HOFF_SC)[lb & 31] = make_uint2(sc[2 * h], sc[2 * h + 1]);
    reinterpret_cast<uint16_t *>(gb + FB_Q6K_HOFF_D)[lb & 31] = d;
}

__global__ void k_gen_shards(uint8_t *dst0, uint64_t rec_stride, uint64_t seed, uint32_t layer, uint32_t matrix,
                             fb_shard_geom_t g) {
    const int n_local = g.rows_local * g.bpr_local;
    const int n_pad = (int)fb_n_groups(n_local) * 32;
    const uint32_t e = blockIdx.y;
    uint8_t *shard = dst0 + (uint64_t)e * rec_stride;
    const uint64_t key = fsyn_key(seed, layer, e, matrix);
    for (int lb = blockIdx.x * blockDim.x + threadIdx.x; lb < n_pad; lb += gridDim.x * blockDim.x) {
        if (g.type == FB_TYPE_Q4_K) {
            uint32_t w[36];
            if (lb < n_local) fsyn_q4k_block(key, full_block_index(g, lb), w);
            else
                for (int i = 0; i < 36; i++) w[i] = 0;
            if (g.half >= 0) store_q4k_half(shard, lb, w, g.half);
            else store_q4k(shard, lb, w);
        } else if (g.type == FB_TYPE_Q5_K) {
            uint32_t w[44];
            if (lb < n_local) fsyn_q5k_block(key, full_block_index(g, lb), w);
            else
                for (int i = 0; i < 44; i++) w[i] = 0;
            if (g.half >= 0) store_q5k_half(shard, lb, w, g.half);
            else store_q5k(shard, lb, w);
        } else {
            uint32_t ql[32], qh[16], sc[4];
            uint16_t d = 0;
            if (lb < n_local) fsyn_q6k_block(key, full_block_index(g, lb), ql, qh, sc, &d);
            else {
                for (int i = 0; i < 32; i++) ql[i] = 0;
                for (int i = 0; i < 16; i++) qh[i] = 0;
                for (int i = 0; i < 4; i++) sc[i] = 0;
            }
            if (g.half >= 0) store_q6k_half(shard, lb, ql, qh, sc, d, g.half);
            else store_q6k(shard, lb, ql, qh, sc, d);
        }
    }
}

__global__ void k_gen_f32(float *dst, uint64_t n, uint64_t key, float mean, float std) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        dst[i] = fsyn_f32(key, i, mean, std);
}

/* ggml bytes of the full matrix -> shard.  Q4_K and Q5_K blocks are 16-byte aligned in ggml order;
 * Q6_K blocks (210 B) are only 2-byte aligned, so they are read as 16-bit pieces. */
__global__ void k_repack(uint8_t *shard, const uint8_t *src, fb_shard_geom_t g) {
    const int n_local = g.rows_local * g.bpr_local;
    const int n_pad = (int)fb_n_groups(n_local) * 32;
    for (int lb = blockIdx.x * blockDim.x + threadIdx.x; lb < n_pad; lb += gridDim.x * blockDim.x) {
        if (g.type == FB_TYPE_Q4_K) {
            uint32_t w[36];
            if (lb < n_local) {
                const uint32_t *s = reinterpret_cast<const uint32_t *>(src + full_block_index(g, lb) * FB_Q4K_BLOCK);
                for (int i = 0; i < 36; i++) w[i] = s[i];
            } else
                for (int i = 0; i < 36; i++) w[i] = 0;
            if (g.half >= 0) store_q4k_half(shard, lb, w, g.half);
            else store_q4k(shard, lb, w);
        } else if (g.type == FB_TYPE_Q5_K) {
            uint32_t w[44];
            if (lb < n_local) {
                const uint32_t *s = reinterpret_cast<const uint32_t *>(src + full_block_index(g, lb) * FB_Q5K_BLOCK);
                for (int i = 0; i < 44; i++) w[i] = s[i];
            } else
                for (int i = 0; i < 44; i++) w[i] = 0;
            if (g.half >= 0) store_q5k_half(shard, lb, w, g.half);
            else store_q5k(shard, lb, w);
        } else {
            uint32_t w[52];
            uint16_t d = 0;
            if (lb < n_local) {
                const uint16_t *s = reinterpret_cast<const uint16_t *>(src + full_block_index(g, lb) * FB_Q6K_BLOCK);
                for (int i = 0; i < 52; i++) w[i] = (uint32_t)s[2 * i] | ((uint32_t)s[2 * i + 1] << 16);
                d = s[104];
            } else
                for (int i = 0; i < 52; i++) w[i] = 0;
            if (g.half >= 0) store_q6k_half(shard, lb, w, w + 32, w + 48, d, g.half);
            else store_q6k(shard, lb, w, w + 32, w + 48, d);
        }
    }
}

/* shard -> ggml bytes of the shard's own blocks, row-major */
__global__ void k_export_ggml(uint8_t *dst, const uint8_t *shard, fb_shard_geom_t g) {
    const int n_local = g.rows_local * g.bpr_local;
    for (int lb = blockIdx.x * blockDim.x + threadIdx.x; lb < n_local; lb += gridDim.x * blockDim.x) {
        if (g.type == FB_TYPE_Q4_K) {
            const uint4 *grp = reinterpret_cast<const uint4 *>(shard + (uint64_t)(lb >> 5) * FB_Q4K_GROUP) + (lb & 31);
            uint4 *o = reinterpret_cast<uint4 *>(dst + (uint64_t)lb * FB_Q4K_BLOCK);
            for (int k = 0; k < 9; k++) o[k] = grp[32 * k];
        } else if (g.type == FB_TYPE_Q5_K) {
            const uint4 *grp = reinterpret_cast<const uint4 *>(shard + (uint64_t)(lb >> 5) * FB_Q5K_GROUP) + (lb & 31);
            uint4 *o = reinterpret_cast<uint4 *>(dst + (uint64_t)lb * FB_Q5K_BLOCK);
            for (int k = 0; k < 11; k++) o[k] = grp[32 * k];
        } else {
            const uint8_t *gb = shard + (uint64_t)(lb >> 5) * FB_Q6K_GROUP;
            const uint4 *grp = reinterpret_cast<const uint4 *>(gb) + (lb & 31);
            uint16_t *o = reinterpret_cast<uint16_t *>(dst + (uint64_t)lb * FB_Q6K_BLOCK);
            for (int k = 0; k < 13; k++) {
                const uint4 v = grp[32 * k];
                const uint32_t c[4] = {v.x, v.y, v.z, v.w};
                for (int i = 0; i < 4; i++) {
                    o[8 * k + 2 * i] = (uint16_t)(c[i] & 0xffff);
                    o[8 * k + 2 * i + 1] = (uint16_t)(c[i] >> 16);
                }
            }
            o[104] = reinterpret_cast<const uint16_t *>(gb + FB_Q6K_OFF_D)[lb & 31];
        }
    }
}

/* one half super-block (layout.h) -> 128 fp32 values: the arithmetic of the whole-block kernel below restricted to
 * chunks 2h, 2h+1 (Q4_K) / half h (Q6_K).  Kept out of line on purpose: inlined into k_dequant, nvcc 12.9 produced a
 * whole-block Q6_K path whose values were exactly twice the right ones (the bit-exact dequant test caught it). */
__device__ __noinline__ void dequant_half_block(float *dst, const uint8_t *shard, int type, int half, int lb) {
        /* half super-blocks: 128 values per block, the arithmetic of the whole-block branches below restricted to
         * chunks 2h, 2h+1 (Q4_K) / half h (Q6_K) */
        const int h = half;
        float *y = dst + (uint64_t)lb * (FB_QK / 2);
        if (type == FB_TYPE_Q4_K) {
            const uint4 *grp = reinterpret_cast<const uint4 *>(shard + (uint64_t)(lb >> 5) * FB_Q4K_HGROUP) + (lb & 31);
            const uint4 hdr = grp[0];
            const float d = fb_half_bits_to_float(hdr.x & 0xffff), mn = fb_half_bits_to_float(hdr.x >> 16);
            const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
            const uint32_t scw = h ? ((u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4)) : (u0 & 0x3f3f3f3fu);
            const uint32_t mw = h ? (((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4)) : (u1 & 0x3f3f3f3fu);
            for (int cc = 0; cc < 2; cc++) {
                const float d1 = __fmul_rn(d, (float)((scw >> (16 * cc)) & 0xff));
                const float d2 = __fmul_rn(d, (float)((scw >> (16 * cc + 8)) & 0xff));
                const float m1 = __fmul_rn(mn, (float)((mw >> (16 * cc)) & 0xff));
                const float m2 = __fmul_rn(mn, (float)((mw >> (16 * cc + 8)) & 0xff));
                for (int kk = 0; kk < 2; kk++) {
                    const uint4 v = grp[32 * (1 + 2 * cc + kk)];
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                    for (int i = 0; i < 16; i++) {
                        const uint32_t byte = (w[i >> 2] >> (8 * (i & 3))) & 0xff;
                        y[64 * cc + 16 * kk + i] = __fsub_rn(__fmul_rn(d1, (float)(byte & 0xf)), m1);
                        y[64 * cc + 32 + 16 * kk + i] = __fsub_rn(__fmul_rn(d2, (float)(byte >> 4)), m2);
                    }
                }
            }
        } else if (type == FB_TYPE_Q5_K) { /* src/quant.c:216-247 restricted to chunks 2h, 2h+1 */
            const uint4 *grp = reinterpret_cast<const uint4 *>(shard + (uint64_t)(lb >> 5) * FB_Q5K_HGROUP) + (lb & 31);
            const uint4 hdr = grp[0];
            const float d = fb_half_bits_to_float(hdr.x & 0xffff), mn = fb_half_bits_to_float(hdr.x >> 16);
            const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
            const uint32_t scw = h ? ((u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4)) : (u0 & 0x3f3f3f3fu);
            const uint32_t mw = h ? (((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4)) : (u1 & 0x3f3f3f3fu);
            for (int cc = 0; cc < 2; cc++) {
                const int c = 2 * h + cc; /* chunk of the whole block: its fifth bits are bits 2c and 2c+1 */
                const float d1 = __fmul_rn(d, (float)((scw >> (16 * cc)) & 0xff));
                const float d2 = __fmul_rn(d, (float)((scw >> (16 * cc + 8)) & 0xff));
                const float m1 = __fmul_rn(mn, (float)((mw >> (16 * cc)) & 0xff));
                const float m2 = __fmul_rn(mn, (float)((mw >> (16 * cc + 8)) & 0xff));
                for (int kk = 0; kk < 2; kk++) {
                    const uint4 v = grp[32 * (3 + 2 * cc + kk)], hv = grp[32 * (1 + kk)];
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w}, hw[4] = {hv.x, hv.y, hv.z, hv.w};
                    for (int i = 0; i < 16; i++) {
                        const uint32_t byte = (w[i >> 2] >> (8 * (i & 3))) & 0xff;
                        const uint32_t hb = (hw[i >> 2] >> (8 * (i & 3))) & 0xff;
                        const uint32_t q1 = (byte & 0xf) + (((hb >> (2 * c)) & 1u) << 4);
                        const uint32_t q2 = (byte >> 4) + (((hb >> (2 * c + 1)) & 1u) << 4);
                        y[64 * cc + 16 * kk + i] = __fsub_rn(__fmul_rn(d1, (float)q1), m1);
                        y[64 * cc + 32 + 16 * kk + i] = __fsub_rn(__fmul_rn(d2, (float)q2), m2);
                    }
                }
            }
        } else {
            const uint8_t *gb = shard + (uint64_t)(lb >> 5) * FB_Q6K_HGROUP;
            const uint4 *grp = reinterpret_cast<const uint4 *>(gb) + (lb & 31);
            const float d = fb_half_bits_to_float(reinterpret_cast<const uint16_t *>(gb + FB_Q6K_HOFF_D)[lb & 31]);
            const uint2 scv = reinterpret_cast<const uint2 *>(gb + FB_Q6K_HOFF_SC)[lb & 31];
            const uint32_t scw[2] = {scv.x, scv.y};
            for (int l = 0; l < 32; l++) {
                auto byte_at = [&](int plane_first, int byte) -> uint32_t {
                    const uint4 v = grp[32 * (plane_first + (byte >> 4))];
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                    return (w[(byte & 15) >> 2] >> (8 * (byte & 3))) & 0xff;
                };
                const uint32_t a = byte_at(0, l), b = byte_at(0, 32 + l), hh = byte_at(4, l);
                const int is = l / 16;
                const int q1 = (int)((a & 0xf) | (((hh >> 0) & 3) << 4)) - 32;
                const int q2 = (int)((b & 0xf) | (((hh >> 2) & 3) << 4)) - 32;
                const int q3 = (int)((a >> 4) | (((hh >> 4) & 3) << 4)) - 32;
                const int q4 = (int)((b >> 4) | (((hh >> 6) & 3) << 4)) - 32;
                auto scale = [&](int idx) -> float {
                    return (float)(int)(signed char)((scw[idx >> 2] >> (8 * (idx & 3))) & 0xff);
                };
                y[l] = __fmul_rn(__fmul_rn(d, scale(is + 0)), (float)q1);
                y[l + 32] = __fmul_rn(__fmul_rn(d, scale(is + 2)), (float)q2);
                y[l + 64] = __fmul_rn(__fmul_rn(d, scale(is + 4)), (float)q3);
                y[l + 96] = __fmul_rn(__fmul_rn(d, scale(is + 6)), (float)q4);
            }
        }
}

/* shard -> fp32, one thread per block; arithmetic of src/quant.c:82-105 and 147-175 */
__global__ void k_dequant(float *dst, const uint8_t *shard, fb_shard_geom_t g) {
    const int n_local = g.rows_local * g.bpr_local;
    for (int lb = blockIdx.x * blockDim.x + threadIdx.x; lb < n_local; lb += gridDim.x * blockDim.x) {
        if (g.half >= 0) {
            dequant_half_block(dst, shard, g.type, g.half, lb);
            continue;
        }
        float *y = dst + (uint64_t)lb * FB_QK; /* row-major: block lb covers row lb/bpr, columns 256*(lb%bpr).. */
        if (g.type == FB_TYPE_Q4_K) {
            const uint4 *grp = reinterpret_cast<const uint4 *>(shard + (uint64_t)(lb >> 5) * FB_Q4K_GROUP) + (lb & 31);
            const uint4 hdr = grp[0];
            const float d = fb_half_bits_to_float(hdr.x & 0xffff), mn = fb_half_bits_to_float(hdr.x >> 16);
            const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
            const uint32_t sc_lo = u0 & 0x3f3f3f3fu, sc_hi = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
            const uint32_t m_lo = u1 & 0x3f3f3f3fu, m_hi = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
            for (int c = 0; c < 4; c++) {
                const uint32_t scw = c < 2 ? sc_lo : sc_hi, mw = c < 2 ? m_lo : m_hi;
                const float d1 = __fmul_rn(d, (float)((scw >> (16 * (c & 1))) & 0xff));
                const float d2 = __fmul_rn(d, (float)((scw >> (16 * (c & 1) + 8)) & 0xff));
                const float m1 = __fmul_rn(mn, (float)((mw >> (16 * (c & 1))) & 0xff));
                const float m2 = __fmul_rn(mn, (float)((mw >> (16 * (c & 1) + 8)) & 0xff));
                for (int kk = 0; kk < 2; kk++) {
                    const uint4 v = grp[32 * (1 + 2 * c + kk)];
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                    for (int i = 0; i < 16; i++) {
                        const uint32_t byte = (w[i >> 2] >> (8 * (i & 3))) & 0xff;
                        y[64 * c + 16 * kk + i] = __fsub_rn(__fmul_rn(d1, (float)(byte & 0xf)), m1);
                        y[64 * c + 32 + 16 * kk + i] = __fsub_rn(__fmul_rn(d2, (float)(byte >> 4)), m2);
                    }
                }
            }
        } else if (g.type == FB_TYPE_Q5_K) { /* src/quant.c:216-247: the nibble plus 16 where the fifth bit is set */
            const uint4 *grp = reinterpret_cast<const uint4 *>(shard + (uint64_t)(lb >> 5) * FB_Q5K_GROUP) + (lb & 31);
            const uint4 hdr = grp[0];
            const float d = fb_half_bits_to_float(hdr.x & 0xffff), mn = fb_half_bits_to_float(hdr.x >> 16);
            const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
            const uint32_t sc_lo = u0 & 0x3f3f3f3fu, sc_hi = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
            const uint32_t m_lo = u1 & 0x3f3f3f3fu, m_hi = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
            const uint4 h0 = grp[32], h1 = grp[64];
            const uint32_t hb[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w}; /* qh bytes 0..31 */
            for (int c = 0; c < 4; c++) {
                const uint32_t scw = c < 2 ? sc_lo : sc_hi, mw = c < 2 ? m_lo : m_hi;
                const float d1 = __fmul_rn(d, (float)((scw >> (16 * (c & 1))) & 0xff));
                const float d2 = __fmul_rn(d, (float)((scw >> (16 * (c & 1) + 8)) & 0xff));
                const float m1 = __fmul_rn(mn, (float)((mw >> (16 * (c & 1))) & 0xff));
                const float m2 = __fmul_rn(mn, (float)((mw >> (16 * (c & 1) + 8)) & 0xff));
                for (int kk = 0; kk < 2; kk++) {
                    const uint4 v = grp[32 * (3 + 2 * c + kk)];
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                    for (int i = 0; i < 16; i++) {
                        const int l = 16 * kk + i; /* byte l of this chunk's 32 quant bytes and of qh */
                        const uint32_t byte = (w[i >> 2] >> (8 * (i & 3))) & 0xff;
                        const uint32_t hbyte = (hb[l >> 2] >> (8 * (l & 3))) & 0xff;
                        const uint32_t q1 = (byte & 0xf) + (((hbyte >> (2 * c)) & 1) ? 16 : 0);
                        const uint32_t q2 = (byte >> 4) + (((hbyte >> (2 * c + 1)) & 1) ? 16 : 0);
                        y[64 * c + l] = __fsub_rn(__fmul_rn(d1, (float)q1), m1);
                        y[64 * c + 32 + l] = __fsub_rn(__fmul_rn(d2, (float)q2), m2);
                    }
                }
            }
        } else {
            const uint8_t *gb = shard + (uint64_t)(lb >> 5) * FB_Q6K_GROUP;
            const uint4 *grp = reinterpret_cast<const uint4 *>(gb) + (lb & 31);
            const float d = fb_half_bits_to_float(reinterpret_cast<const uint16_t *>(gb + FB_Q6K_OFF_D)[lb & 31]);
            const uint4 scv = grp[32 * 12];
            const uint32_t scw[4] = {scv.x, scv.y, scv.z, scv.w};
            for (int h = 0; h < 2; h++) {
                for (int l = 0; l < 32; l++) {
                    /* ql byte 64h+l, ql byte 64h+32+l, qh byte 32h+l */
                    auto byte_at = [&](int plane_first, int byte) -> uint32_t {
                        const uint4 v = grp[32 * (plane_first + (byte >> 4))];
                        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                        return (w[(byte & 15) >> 2] >> (8 * (byte & 3))) & 0xff;
                    };
                    const uint32_t a = byte_at(0, 64 * h + l), b = byte_at(0, 64 * h + 32 + l);
                    const uint32_t hh = byte_at(8, 32 * h + l);
                    const int is = l / 16;
                    const int q1 = (int)((a & 0xf) | (((hh >> 0) & 3) << 4)) - 32;
                    const int q2 = (int)((b & 0xf) | (((hh >> 2) & 3) << 4)) - 32;
                    const int q3 = (int)((a >> 4) | (((hh >> 4) & 3) << 4)) - 32;
                    const int q4 = (int)((b >> 4) | (((hh >> 6) & 3) << 4)) - 32;
                    auto scale = [&](int idx) -> float {
                        return (float)(int)(signed char)((scw[idx >> 2] >> (8 * (idx & 3))) & 0xff);
                    };
                    float *yy = y + 128 * h;
                    yy[l] = __fmul_rn(__fmul_rn(d, scale(8 * h + is + 0)), (float)q1);
                    yy[l + 32] = __fmul_rn(__fmul_rn(d, scale(8 * h + is + 2)), (float)q2);
                    yy[l + 64] = __fmul_rn(__fmul_rn(d, scale(8 * h + is + 4)), (float)q3);
                    yy[l + 96] = __fmul_rn(__fmul_rn(d, scale(8 * h + is + 6)), (float)q4);
                }
            }
        }
    }
}

/* single dequant-matvec: out[row] = shard[row, :] . q8 */
template <int TYPE>
__global__ void __launch_bounds__(256) k_matvec(float *out, const uint8_t *shard, fb_shard_geom_t g,
                                                const fb_q8_entry_t *q8) {
    extern __shared__ uint4 smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int bpr = g.bpr_local;
    const uint4 *src = reinterpret_cast<const uint4 *>(q8);
    for (int i = threadIdx.x; i < bpr * FB_Q8_U4; i += blockDim.x) smem[i] = src[i];
    __syncthreads();
    const uint4 *a = smem + (lane % bpr) * FB_Q8_U4;
    const int rpg = 32 / bpr;
    const int n_groups = (int)fb_n_groups((uint64_t)g.rows_local * bpr);
    for (int gi = blockIdx.x * wpb + warp; gi < n_groups; gi += gridDim.x * wpb) {
        float f;
        if (TYPE == FB_TYPE_Q4_K) {
            const uint4 *p = reinterpret_cast<const uint4 *>(shard + (uint64_t)gi * FB_Q4K_GROUP) + lane;
            uint4 hd = p[0];
            uint4 q[8];
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = p[32 * (i + 1)];
            f = fb_dot_q4k(hd, q, a);
        } else if (TYPE == FB_TYPE_Q5_K) {
            const uint4 *p = reinterpret_cast<const uint4 *>(shard + (uint64_t)gi * FB_Q5K_GROUP) + lane;
            const uint4 hd = p[0], h0 = p[32], h1 = p[64];
            uint4 q[8];
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = p[32 * (i + 3)];
            f = fb_dot_q5k(hd, h0, h1, q, a);
        } else {
            const uint8_t *gb = shard + (uint64_t)gi * FB_Q6K_GROUP;
            const uint4 *p = reinterpret_cast<const uint4 *>(gb) + lane;
            uint4 ql[8], qh[4];
#pragma unroll
            for (int i = 0; i < 8; i++) ql[i] = p[32 * i];
#pragma unroll
            for (int i = 0; i < 4; i++) qh[i] = p[32 * (8 + i)];
            const uint4 sc = p[32 * 12];
            const uint32_t d16 = reinterpret_cast<const unsigned short *>(gb + FB_Q6K_OFF_D)[lane];
            f = fb_dot_q6k(ql, qh, sc, d16, a);
        }
        f = fb_span_sum(f, bpr);
        const int row = gi * rpg + lane / bpr;
        if (lane % bpr == 0 && row < g.rows_local) out[row] = f;
    }
}

__global__ void k_quantize(fb_q8_entry_t *dst, const float *src, int n_blocks) {
    const int lane = threadIdx.x & 31, warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (warp >= n_blocks) return;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = src[warp * FB_QK + 8 * lane + i];
    fb_warp_quantize(v, dst + warp, lane);
}

/* ------------------------------------------------------------------ launchers */
static int grid_for(int n, int block) {
    int g = (n + block - 1) / block;
    return g < 1 ? 1 : (g > 1184 ? 1184 : g);
}

extern "C" int fb_launch_gen_shards(uint8_t *dst0, uint64_t rec_stride, int n_recs, uint64_t seed, uint32_t layer,
                                    uint32_t matrix, fb_shard_geom_t g, void *stream) {
    const int n_pad = (int)fb_n_groups((uint64_t)g.rows_local * g.bpr_local) * 32;
    dim3 grid(grid_for(n_pad, 128) > 64 ? 64 : grid_for(n_pad, 128), n_recs);
    k_gen_shards<<<grid, 128, 0, (cudaStream_t)stream>>>(dst0, rec_stride, seed, layer, matrix, g);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_gen_f32(float *dst, uint64_t n, uint64_t seed, uint32_t layer, uint32_t stream_id,
                                 float mean, float std, void *stream) {
    const uint64_t key = fsyn_key(seed, layer, 0, stream_id);
    k_gen_f32<<<grid_for((int)(n > (1u << 30) ? (1u << 30) : n), 256), 256, 0, (cudaStream_t)stream>>>(dst, n, key,
                                                                                                     mean, std);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_repack(uint8_t *dst, const uint8_t *src_ggml, fb_shard_geom_t g, void *stream) {
    const int n_pad = (int)fb_n_groups((uint64_t)g.rows_local * g.bpr_local) * 32;
    k_repack<<<grid_for(n_pad, 128), 128, 0, (cudaStream_t)stream>>>(dst, src_ggml, g);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_export_ggml(uint8_t *dst_ggml, const uint8_t *shard, fb_shard_geom_t g, void *stream) {
    k_export_ggml<<<grid_for(g.rows_local * g.bpr_local, 128), 128, 0, (cudaStream_t)stream>>>(dst_ggml, shard, g);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_dequant(float *dst, const uint8_t *shard, fb_shard_geom_t g, void *stream) {
    k_dequant<<<grid_for(g.rows_local * g.bpr_local, 128), 128, 0, (cudaStream_t)stream>>>(dst, shard, g);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_matvec(float *out, const uint8_t *shard, fb_shard_geom_t g, const fb_q8_entry_t *q8,
                                int grid, void *stream) {
    const size_t sm = (size_t)g.bpr_local * sizeof(fb_q8_entry_t);
    if (g.type == FB_TYPE_Q4_K)
        k_matvec<FB_TYPE_Q4_K><<<grid, 256, sm, (cudaStream_t)stream>>>(out, shard, g, q8);
    else if (g.type == FB_TYPE_Q5_K)
        k_matvec<FB_TYPE_Q5_K><<<grid, 256, sm, (cudaStream_t)stream>>>(out, shard, g, q8);
    else
        k_matvec<FB_TYPE_Q6_K><<<grid, 256, sm, (cudaStream_t)stream>>>(out, shard, g, q8);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_quantize(fb_q8_entry_t *dst, const float *src, int n_blocks, void *stream) {
    k_quantize<<<(n_blocks * 32 + 255) / 256, 256, 0, (cudaStream_t)stream>>>(dst, src, n_blocks);
    return (int)cudaGetLastError();
}

/* ------------------------------------------------------------------ matvec without any allocation
 *
 * Some callers may not allocate device memory while they run: a serving loop whose memory pool was sized and
 * handed out at start-up, code running under a framework that owns every byte of the GPU, or a latency-critical
 * path where cudaMalloc's implicit device synchronisation is not acceptable.  fomoe_b200_matvec() allocates its
 * two temporaries (the weight matrix regrouped into the lane-striped layout, and the Q8_K-quantised input) on
 * every call; this variant keeps them in one fixed array that is part of the library image instead.
 *
 * The array lives in every GPU context that loads the library until the process exits (FB_NOALLOC_BYTES, 4 MiB
 * plus the quantised input).  All calls on a device share it and it keeps the previous call's contents, so two
 * calls whose kernels could overlap on the GPU (different streams, no ordering between them) race; calls on one
 * stream are safe.  Nothing in it needs to start at zero: every byte that is read has been written by the same
 * call's kernels (the regrouping kernel also writes the zero padding of the last group).
 */
#define FB_NOALLOC_SHARD_BYTES (4u << 20)                                  /* regrouped weights: up to 4 MiB */
#define FB_NOALLOC_Q8_ENTRIES 32                                           /* cols <= 8192 */
#define FB_NOALLOC_BYTES (FB_NOALLOC_SHARD_BYTES + FB_NOALLOC_Q8_ENTRIES * sizeof(fb_q8_entry_t))
#define FB_NOALLOC_MAX_DEVICES 64

static __device__ __align__(256) unsigned char fb_noalloc_scratch[FB_NOALLOC_BYTES];

/* In host code the name above is only a stand-in for the symbol, not an address the GPU can use: the device
 * address is looked up once per device, with that device current, and that pointer is what the kernels get. */
static unsigned char *fb_noalloc_ptr[FB_NOALLOC_MAX_DEVICES];

extern "C" int fomoe_b200_matvec_noalloc(int type, const void *w_ggml_dev, int rows, int cols, const float *x_dev,
                                         float *y_dev, void *stream) {
    if (!w_ggml_dev || !x_dev || !y_dev || rows < 1 || cols < FB_QK || cols % FB_QK) {
        fprintf(stderr, "fomoe_b200_matvec_noalloc: bad arguments\n");
        return -1;
    }
    const int bpr = cols / FB_QK;
    if ((type != FB_TYPE_Q4_K && type != FB_TYPE_Q5_K && type != FB_TYPE_Q6_K) || (bpr & (bpr - 1)) ||
        bpr > FB_NOALLOC_Q8_ENTRIES) {
        fprintf(stderr, "fomoe_b200_matvec_noalloc: unsupported type %d or column count %d (a power-of-two number of "
                        "256-column blocks, at most %d columns)\n", type, cols, FB_NOALLOC_Q8_ENTRIES * FB_QK);
        return -1;
    }
    const uint64_t shard_bytes = fb_shard_bytes(type, (uint64_t)rows * bpr);
    if (shard_bytes > FB_NOALLOC_SHARD_BYTES) {
        fprintf(stderr, "fomoe_b200_matvec_noalloc: a %d x %d matrix needs %llu bytes of scratch, the fixed array holds "
                        "%u; use fomoe_b200_matvec for larger matrices\n", rows, cols, (unsigned long long)shard_bytes,
                FB_NOALLOC_SHARD_BYTES);
        return -1;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= FB_NOALLOC_MAX_DEVICES) {
        fprintf(stderr, "fomoe_b200_matvec_noalloc: no current CUDA device\n");
        return -1;
    }
    if (!fb_noalloc_ptr[dev]) { /* first call on this device: not capturable, do it before any stream capture */
        void *p = NULL;
        const cudaError_t e = cudaGetSymbolAddress(&p, fb_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            fprintf(stderr, "fomoe_b200_matvec_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
            return -1;
        }
        fb_noalloc_ptr[dev] = (unsigned char *)p;
    }
    unsigned char *shard = fb_noalloc_ptr[dev];
    fb_q8_entry_t *q8 = reinterpret_cast<fb_q8_entry_t *>(fb_noalloc_ptr[dev] + FB_NOALLOC_SHARD_BYTES);
    const fb_shard_geom_t g = {type, rows, bpr, 0, 0, bpr, -1};
    const int n_groups = (int)fb_n_groups((uint64_t)rows * bpr);
    int rc = fb_launch_repack(shard, (const uint8_t *)w_ggml_dev, g, stream);
    if (!rc) rc = fb_launch_quantize(q8, x_dev, bpr, stream);
    if (!rc) rc = fb_launch_matvec(y_dev, shard, g, q8, grid_for(n_groups, 8), stream);
    if (rc) {
        fprintf(stderr, "fomoe_b200_matvec_noalloc: launch failed: %s\n", cudaGetErrorString((cudaError_t)rc));
        return -1;
    }
    return 0;
}
