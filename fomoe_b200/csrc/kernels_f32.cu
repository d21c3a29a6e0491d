/*
 * kernels_f32.cu -- the expert phases with fp32 activations.
 *
 * The reference defines the expert FFN twice: with Q8_K int8 activations (src/cpu_expert.c, the definition every
 * other kernel of this library follows) and with fp32 activations -- its CPU forward pass without cpu_expert
 * (src/inference.c:556-575 through src/tensor.c:102-160, dots src/quant.c:109-143, 177-212, 249-262) and, up to
 * summation order, its GPU kernels (src/gpu_kernels.hip:1121, 1261, 1320).  The two differ by a few percent on the
 * same inputs, so a caller that compares against the fp32 definition selects it (fomoe_b200_set_act_mode) and
 * gets these kernels: same table, same task split and combine as kernels.cu, activations read as floats.  They
 * are the parity path for that definition, not a tuned one.
 *
 * Per 32-weight sub-block j the dot is  d*sc_j * sum(q*y) - dmin*m_j * sum(y)  (Q4_K, Q5_K) or
 * d*sc_g * sum((q-32)*y)  (Q6_K, 16-weight groups) in fp32: the reference's per-element products, regrouped.
 */
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "dots.cuh"
#include "launch.h"

#ifndef FULL
#define FULL 0xffffffffu
#endif

__device__ __forceinline__ uint4 ldg_w(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

/* sum of q*y over the 16 bytes of one piece: low nibbles against y[0..15], high nibbles against yh[0..15] */
__device__ __forceinline__ void nib_dot(const uint4 &w, const float *yl, const float *yh, float &lo, float &hi) {
    const uint32_t c[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const uint32_t b = (c[i >> 2] >> (8 * (i & 3))) & 0xff;
        lo = fmaf((float)(b & 0xf), yl[i], lo);
        hi = fmaf((float)(b >> 4), yh[i], hi);
    }
}

/* Q4_K / Q5_K block (header, optional fifth bits h0,h1, eight quant pieces) against 256 floats */
template <bool Q5>
__device__ __forceinline__ float dot_q45k_f32(const uint4 &hdr, const uint4 &h0, const uint4 &h1, const uint4 (&qs)[8],
                                              const float *y) {
    const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
    const uint32_t sc_lo = u0 & 0x3f3f3f3fu, sc_hi = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
    const uint32_t m_lo = u1 & 0x3f3f3f3fu, m_hi = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
    const float d = fb_half_bits_to_float(hdr.x & 0xffff), dmin = fb_half_bits_to_float(hdr.x >> 16);
    float total = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        float lo = 0.0f, hi = 0.0f, ylo = 0.0f, yhi = 0.0f;
        const float *yl = y + 64 * c, *yh = y + 64 * c + 32;
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            nib_dot(qs[2 * c + kk], yl + 16 * kk, yh + 16 * kk, lo, hi);
            if (Q5) { /* the fifth bit adds 16: byte l of the fifth-bit field, bit 2c (low half) / 2c+1 (high half) */
                const uint4 hb = kk ? h1 : h0;
                const uint32_t hc[4] = {hb.x, hb.y, hb.z, hb.w};
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const uint32_t b = (hc[i >> 2] >> (8 * (i & 3))) & 0xff;
                    if ((b >> (2 * c)) & 1u) lo += 16.0f * yl[16 * kk + i];
                    if ((b >> (2 * c + 1)) & 1u) hi += 16.0f * yh[16 * kk + i];
                }
            }
        }
#pragma unroll 8
        for (int i = 0; i < 32; i++) {
            ylo += yl[i];
            yhi += yh[i];
        }
        const uint32_t scw = (c < 2) ? sc_lo : sc_hi, mw = (c < 2) ? m_lo : m_hi;
        const int sh = 16 * (c & 1);
        total += d * (float)((scw >> sh) & 0xff) * lo - dmin * (float)((mw >> sh) & 0xff) * ylo;
        total += d * (float)((scw >> (sh + 8)) & 0xff) * hi - dmin * (float)((mw >> (sh + 8)) & 0xff) * yhi;
    }
    return total;
}

__device__ __forceinline__ float dot_q6k_f32(const uint4 (&ql)[8], const uint4 (&qh)[4], const uint4 &sc, uint32_t d16,
                                             const float *y) {
    const float d = fb_half_bits_to_float(d16);
    const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
    float total = 0.0f;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float *yp = y + 128 * h;
#pragma unroll
        for (int half = 0; half < 2; half++) { /* l = 16*half .. 16*half+15: scale index is = half */
            const uint4 A = ql[4 * h + half], B = ql[4 * h + 2 + half], H = qh[2 * h + half];
            const uint32_t a[4] = {A.x, A.y, A.z, A.w}, b[4] = {B.x, B.y, B.z, B.w}, hh[4] = {H.x, H.y, H.z, H.w};
            float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int l = 16 * half + i;
                const uint32_t qa = (a[i >> 2] >> (8 * (i & 3))) & 0xff, qb = (b[i >> 2] >> (8 * (i & 3))) & 0xff;
                const uint32_t hb = (hh[i >> 2] >> (8 * (i & 3))) & 0xff;
                s0 = fmaf((float)((int)((qa & 0xf) | ((hb & 3) << 4)) - 32), yp[l], s0);
                s1 = fmaf((float)((int)((qb & 0xf) | (((hb >> 2) & 3) << 4)) - 32), yp[l + 32], s1);
                s2 = fmaf((float)((int)((qa >> 4) | (((hb >> 4) & 3) << 4)) - 32), yp[l + 64], s2);
                s3 = fmaf((float)((int)((qb >> 4) | (((hb >> 6) & 3) << 4)) - 32), yp[l + 96], s3);
            }
            auto scale = [&](int idx) { return (float)(int)(signed char)((scw[idx >> 2] >> (8 * (idx & 3))) & 0xff); };
            const int is = 8 * h + half;
            total += d * scale(is + 0) * s0 + d * scale(is + 2) * s1 + d * scale(is + 4) * s2 + d * scale(is + 6) * s3;
        }
    }
    return total;
}

/* gate/up + SwiGLU: tasks and row mapping as k_gate_up (kernels.cu); the hidden state sits in shared memory as floats */
template <int GT>
__global__ void __launch_bounds__(256) k_gate_up_f32(fb_args_t A) {
    extern __shared__ float hs[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int bpr = A.gate_bpr;
    for (int i = threadIdx.x; i < A.n_embd; i += blockDim.x) hs[i] = A.h[i];
    __syncthreads();
    const float *y = hs + (lane % bpr) * FB_QK;
    const int rpg = 32 / bpr;
    const int total = A.n_slots * A.gate_groups;
    for (int t = blockIdx.x * wpb + warp; t < total; t += gridDim.x * wpb) {
        const int slot = t / A.gate_groups, g = t - slot * A.gate_groups;
        const uint8_t *rec = A.slot_rec[slot];
        float f[2];
#pragma unroll
        for (int which = 0; which < 2; which++) {
            if (GT == FB_TYPE_Q6_K) {
                const uint8_t *gb = rec + (which ? A.up_off : 0) + (uint64_t)g * FB_Q6K_GROUP;
                const uint4 *p = reinterpret_cast<const uint4 *>(gb) + lane;
                uint4 ql[8], qh[4];
#pragma unroll
                for (int i = 0; i < 8; i++) ql[i] = ldg_w(p + 32 * i);
#pragma unroll
                for (int i = 0; i < 4; i++) qh[i] = ldg_w(p + 32 * (8 + i));
                const uint4 sc = ldg_w(p + 32 * 12);
                const uint32_t d16 = __ldg(reinterpret_cast<const unsigned short *>(gb + FB_Q6K_OFF_D) + lane);
                f[which] = fb_span_sum(dot_q6k_f32(ql, qh, sc, d16, y), bpr);
            } else {
                const uint4 *p = reinterpret_cast<const uint4 *>(rec + (which ? A.up_off : 0) + (uint64_t)g * FB_Q4K_GROUP) + lane;
                const uint4 hd = ldg_w(p);
                uint4 q[8];
#pragma unroll
                for (int i = 0; i < 8; i++) q[i] = ldg_w(p + 32 * (i + 1));
                f[which] = fb_span_sum(dot_q45k_f32<false>(hd, hd, hd, q, y), bpr);
            }
        }
        const int row = g * rpg + lane / bpr;
        if (lane % bpr == 0 && row < A.inter_local) {
            const float s = __fdiv_rn(f[0], __fadd_rn(1.0f, expf(-f[0]))); /* silu, src/tensor.c:202-206 */
            A.act[slot * A.inter_local + row] = __fmul_rn(s, f[1]);
        }
    }
}

/* down + combine: as k_down; every slot's activation vector sits in shared memory as floats */
template <int TYPE>
__global__ void __launch_bounds__(256) k_down_f32(fb_args_t A) {
    extern __shared__ float as[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int bpr = A.down_bpr;
    for (int i = threadIdx.x; i < A.n_slots * A.inter_local; i += blockDim.x) as[i] = __ldcg(A.act + i);
    __syncthreads();
    const int rpg = 32 / bpr;
    const int total = A.n_slots * A.down_groups;
    unsigned *cnt_rg = A.counters + FB_CNT_WIN + FB_MAX_SLOTS * 32;
    for (int t = blockIdx.x * wpb + warp; t < total; t += gridDim.x * wpb) {
        const int rg = t / A.n_slots, slot = t - rg * A.n_slots;
        const uint8_t *rec = A.slot_rec[slot] + A.down_off;
        const float *y = as + slot * A.inter_local + (lane % bpr) * FB_QK;
        float f;
        if (TYPE == FB_TYPE_Q6_K) {
            const uint8_t *gb = rec + (uint64_t)rg * FB_Q6K_GROUP;
            const uint4 *p = reinterpret_cast<const uint4 *>(gb) + lane;
            uint4 ql[8], qh[4];
#pragma unroll
            for (int i = 0; i < 8; i++) ql[i] = ldg_w(p + 32 * i);
#pragma unroll
            for (int i = 0; i < 4; i++) qh[i] = ldg_w(p + 32 * (8 + i));
            const uint4 sc = ldg_w(p + 32 * 12);
            const uint32_t d16 = __ldg(reinterpret_cast<const unsigned short *>(gb + FB_Q6K_OFF_D) + lane);
            f = dot_q6k_f32(ql, qh, sc, d16, y);
        } else if (TYPE == FB_TYPE_Q5_K) {
            const uint4 *p = reinterpret_cast<const uint4 *>(rec + (uint64_t)rg * FB_Q5K_GROUP) + lane;
            const uint4 hd = ldg_w(p), h0 = ldg_w(p + 32), h1 = ldg_w(p + 64);
            uint4 q[8];
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = ldg_w(p + 32 * (i + 3));
            f = dot_q45k_f32<true>(hd, h0, h1, q, y);
        } else {
            const uint4 *p = reinterpret_cast<const uint4 *>(rec + (uint64_t)rg * FB_Q4K_GROUP) + lane;
            const uint4 hd = ldg_w(p);
            uint4 q[8];
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = ldg_w(p + 32 * (i + 1));
            f = dot_q45k_f32<false>(hd, hd, hd, q, y);
        }
        f = fb_span_sum(f, bpr);
        const int row = rg * rpg + lane / bpr;
        if (lane % bpr == 0 && row < A.n_embd) A.dots[slot * A.n_embd + row] = f;
        /* the last warp to finish a row group combines: out += score * down in list order (vec_scaled_add,
         * src/inference.c:574), the shared expert added after with weight 1 or its gate (582-596) */
        int last = 0;
        __syncwarp();
        if (lane == 0) {
            __threadfence();
            const unsigned old = atomicAdd(cnt_rg + rg, 1u);
            last = (old == (unsigned)A.n_slots - 1);
        }
        last = __shfl_sync(FULL, last, 0);
        if (last) {
            __threadfence();
            const int r = rg * rpg + lane;
            if (lane < rpg && r < A.n_embd) {
                float acc = A.accumulate ? A.moe_out[r] : 0.0f;
                for (int s = 0; s < A.top_k; s++)
                    acc = __fmaf_rn(__ldcg(A.scores + s), __ldcg(A.dots + s * A.n_embd + r), acc);
                if (A.has_shared) {
                    const float sh = __ldcg(A.dots + A.top_k * A.n_embd + r);
                    acc = __fadd_rn(acc, A.shared_gate_w ? __fmul_rn(sh, __ldcg(A.scores + A.top_k)) : sh);
                }
                A.moe_out[r] = acc;
            }
            if (lane == 0) cnt_rg[rg] = 0;
        }
    }
}

extern "C" int fb_launch_gate_up_f32(const fb_args_t *a, int grid, void *stream) {
    const size_t sm = sizeof(float) * (size_t)a->n_embd;
    static unsigned char configured[64]; /* the attribute holds for one device */
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_gate_up_f32<FB_TYPE_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(k_gate_up_f32<FB_TYPE_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = 1;
    }
    if (sm > 128 * 1024) return (int)cudaErrorInvalidValue;
    if (a->gate_type == FB_TYPE_Q6_K) k_gate_up_f32<FB_TYPE_Q6_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    else k_gate_up_f32<FB_TYPE_Q4_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_down_f32(const fb_args_t *a, int grid, void *stream) {
    const size_t sm = sizeof(float) * (size_t)a->n_slots * a->inter_local;
    if (a->down_half >= 0) return (int)cudaErrorInvalidValue; /* the fp32 definition is not built for half super-blocks */
    static unsigned char configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_down_f32<FB_TYPE_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(k_down_f32<FB_TYPE_Q5_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(k_down_f32<FB_TYPE_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = 1;
    }
    if (sm > 160 * 1024) return (int)cudaErrorInvalidValue;
    if (a->down_type == FB_TYPE_Q4_K)
        k_down_f32<FB_TYPE_Q4_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    else if (a->down_type == FB_TYPE_Q5_K)
        k_down_f32<FB_TYPE_Q5_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    else
        k_down_f32<FB_TYPE_Q6_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}
