/*
 * kernels.cu -- the decode hot path as per-phase kernels (sm_100a):
 *
 *   k_prologue   x += moe_out (+ resid); h = rmsnorm(x) * w; q8h = Q8_K(h)
 *   k_router     fp32 router logits (warp per expert row); the last block to finish runs
 *                softmax, ordered top-k, renormalise and CAR substitute-and-dampen in one warp
 *   k_gate_up    Q4_K gate and up dequant-matvec of every selected expert + the shared expert,
 *                SwiGLU in the epilogue; the last warp to finish a 256-row window quantises it
 *   k_down       Q4_K / Q5_K / Q6_K down dequant-matvec per expert; the last warp to finish a row group
 *                combines the experts with their routing weights in list order
 *
 * Reference counterparts: src/gpu_kernels.hip:2127 (router matvec), 2668 (softmax), 2745 (top-k),
 * 7097-7187 (host classify + car_evaluate), 1320 (fused gate/up/SiLU), 1121/1261 (down per expert),
 * 1631/1647 (weighted sum), 2427/2818 (RMSNorm); numerics follow src/cpu_expert.c and src/quant.c.
 *
 * All weights stream once from HBM in the lane-striped layout (layout.h) with 128-bit,
 * fully coalesced loads; the work is integer dp4a + warp shuffles; no tensor cores (batch 1
 * is a memory-bound matvec).
 */
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "dots.cuh"
#include "launch.h"
#include "route.cuh"
#include "stream.cuh"

#ifndef FULL
#define FULL 0xffffffffu
#endif

/* template selectors of the down kernels for shards of half super-blocks (never stored anywhere) */
#define FB_TYPE_Q4_K_H 112
#define FB_TYPE_Q5_K_H 113
#define FB_TYPE_Q6_K_H 114

/* cudaFuncSetAttribute holds for one device: remember per device ordinal whether it has been done */
#define FB_MAX_DEVICES 64
static bool fb_device_once(unsigned char (&done)[FB_MAX_DEVICES], int &dev) {
    dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= FB_MAX_DEVICES) dev = 0;
    return done[dev] != 0;
}

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    /* weights are read exactly once: keep them out of L1 */
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

/* ------------------------------------------------------------------ prologue */
__global__ void __launch_bounds__(1024) k_prologue(fb_args_t A, int flags) {
    __shared__ float red[32];
    __shared__ float s_scale;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = A.n_embd;
    if (tid == 0) {
        /* arrival counters start every layer at zero */
        A.counters[FB_CNT_ROUTER] = 0;
    }
    const unsigned tok = (flags & (FB_PRO_LOAD | FB_PRO_STORE)) ? *A.tok_ctr : 0u;
    float ss = 0.0f;
    for (int i = tid; i < n; i += blockDim.x) {
        float v = (flags & FB_PRO_LOAD) ? A.tok_in[(size_t)tok * n + i] : A.x[i];
        if (flags & FB_PRO_ADD_PREV) v = __fadd_rn(v, A.moe_out[i]);
        if ((flags & FB_PRO_RESID) && A.resid) v = __fadd_rn(v, A.resid[i]);
        A.x[i] = v;
        if (flags & FB_PRO_STORE) A.tok_out[(size_t)tok * n + i] = v;
        ss = __fmaf_rn(v, v, ss);
    }
    if (flags & FB_PRO_STORE) {
        __syncthreads();
        if (tid == 0) *A.tok_ctr = tok + 1;
        return;
    }
    if (flags & FB_PRO_NORM) {
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(FULL, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (warp == 0) {
            float t = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.0f;
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(FULL, t, o);
            if (lane == 0) s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)n), A.rms_eps)));
        }
        __syncthreads();
        const float sc = s_scale;
        for (int i = tid; i < n; i += blockDim.x) {
            const float w = A.normw ? A.normw[i] : 1.0f;
            A.h[i] = __fmul_rn(__fmul_rn(A.x[i], sc), w); /* x * s * w, left to right (src/tensor.c:181-183) */
        }
    } else {
        for (int i = tid; i < n; i += blockDim.x) A.h[i] = A.x[i];
    }
    if (A.shared_gate_w) {
        /* scalar gate of the shared expert: sigmoid(h . w) (src/inference.c:586-592) */
        __syncthreads();
        float p = 0.0f;
        for (int i = tid; i < n; i += blockDim.x) p = __fmaf_rn(A.h[i], A.shared_gate_w[i], p);
        for (int o = 16; o > 0; o >>= 1) p += __shfl_xor_sync(FULL, p, o);
        if (lane == 0) red[warp] = p;
        __syncthreads();
        if (warp == 0) {
            float t = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.0f;
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(FULL, t, o);
            if (lane == 0) *A.shared_gate = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-t)));
        }
    }
    if (flags & FB_PRO_QUANT) {
        __syncthreads();
        for (int b = warp; b < n / FB_QK; b += (blockDim.x >> 5)) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = A.h[b * FB_QK + 8 * lane + i];
            fb_warp_quantize(v, &A.q8h[b], lane);
        }
    }
}

/* ------------------------------------------------------------------ router */
__global__ void __launch_bounds__(256) k_router(fb_args_t A) {
    __shared__ int s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wpb = blockDim.x >> 5;
    const int n4 = A.n_embd >> 2;
    const float4 *h4 = reinterpret_cast<const float4 *>(A.h);
    for (int row = blockIdx.x * wpb + warp; row < A.n_experts; row += gridDim.x * wpb) {
        const float4 *w4 = reinterpret_cast<const float4 *>(A.router_w + (size_t)row * A.n_embd);
        float acc = 0.0f;
        for (int i0 = 0; i0 < n4; i0 += 256) {
            float4 w[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u * 32 + lane;
                w[u] = (i < n4) ? __ldg(w4 + i) : make_float4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u * 32 + lane;
                if (i < n4) {
                    const float4 x = h4[i];
                    acc = fmaf(w[u].x, x.x, acc);
                    acc = fmaf(w[u].y, x.y, acc);
                    acc = fmaf(w[u].z, x.z, acc);
                    acc = fmaf(w[u].w, x.w, acc);
                }
            }
        }
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(FULL, acc, o);
        if (lane == 0) A.logits[row] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned old = atomicAdd(A.counters + FB_CNT_ROUTER, 1u);
        s_last = (old == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (warp == 0) fb_route_select(A, lane, true);
}

/* ids/scores given by the caller (operator form: the reference's gpu_expert_ffn takes them) */
__global__ void k_set_slots(fb_args_t A) {
    const int r = threadIdx.x;
    if (r < A.top_k) {
        int e = A.ids[r];
        if (e < 0 || e >= A.n_experts) {
            atomicExch(A.status, FB_ST_BAD_ID);
            e = 0;
        }
        A.slot_rec[r] = A.table_layer + (uint64_t)e * A.rec_bytes;
    } else if (r == A.top_k && A.has_shared) {
        A.ids[r] = A.n_experts;
        A.scores[r] = 1.0f;
        A.slot_rec[r] = A.table_layer + (uint64_t)A.n_experts * A.rec_bytes;
    }
}

/* ------------------------------------------------------------------ gate / up / SwiGLU */
template <int GT>
__global__ void __launch_bounds__(256) k_gate_up(fb_args_t A) {
    extern __shared__ uint4 smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int bpr = A.gate_bpr;
    {   /* stage the quantised hidden state */
        const uint4 *src = reinterpret_cast<const uint4 *>(A.q8h);
        for (int i = threadIdx.x; i < bpr * FB_Q8_U4; i += blockDim.x) smem[i] = src[i];
    }
    __syncthreads();
    const uint4 *a = smem + (lane % bpr) * FB_Q8_U4;
    const int rpg = 32 / bpr;             /* rows per group */
    const int gpw = FB_QK / rpg;          /* groups per 256-row window */
    const int nwin = A.inter_local / FB_QK;
    const int total = A.n_slots * A.gate_groups;
    for (int t = blockIdx.x * wpb + warp; t < total; t += gridDim.x * wpb) {
        const int slot = t / A.gate_groups, g = t - slot * A.gate_groups;
        const uint8_t *rec = A.slot_rec[slot];
        float fg, fu;
        if (GT == FB_TYPE_Q6_K) { /* src/quant.c:478-607 on both matrices, one after the other */
            float f2[2];
#pragma unroll 1
            for (int which = 0; which < 2; which++) {
                const uint8_t *gb = rec + (which ? A.up_off : 0) + (uint64_t)g * FB_Q6K_GROUP;
                const uint4 *p = reinterpret_cast<const uint4 *>(gb) + lane;
                uint4 ql[8], qh[4];
#pragma unroll
                for (int i = 0; i < 8; i++) ql[i] = ldg_stream(p + 32 * i);
#pragma unroll
                for (int i = 0; i < 4; i++) qh[i] = ldg_stream(p + 32 * (8 + i));
                const uint4 sc = ldg_stream(p + 32 * 12);
                const uint32_t d16 = __ldg(reinterpret_cast<const unsigned short *>(gb + FB_Q6K_OFF_D) + lane);
                f2[which] = fb_dot_q6k(ql, qh, sc, d16, a);
            }
            fg = f2[0];
            fu = f2[1];
        } else {
            const uint4 *pg = reinterpret_cast<const uint4 *>(rec + (uint64_t)g * FB_Q4K_GROUP) + lane;
            const uint4 *pu = reinterpret_cast<const uint4 *>(rec + A.up_off + (uint64_t)g * FB_Q4K_GROUP) + lane;
            uint4 hg = ldg_stream(pg), hu = ldg_stream(pu);
            uint4 qg[8], qu[8];
#pragma unroll
            for (int i = 0; i < 8; i++) qg[i] = ldg_stream(pg + 32 * (i + 1));
#pragma unroll
            for (int i = 0; i < 8; i++) qu[i] = ldg_stream(pu + 32 * (i + 1));
            fg = fb_dot_q4k(hg, qg, a);
            fu = fb_dot_q4k(hu, qu, a);
        }
        fg = fb_span_sum(fg, bpr);
        fu = fb_span_sum(fu, bpr);
        const int row = g * rpg + lane / bpr;
        if (lane % bpr == 0 && row < A.inter_local) {
            /* SiLU(gate) * up exactly as src/cpu_expert.c:103-106 */
            const float s = __fdiv_rn(fg, __fadd_rn(1.0f, expf(-fg)));
            A.act[slot * A.inter_local + row] = __fmul_rn(s, fu);
        }
        /* the last warp to finish a 256-row window quantises it (src/cpu_expert.c:109-110) */
        const int win = (g * rpg) / FB_QK;
        int last = 0;
        __syncwarp();
        if (lane == 0) {
            __threadfence();
            const unsigned old = atomicAdd(A.counters + FB_CNT_WIN + slot * nwin + win, 1u);
            last = (old == (unsigned)gpw - 1);
        }
        last = __shfl_sync(FULL, last, 0);
        if (last) {
            __threadfence();
            const float *src = A.act + slot * A.inter_local + win * FB_QK + 8 * lane;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = __ldcg(src + i);
            fb_warp_quantize(v, &A.q8a[slot * nwin + win], lane);
            if (lane == 0) A.counters[FB_CNT_WIN + slot * nwin + win] = 0;
        }
    }
}

/* ------------------------------------------------------------------ down + combine */
template <int TYPE>
__global__ void __launch_bounds__(256) k_down(fb_args_t A) {
    extern __shared__ uint4 smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int bpr = A.down_bpr;
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(A.q8a);
        for (int i = threadIdx.x; i < A.n_slots * bpr * FB_Q8_U4; i += blockDim.x) smem[i] = src[i];
    }
    __syncthreads();
    const int rpg = 32 / bpr;
    const int total = A.n_slots * A.down_groups;
    unsigned *cnt_rg = A.counters + FB_CNT_WIN + FB_MAX_SLOTS * 32;
    for (int t = blockIdx.x * wpb + warp; t < total; t += gridDim.x * wpb) {
        const int rg = t / A.n_slots, slot = t - rg * A.n_slots;
        const uint8_t *rec = A.slot_rec[slot] + A.down_off;
        const uint4 *a = smem + (slot * bpr + lane % bpr) * FB_Q8_U4;
        float f;
        if (TYPE == FB_TYPE_Q4_K_H) { /* half super-blocks: one half-block per row, 32 rows per group */
            const uint4 *p = reinterpret_cast<const uint4 *>(rec + (uint64_t)rg * FB_Q4K_HGROUP) + lane;
            const uint4 hd = ldg_stream(p);
            uint4 q[4];
#pragma unroll
            for (int i = 0; i < 4; i++) q[i] = ldg_stream(p + 32 * (i + 1));
            f = fb_dot_q4k_half_sm(hd, q, fb_smem_u32(a), A.down_half);
        } else if (TYPE == FB_TYPE_Q5_K_H) {
            const uint4 *p = reinterpret_cast<const uint4 *>(rec + (uint64_t)rg * FB_Q5K_HGROUP) + lane;
            const uint4 hd = ldg_stream(p), h0 = ldg_stream(p + 32), h1 = ldg_stream(p + 64);
            uint4 q[4];
#pragma unroll
            for (int i = 0; i < 4; i++) q[i] = ldg_stream(p + 32 * (i + 3));
            f = fb_dot_q5k_half_sm(hd, h0, h1, q, fb_smem_u32(a), A.down_half);
        } else if (TYPE == FB_TYPE_Q6_K_H) {
            const uint8_t *gb = rec + (uint64_t)rg * FB_Q6K_HGROUP;
            const uint4 *p = reinterpret_cast<const uint4 *>(gb) + lane;
            uint4 ql[4], qh[2];
#pragma unroll
            for (int i = 0; i < 4; i++) ql[i] = ldg_stream(p + 32 * i);
#pragma unroll
            for (int i = 0; i < 2; i++) qh[i] = ldg_stream(p + 32 * (4 + i));
            const uint2 sc = __ldg(reinterpret_cast<const uint2 *>(gb + FB_Q6K_HOFF_SC) + lane);
            const uint32_t d16 = __ldg(reinterpret_cast<const unsigned short *>(gb + FB_Q6K_HOFF_D) + lane);
            f = fb_dot_q6k_half_sm(ql, qh, sc, d16, fb_smem_u32(a), A.down_half);
        } else if (TYPE == FB_TYPE_Q4_K) {
            const uint4 *p = reinterpret_cast<const uint4 *>(rec + (uint64_t)rg * FB_Q4K_GROUP) + lane;
            uint4 hd = ldg_stream(p);
            uint4 q[8];
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = ldg_stream(p + 32 * (i + 1));
            f = fb_dot_q4k(hd, q, a);
        } else if (TYPE == FB_TYPE_Q5_K) {
            const uint4 *p = reinterpret_cast<const uint4 *>(rec + (uint64_t)rg * FB_Q5K_GROUP) + lane;
            const uint4 hd = ldg_stream(p), h0 = ldg_stream(p + 32), h1 = ldg_stream(p + 64);
            uint4 q[8];
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = ldg_stream(p + 32 * (i + 3));
            f = fb_dot_q5k(hd, h0, h1, q, a);
        } else {
            const uint8_t *gb = rec + (uint64_t)rg * FB_Q6K_GROUP;
            const uint4 *p = reinterpret_cast<const uint4 *>(gb) + lane;
            uint4 ql[8], qh[4];
#pragma unroll
            for (int i = 0; i < 8; i++) ql[i] = ldg_stream(p + 32 * i);
#pragma unroll
            for (int i = 0; i < 4; i++) qh[i] = ldg_stream(p + 32 * (8 + i));
            const uint4 sc = ldg_stream(p + 32 * 12);
            const uint32_t d16 = __ldg(reinterpret_cast<const unsigned short *>(gb + FB_Q6K_OFF_D) + lane);
            f = fb_dot_q6k(ql, qh, sc, d16, a);
        }
        f = fb_span_sum(f, bpr);
        const int row = rg * rpg + lane / bpr;
        if (lane % bpr == 0 && row < A.n_embd) A.dots[slot * A.n_embd + row] = f;
        /* the last warp to finish a row group combines all experts in list order:
         * partial += score * down (src/cpu_expert.c:114-115), shared expert added after
         * (src/inference.c:595) */
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

/* ------------------------------------------------------------------ bulk-copy ring variants */
#define GU_WARPS 8
#define GU_STAGES 3
#define GU_STAGE_BYTES (2 * FB_Q4K_GROUP) /* gate group + up group */

/* Same work split and arithmetic as k_gate_up; weights arrive through per-warp rings of
 * bulk copies and the quantised hidden state sits in registers (a lane always meets the
 * same 256-column block). */
__global__ void __launch_bounds__(GU_WARPS * 32, 1) k_gate_up_ring(fb_args_t A) {
    extern __shared__ __align__(128) uint8_t dsm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int bpr = A.gate_bpr;
    uint8_t *ring = dsm + (size_t)warp * GU_STAGES * GU_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(dsm + (size_t)GU_WARPS * GU_STAGES * GU_STAGE_BYTES) + warp * GU_STAGES;
    const uint32_t ring_u = fb_smem_u32(ring), bar_u = fb_smem_u32(bars);
    if (lane == 0) {
        for (int s = 0; s < GU_STAGES; s++) fb_mbar_init(bar_u + 8 * s, 1);
        fb_mbar_init_fence();
    }
    __syncwarp();

    const int rpg = 32 / bpr, gpw = FB_QK / rpg, nwin = A.inter_local / FB_QK;
    const int total = A.n_slots * A.gate_groups;
    const int first = blockIdx.x * GU_WARPS + warp, stride = gridDim.x * GU_WARPS;
    const int n_my = first < total ? (total - first + stride - 1) / stride : 0;

    auto issue = [&](int i) {
        const int t = first + i * stride;
        const int slot = t / A.gate_groups, g = t - slot * A.gate_groups;
        const uint8_t *rec = A.slot_rec[slot];
        const uint32_t st = ring_u + (i % GU_STAGES) * GU_STAGE_BYTES, bar = bar_u + 8 * (i % GU_STAGES);
        fb_mbar_expect_tx(bar, GU_STAGE_BYTES);
        fb_bulk_g2s(st, rec + (uint64_t)g * FB_Q4K_GROUP, FB_Q4K_GROUP, bar);
        fb_bulk_g2s(st + FB_Q4K_GROUP, rec + A.up_off + (uint64_t)g * FB_Q4K_GROUP, FB_Q4K_GROUP, bar);
    };
    if (lane == 0)
        for (int i = 0; i < GU_STAGES && i < n_my; i++) issue(i);

    /* this lane's activation block, in registers */
    uint4 a[FB_Q8_U4];
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(A.q8h + (lane % bpr));
#pragma unroll
        for (int i = 0; i < FB_Q8_U4; i++) a[i] = src[i];
    }

    for (int i = 0; i < n_my; i++) {
        const int s = i % GU_STAGES;
        if (!fb_mbar_wait(bar_u + 8 * s, (i / GU_STAGES) & 1)) {
            if (lane == 0) atomicExch(A.status, FB_ST_WAIT_TIMEOUT);
            break;
        }
        const uint32_t st = ring_u + s * GU_STAGE_BYTES + 16 * lane;
        float fg, fu;
        {
            const uint4 hd = fb_lds128(st);
            uint4 q[8];
#pragma unroll
            for (int k = 0; k < 8; k++) q[k] = fb_lds128(st + 512 * (k + 1));
            fg = fb_dot_q4k(hd, q, a);
        }
        {
            const uint4 hd = fb_lds128(st + FB_Q4K_GROUP);
            uint4 q[8];
#pragma unroll
            for (int k = 0; k < 8; k++) q[k] = fb_lds128(st + FB_Q4K_GROUP + 512 * (k + 1));
            fu = fb_dot_q4k(hd, q, a);
        }
        __syncwarp(); /* every lane has read the stage: refill it */
        if (lane == 0 && i + GU_STAGES < n_my) issue(i + GU_STAGES);
        fg = fb_span_sum(fg, bpr);
        fu = fb_span_sum(fu, bpr);
        const int t = first + i * stride;
        const int slot = t / A.gate_groups, g = t - slot * A.gate_groups;
        const int row = g * rpg + lane / bpr;
        if (lane % bpr == 0 && row < A.inter_local) {
            const float sl = __fdiv_rn(fg, __fadd_rn(1.0f, expf(-fg)));
            A.act[slot * A.inter_local + row] = __fmul_rn(sl, fu);
        }
        const int win = (g * rpg) / FB_QK;
        int last = 0;
        __syncwarp();
        if (lane == 0) {
            __threadfence();
            const unsigned old = atomicAdd(A.counters + FB_CNT_WIN + slot * nwin + win, 1u);
            last = (old == (unsigned)gpw - 1);
        }
        last = __shfl_sync(FULL, last, 0);
        if (last) {
            __threadfence();
            const float *src = A.act + slot * A.inter_local + win * FB_QK + 8 * lane;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = __ldcg(src + j);
            fb_warp_quantize(v, &A.q8a[slot * nwin + win], lane);
            if (lane == 0) A.counters[FB_CNT_WIN + slot * nwin + win] = 0;
        }
    }
}

#define DN_STAGES 2
#define DN_STAGE_BYTES FB_Q6K_GROUP /* room for either type */

/* Down projection + combine inside one block: warp s streams expert slot s's groups, one extra
 * warp adds the experts up in list order as soon as a row group is complete.  No global scratch,
 * no atomics: the per-expert results pass through double-buffered shared memory. */
template <int TYPE>
__global__ void __launch_bounds__(512, 1) k_down_ring(fb_args_t A) {
    extern __shared__ __align__(128) uint8_t dsm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ns = A.n_slots, bpr = A.down_bpr, rpg = 32 / bpr;
    constexpr uint32_t GB = (TYPE == FB_TYPE_Q4_K) ? FB_Q4K_GROUP : FB_Q6K_GROUP;
    uint8_t *rings = dsm;
    float *dots = reinterpret_cast<float *>(dsm + (size_t)ns * DN_STAGES * DN_STAGE_BYTES); /* [2][ns][32] */
    uint64_t *bars = reinterpret_cast<uint64_t *>(dots + 2 * ns * 32);
    /* bars: full[ns][DN_STAGES], ready[2], empty[2] */
    const uint32_t bar0 = fb_smem_u32(bars);
    const uint32_t ready_u = bar0 + 8 * ns * DN_STAGES, empty_u = ready_u + 16;
    if (threadIdx.x == 0) {
        for (int i = 0; i < ns * DN_STAGES; i++) fb_mbar_init(bar0 + 8 * i, 1);
        for (int b = 0; b < 2; b++) {
            fb_mbar_init(ready_u + 8 * b, ns);
            fb_mbar_init(empty_u + 8 * b, 1);
        }
        fb_mbar_init_fence();
    }
    __syncthreads();
    const int n_my = (int)blockIdx.x < A.down_groups ? (A.down_groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (warp < ns) {
        const int slot = warp;
        const uint32_t ring_u = fb_smem_u32(rings + (size_t)slot * DN_STAGES * DN_STAGE_BYTES);
        const uint32_t full_u = bar0 + 8 * slot * DN_STAGES;
        const uint8_t *base = A.slot_rec[slot] + A.down_off;
        auto issue = [&](int i) {
            const int rg = blockIdx.x + i * gridDim.x;
            const uint32_t bar = full_u + 8 * (i % DN_STAGES);
            fb_mbar_expect_tx(bar, GB);
            fb_bulk_g2s(ring_u + (i % DN_STAGES) * DN_STAGE_BYTES, base + (uint64_t)rg * GB, GB, bar);
        };
        if (lane == 0)
            for (int i = 0; i < DN_STAGES && i < n_my; i++) issue(i);
        uint4 a[FB_Q8_U4];
        {
            const uint4 *src = reinterpret_cast<const uint4 *>(A.q8a + slot * bpr + (lane % bpr));
#pragma unroll
            for (int i = 0; i < FB_Q8_U4; i++) a[i] = src[i];
        }
        for (int i = 0; i < n_my; i++) {
            const int s = i % DN_STAGES;
            if (!fb_mbar_wait(full_u + 8 * s, (i / DN_STAGES) & 1)) {
                if (lane == 0) atomicExch(A.status, FB_ST_WAIT_TIMEOUT);
                break;
            }
            const uint32_t st = ring_u + s * DN_STAGE_BYTES + 16 * lane;
            float f;
            if (TYPE == FB_TYPE_Q4_K) {
                const uint4 hd = fb_lds128(st);
                uint4 q[8];
#pragma unroll
                for (int k = 0; k < 8; k++) q[k] = fb_lds128(st + 512 * (k + 1));
                f = fb_dot_q4k(hd, q, a);
            } else {
                uint4 ql[8], qh[4];
#pragma unroll
                for (int k = 0; k < 8; k++) ql[k] = fb_lds128(st + 512 * k);
#pragma unroll
                for (int k = 0; k < 4; k++) qh[k] = fb_lds128(st + 512 * (8 + k));
                const uint4 sc = fb_lds128(st + 512 * 12);
                uint32_t d16;
                asm volatile("ld.shared.u16 %0, [%1];" : "=r"(d16) : "r"(ring_u + s * DN_STAGE_BYTES + FB_Q6K_OFF_D + 2 * lane));
                f = fb_dot_q6k(ql, qh, sc, d16, a);
            }
            __syncwarp();
            if (lane == 0 && i + DN_STAGES < n_my) issue(i + DN_STAGES);
            f = fb_span_sum(f, bpr);
            const int buf = i & 1;
            if (i >= 2 && !fb_mbar_wait(empty_u + 8 * buf, ((i >> 1) - 1) & 1)) {
                if (lane == 0) atomicExch(A.status, FB_ST_WAIT_TIMEOUT);
                break;
            }
            if (lane % bpr == 0) dots[(buf * ns + slot) * 32 + lane / bpr] = f;
            __syncwarp();
            if (lane == 0) fb_mbar_arrive(ready_u + 8 * buf);
        }
    } else if (warp == ns) {
        for (int i = 0; i < n_my; i++) {
            const int buf = i & 1, rg = blockIdx.x + i * gridDim.x;
            if (!fb_mbar_wait(ready_u + 8 * buf, (i >> 1) & 1)) {
                if (lane == 0) atomicExch(A.status, FB_ST_WAIT_TIMEOUT);
                break;
            }
            const int r = rg * rpg + lane;
            if (lane < rpg && r < A.n_embd) {
                float acc = A.accumulate ? A.moe_out[r] : 0.0f;
                for (int s = 0; s < A.top_k; s++) acc = __fmaf_rn(A.scores[s], dots[(buf * ns + s) * 32 + lane], acc);
                if (A.has_shared) {
                    const float sh = dots[(buf * ns + A.top_k) * 32 + lane];
                    acc = __fadd_rn(acc, A.shared_gate_w ? __fmul_rn(sh, __ldcg(A.scores + A.top_k)) : sh);
                }
                A.moe_out[r] = acc;
            }
            __syncwarp();
            if (lane == 0) fb_mbar_arrive(empty_u + 8 * buf);
        }
    }
}

/* ------------------------------------------------------------------ launchers */
extern "C" int fb_launch_prologue(const fb_args_t *a, int flags, void *stream) {
    k_prologue<<<1, 1024, 0, (cudaStream_t)stream>>>(*a, flags);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_router(const fb_args_t *a, int grid, void *stream) {
    k_router<<<grid, 256, 0, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_set_slots(const fb_args_t *a, void *stream) {
    k_set_slots<<<1, 32, 0, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_gate_up(const fb_args_t *a, int grid, void *stream) {
    const size_t sm = (size_t)a->gate_bpr * sizeof(fb_q8_entry_t);
    if (a->gate_type == FB_TYPE_Q6_K) k_gate_up<FB_TYPE_Q6_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    else k_gate_up<FB_TYPE_Q4_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_gate_up_ring(const fb_args_t *a, int grid, void *stream) {
    if (a->gate_type != FB_TYPE_Q4_K) return (int)cudaErrorInvalidValue; /* the rings are sized for Q4_K groups */
    const size_t sm = (size_t)GU_WARPS * GU_STAGES * GU_STAGE_BYTES + (size_t)GU_WARPS * GU_STAGES * 8;
    static unsigned char configured[FB_MAX_DEVICES];
    int dev;
    if (!fb_device_once(configured, dev)) {
        cudaError_t e = cudaFuncSetAttribute(k_gate_up_ring, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = 1;
    }
    k_gate_up_ring<<<grid, GU_WARPS * 32, sm, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_down_ring(const fb_args_t *a, int grid, void *stream) {
    if (a->down_type == FB_TYPE_Q5_K || a->down_half >= 0) {
        /* no ring variant for Q5_K or half super-blocks: the plain kernel with its own grid (8 warps per block) */
        const int tasks = a->n_slots * a->down_groups, g = (tasks + 7) / 8;
        return fb_launch_down(a, g < 1 ? 1 : (g > 2 * grid ? 2 * grid : g), stream);
    }
    const int ns = a->n_slots;
    const size_t sm = (size_t)ns * DN_STAGES * DN_STAGE_BYTES + sizeof(float) * 2 * ns * 32 + 8 * (ns * DN_STAGES + 4);
    static unsigned char configured[FB_MAX_DEVICES];
    int dev;
    if (!fb_device_once(configured, dev)) {
        const int mx = FB_MAX_SLOTS * DN_STAGES * DN_STAGE_BYTES + 4 * 2 * FB_MAX_SLOTS * 32 + 8 * (FB_MAX_SLOTS * DN_STAGES + 4);
        cudaError_t e = cudaFuncSetAttribute(k_down_ring<FB_TYPE_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, mx);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(k_down_ring<FB_TYPE_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, mx);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = 1;
    }
    if (a->down_type == FB_TYPE_Q4_K)
        k_down_ring<FB_TYPE_Q4_K><<<grid, (ns + 1) * 32, sm, (cudaStream_t)stream>>>(*a);
    else
        k_down_ring<FB_TYPE_Q6_K><<<grid, (ns + 1) * 32, sm, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_down(const fb_args_t *a, int grid, void *stream) {
    const size_t sm = (size_t)a->n_slots * a->down_bpr * sizeof(fb_q8_entry_t);
    if (a->down_half >= 0) {
        if (a->down_type == FB_TYPE_Q4_K)
            k_down<FB_TYPE_Q4_K_H><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
        else if (a->down_type == FB_TYPE_Q6_K)
            k_down<FB_TYPE_Q6_K_H><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
        else if (a->down_type == FB_TYPE_Q5_K)
            k_down<FB_TYPE_Q5_K_H><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
        else
            return (int)cudaErrorInvalidValue;
    } else if (a->down_type == FB_TYPE_Q4_K)
        k_down<FB_TYPE_Q4_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    else if (a->down_type == FB_TYPE_Q5_K)
        k_down<FB_TYPE_Q5_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    else
        k_down<FB_TYPE_Q6_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}
