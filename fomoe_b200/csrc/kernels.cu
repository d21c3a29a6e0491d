/*
 * kernels.cu -- the decode hot path as per-phase kernels (sm_100a):
 *
 *   k_prologue   x += moe_out (+ resid); h = rmsnorm(x) * w; q8h = Q8_K(h)
 *   k_router     fp32 router logits (warp per expert row); the last block to finish runs
 *                softmax, ordered top-k, renormalise and CAR substitute-and-dampen in one warp
 *   k_gate_up    Q4_K gate and up dequant-matvec of every selected expert + the shared expert,
 *                SwiGLU in the epilogue; the last warp to finish a 256-row window quantises it
 *   k_down       Q4_K / Q6_K down dequant-matvec per expert; the last warp to finish a row group
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

#define FULL 0xffffffffu

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
__device__ __forceinline__ bool fb_better(float av, int ai, float bv, int bi) {
    return av > bv || (av == bv && ai < bi);
}

/* warp-wide arg-best over (value desc, index asc); every lane returns the winner */
__device__ __forceinline__ void fb_warp_best(float &v, int &i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(FULL, v, o);
        const int oi = __shfl_xor_sync(FULL, i, o);
        if (fb_better(ov, oi, v, i)) {
            v = ov;
            i = oi;
        }
    }
}

#define FB_EPL 16 /* experts per lane: 512 / 32 */

/* Softmax, ordered top-k, renormalise and cache-aware routing in one warp.
 *
 * Ordering rule is the CPU's (src/tensor.c:226-252): value descending, lower index first on
 * ties.  The fast logits are summed in a different order from the CPU's sequential loop
 * (src/tensor.c:104-113), so whenever two neighbours among the best k+1 are closer than
 * `tie_tol` the affected rows are recomputed in exactly the CPU's order (sequential
 * multiply-then-add) before ranking.  CAR follows src/car.c:36-264 with one residency tier. */
__device__ void fb_route_select(const fb_args_t &A, int lane) {
    const int nE = A.n_experts, k = A.top_k;
    float lg[FB_EPL];
#pragma unroll
    for (int j = 0; j < FB_EPL; j++) {
        const int e = j * 32 + lane;
        lg[j] = (e < nE) ? __ldcg(A.logits + e) : -INFINITY;
    }
    int cand_id[FB_MAX_TOPK + 1];
    float cand_v[FB_MAX_TOPK + 1];
    const int kk = min(k + 1, nE);

    for (int pass = 0; pass < 2; pass++) {
        uint32_t taken = 0;
        for (int r = 0; r < kk; r++) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
#pragma unroll
            for (int j = 0; j < FB_EPL; j++) {
                const int e = j * 32 + lane;
                if (e < nE && !((taken >> j) & 1u) && fb_better(lg[j], e, bv, bi)) {
                    bv = lg[j];
                    bi = e;
                }
            }
            fb_warp_best(bv, bi);
            cand_id[r] = bi;
            cand_v[r] = bv;
            if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
        }
        if (pass == 1) break;
        /* near-tie arbiter */
        uint32_t flag = 0;
        for (int r = 0; r + 1 < kk; r++) {
            const float tol = 1e-4f * fmaxf(1.0f, fabsf(cand_v[r]));
            if (cand_v[r] - cand_v[r + 1] <= tol) flag |= (1u << r) | (1u << (r + 1));
        }
        if (!flag) break;
        /* lane r recomputes row cand_id[r] in the CPU's order */
        float exact = 0.0f;
        int my_row = -1;
        for (int r = 0; r < kk; r++)
            if (r == lane && ((flag >> r) & 1u)) my_row = cand_id[r];
        if (my_row >= 0) {
            const float *w = A.router_w + (size_t)my_row * A.n_embd;
            for (int j = 0; j < A.n_embd; j++) exact = __fadd_rn(exact, __fmul_rn(__ldg(w + j), __ldcg(A.h + j)));
        }
        for (int r = 0; r < kk; r++) {
            if (!((flag >> r) & 1u)) continue;
            const float ev = __shfl_sync(FULL, exact, r);
            const int e = cand_id[r];
            if ((e & 31) == lane) {
#pragma unroll
                for (int j = 0; j < FB_EPL; j++)
                    if (j == (e >> 5)) lg[j] = ev;
                A.logits[e] = ev;
            }
        }
    }

    /* softmax over all experts (src/tensor.c:186-200) */
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < FB_EPL; j++) mx = fmaxf(mx, lg[j]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, o));
    float p[FB_EPL], sum = 0.0f;
#pragma unroll
    for (int j = 0; j < FB_EPL; j++) {
        const int e = j * 32 + lane;
        p[j] = (e < nE) ? expf(lg[j] - mx) : 0.0f;
        sum += p[j];
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(FULL, sum, o);
    const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
    for (int j = 0; j < FB_EPL; j++) {
        const int e = j * 32 + lane;
        p[j] = __fmul_rn(p[j], inv);
        if (e < nE) A.all_scores[e] = p[j];
    }
    /* scores of the candidates; equal probabilities order by index like the CPU */
    for (int r = 0; r < kk; r++) {
        const int e = cand_id[r];
        float v = 0.0f;
#pragma unroll
        for (int j = 0; j < FB_EPL; j++)
            if (j == (e >> 5)) v = p[j];
        cand_v[r] = __shfl_sync(FULL, v, e & 31);
    }
    for (int a = 1; a < kk; a++) { /* stable insertion by (score desc, index asc) */
        const float tv = cand_v[a];
        const int ti = cand_id[a];
        int b = a - 1;
        while (b >= 0 && fb_better(tv, ti, cand_v[b], cand_id[b])) {
            cand_v[b + 1] = cand_v[b];
            cand_id[b + 1] = cand_id[b];
            b--;
        }
        cand_v[b + 1] = tv;
        cand_id[b + 1] = ti;
    }
    /* renormalise (src/inference.c:496-502) */
    float ssum = 0.0f;
    for (int r = 0; r < k; r++) ssum = __fadd_rn(ssum, cand_v[r]);
    if (ssum > 0.0f) {
        const float sinv = __fdiv_rn(1.0f, ssum);
        for (int r = 0; r < k; r++) cand_v[r] = __fmul_rn(cand_v[r], sinv);
    }
    if (lane == 0)
        for (int r = 0; r < k; r++) A.ids_orig[r] = cand_id[r];
    if (A.freq && lane < k) {
        int e = 0;
        for (int r = 0; r < k; r++)
            if (r == lane) e = cand_id[r];
        atomicAdd(A.freq + e, 1u); /* histogram counts the ids before substitution (src/gpu_kernels.hip:7832-7835) */
    }

    /* ---- CAR ---- */
    int n_subs = 0;
    if (A.resident && A.car_threshold > 0.0f && A.car_threshold < 1.0f) {
        /* per-lane view: bit j <-> expert j*32 + lane */
        uint32_t res = 0, sel = 0;
#pragma unroll
        for (int j = 0; j < FB_EPL; j++)
            if ((__ldg(A.resident + j) >> lane) & 1u) res |= 1u << j;
        for (int r = 0; r < k; r++)
            if ((cand_id[r] & 31) == lane) sel |= 1u << (cand_id[r] >> 5);
        int c_idx[FB_MAX_TOPK], c_best[FB_MAX_TOPK];
        float c_score[FB_MAX_TOPK], c_ratio[FB_MAX_TOPK];
        int nc = 0;
        for (int r = 0; r < k; r++) {
            const int orig = cand_id[r];
            const bool cached = (__ldg(A.resident + (orig >> 5)) >> (orig & 31)) & 1u;
            if (cached) continue; /* uniform across the warp */
            float bv = 0.0f; /* strict improvement over 0: src/car.c:104-112 */
            int bi = 0x7fffffff;
#pragma unroll
            for (int j = 0; j < FB_EPL; j++) {
                const int e = j * 32 + lane;
                if (((res >> j) & 1u) && !((sel >> j) & 1u) && e < nE && p[j] > 0.0f && fb_better(p[j], e, bv, bi)) {
                    bv = p[j];
                    bi = e;
                }
            }
            fb_warp_best(bv, bi);
            float ov = 0.0f;
#pragma unroll
            for (int j = 0; j < FB_EPL; j++)
                if (j == (orig >> 5)) ov = p[j];
            ov = __shfl_sync(FULL, ov, orig & 31);
            const float ratio = (ov > 0.0f) ? __fdiv_rn(bv, ov) : 0.0f;
            if (bi != 0x7fffffff && ratio >= A.car_threshold) {
                c_idx[nc] = r;
                c_best[nc] = bi;
                c_score[nc] = bv;
                c_ratio[nc] = ratio;
                nc++;
                if ((bi & 31) == lane) sel |= 1u << (bi >> 5); /* reserved at once */
            }
        }
        /* stable insertion sort by ratio descending (src/car.c:168-176); application order only
         * matters with budgets, which are off, but keep the reference's order */
        for (int a = 1; a < nc; a++) {
            const int ti = c_idx[a], tb = c_best[a];
            const float ts = c_score[a], tr = c_ratio[a];
            int b = a - 1;
            while (b >= 0 && c_ratio[b] < tr) {
                c_idx[b + 1] = c_idx[b];
                c_best[b + 1] = c_best[b];
                c_score[b + 1] = c_score[b];
                c_ratio[b + 1] = c_ratio[b];
                b--;
            }
            c_idx[b + 1] = ti;
            c_best[b + 1] = tb;
            c_score[b + 1] = ts;
            c_ratio[b + 1] = tr;
        }
        for (int c = 0; c < nc; c++) {
            for (int r = 0; r < k; r++) {
                if (r == c_idx[c]) {
                    cand_id[r] = c_best[c];
                    cand_v[r] = A.car_dampen ? __fmul_rn(cand_v[r], c_ratio[c]) : c_score[c];
                }
            }
        }
        n_subs = nc;
        if (nc > 0 && !A.car_dampen) {
            float s2 = 0.0f;
            for (int r = 0; r < k; r++) s2 = __fadd_rn(s2, cand_v[r]);
            if (s2 > 0.0f) {
                const float i2 = __fdiv_rn(1.0f, s2);
                for (int r = 0; r < k; r++) cand_v[r] = __fmul_rn(cand_v[r], i2);
            }
        }
    }
    if (lane == 0) {
        for (int r = 0; r < k; r++) {
            int e = cand_id[r];
            if (e < 0 || e >= nE) {
                atomicExch(A.status, FB_ST_BAD_ID);
                e = 0;
            }
            A.ids[r] = e;
            A.scores[r] = cand_v[r];
            A.slot_rec[r] = A.table_layer + (uint64_t)e * A.rec_bytes;
        }
        if (A.has_shared) {
            A.ids[k] = nE;
            A.scores[k] = 1.0f;
            A.slot_rec[k] = A.table_layer + (uint64_t)nE * A.rec_bytes;
        }
        if (n_subs) atomicAdd(A.counters + FB_CNT_SUBS, (unsigned)n_subs);
    }
}

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
    if (warp == 0) fb_route_select(A, lane);
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
        const uint4 *pg = reinterpret_cast<const uint4 *>(rec + (uint64_t)g * FB_Q4K_GROUP) + lane;
        const uint4 *pu = reinterpret_cast<const uint4 *>(rec + A.up_off + (uint64_t)g * FB_Q4K_GROUP) + lane;
        uint4 hg = ldg_stream(pg), hu = ldg_stream(pu);
        uint4 qg[8], qu[8];
#pragma unroll
        for (int i = 0; i < 8; i++) qg[i] = ldg_stream(pg + 32 * (i + 1));
#pragma unroll
        for (int i = 0; i < 8; i++) qu[i] = ldg_stream(pu + 32 * (i + 1));
        float fg = fb_dot_q4k(hg, qg, a);
        float fu = fb_dot_q4k(hu, qu, a);
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
        if (TYPE == FB_TYPE_Q4_K) {
            const uint4 *p = reinterpret_cast<const uint4 *>(rec + (uint64_t)rg * FB_Q4K_GROUP) + lane;
            uint4 hd = ldg_stream(p);
            uint4 q[8];
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = ldg_stream(p + 32 * (i + 1));
            f = fb_dot_q4k(hd, q, a);
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
                if (A.has_shared) acc = __fadd_rn(acc, __ldcg(A.dots + A.top_k * A.n_embd + r));
                A.moe_out[r] = acc;
            }
            if (lane == 0) cnt_rg[rg] = 0;
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
    k_gate_up<<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_down(const fb_args_t *a, int grid, void *stream) {
    const size_t sm = (size_t)a->n_slots * a->down_bpr * sizeof(fb_q8_entry_t);
    if (a->down_type == FB_TYPE_Q4_K)
        k_down<FB_TYPE_Q4_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    else
        k_down<FB_TYPE_Q6_K><<<grid, 256, sm, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}
