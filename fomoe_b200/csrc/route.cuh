/*
 * route.cuh -- softmax, ordered top-k, renormalise and cache-aware routing in one warp.
 * Shared by the per-phase router kernel and the persistent stack kernel.
 */
#pragma once
#include <math.h>
#include <stdint.h>

#include "launch.h"

#ifndef FULL
#define FULL 0xffffffffu
#endif

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
static __device__ void fb_route_select(const fb_args_t &A, int lane, bool leader) {
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
    /* the routing log (when attached) keeps this layer-token's decision for the trace writer */
    fb_route_rec_t *rec = (leader && A.route_log) ? A.route_log + (size_t)(*A.tok_ctr) * A.route_stride : nullptr;
    if (lane == 0)
        for (int r = 0; r < k; r++) {
            A.ids_orig[r] = cand_id[r];
            if (rec) {
                rec->ids_orig[r] = cand_id[r];
                rec->scores_orig[r] = cand_v[r];
            }
        }
    if (leader && A.freq && lane < k) {
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
            if (rec) {
                rec->ids[r] = e;
                rec->scores[r] = cand_v[r];
            }
        }
        if (A.has_shared) {
            A.ids[k] = nE;
            A.scores[k] = A.shared_gate_w ? __ldcg(A.shared_gate) : 1.0f; /* weight 1, or its scalar gate */
            A.slot_rec[k] = A.table_layer + (uint64_t)nE * A.rec_bytes;
        }
        if (leader && n_subs) atomicAdd(A.counters + FB_CNT_SUBS, (unsigned)n_subs);
    }
}

