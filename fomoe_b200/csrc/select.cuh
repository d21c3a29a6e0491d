/*
 * select.cuh -- block-wide routing decision for the persistent stack kernel (512 threads, one per expert).
 *
 * Same result as route.cuh's single-warp routine, built for latency:
 *   1. every warp sorts its 32 (logit, expert) pairs with a shuffle bitonic network, best first;
 *   2. the best 16 of each warp (256 candidates) are merged by rank: every candidate counts, by binary search in
 *      the other 15 sorted lists, how many entries beat it; ranks 0..15 are the block's best 16;
 *   3. near-ties among the best k+1 are recomputed in the CPU's summation order (src/tensor.c:104-113) and the
 *      ranking repeated, so the selected ids match the CPU's top_k (src/tensor.c:226-252) index for index;
 *   4. softmax over all experts (src/tensor.c:186-200), renormalised top-k weights (src/inference.c:496-502);
 *   5. cache-aware routing over one residency tier (src/car.c:36-264, classify src/gpu_kernels.hip:7097-7149).
 * Ordering everywhere is (value descending, lower index first).
 */
#pragma once
#include <math.h>
#include <stdint.h>

#include "launch.h"
#include "route.cuh"

/* Two logits closer than this (relative to max(1, |logit|)) are re-summed in the CPU's order.  The block's
 * reduction and the CPU's sequential loop differ by a few 1e-6 at the 397B router's scale (4096 terms of
 * magnitude 1e-2), so 4e-5 leaves an order of magnitude of margin while triggering in under 1 % of layers. */
#define FB_TIE_TOL 4e-5f

struct fb_sel_smem_t {
    float lv[2][16][16];
    int li[2][16][16];
    float psum[16];
    float cv[16]; /* working copy of the candidates: scores */
    int ci[16];   /* ... and expert ids */
};

__device__ __forceinline__ void fb_cmpx(float &v, int &i, int d, bool keep_better) {
    const float ov = __shfl_xor_sync(FULL, v, d);
    const int oi = __shfl_xor_sync(FULL, i, d);
    const bool other_better = fb_better(ov, oi, v, i);
    if (other_better == keep_better) {
        v = ov;
        i = oi;
    }
}

/* full bitonic sort of one value per lane, best first */
__device__ __forceinline__ void fb_sort32(float &v, int &i, int lane) {
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            const bool up = (lane & k) == 0 || k == 32;
            const bool lower = (lane & j) == 0;
            fb_cmpx(v, i, j, lower == up);
        }
    }
}

/* One router row re-summed in the CPU's order: sequential multiply-then-add (src/tensor.c:104-113).  Rarely called
 * and kept out of line so that its unrolled body does not sit in the instruction stream of every layer. */
static __device__ __noinline__ float fb_exact_logit(const fb_args_t &A, const float *h_smem, int row) {
    const float4 *w = reinterpret_cast<const float4 *>(A.router_w + (size_t)row * A.n_embd);
    const float4 *hh = reinterpret_cast<const float4 *>(h_smem);
    float exact = 0.0f;
    for (int j0 = 0; j0 < A.n_embd / 4; j0 += 8) {
        float4 wv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) wv[u] = __ldg(w + j0 + u);
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const float4 hv = hh[j0 + u];
            exact = __fadd_rn(exact, __fmul_rn(wv[u].x, hv.x));
            exact = __fadd_rn(exact, __fmul_rn(wv[u].y, hv.y));
            exact = __fadd_rn(exact, __fmul_rn(wv[u].z, hv.z));
            exact = __fadd_rn(exact, __fmul_rn(wv[u].w, hv.w));
        }
    }
    return exact;
}

/* Cache-aware routing over one residency tier (src/car.c:36-264; classify as src/gpu_kernels.hip:7097-7149), run by
 * one warp on the renormalised selection in W->ci / W->cv.  Returns the number of substitutions.  Out of line: it
 * only runs when a residency mask and a threshold inside (0, 1) are set. */
static __device__ __noinline__ int fb_select_car(const fb_args_t &A, fb_sel_smem_t *W, const float *all_scores, int lane) {
    const int nE = A.n_experts, k = A.top_k;
    int n_subs = 0;

    uint32_t res = 0, sel = 0; /* bit j <-> expert j*32 + lane */
#pragma unroll
    for (int j = 0; j < FB_EPL; j++)
        if ((__ldg(A.resident + j) >> lane) & 1u) res |= 1u << j;
    for (int r = 0; r < k; r++) {
        const int e = W->ci[r];
        if ((e & 31) == lane) sel |= 1u << (e >> 5);
    }
    int c_idx[FB_MAX_TOPK], c_best[FB_MAX_TOPK];
    float c_score[FB_MAX_TOPK], c_ratio[FB_MAX_TOPK];
    int nc = 0;
    for (int r = 0; r < k; r++) {
        const int orig = W->ci[r];
        if ((__ldg(A.resident + (orig >> 5)) >> (orig & 31)) & 1u) continue; /* cached: uniform */
        float bv = 0.0f; /* strict improvement over 0: src/car.c:104-112 */
        int bi = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < FB_EPL; j++) {
            const int e = j * 32 + lane;
            if (((res >> j) & 1u) && !((sel >> j) & 1u) && e < nE) {
                const float pe = all_scores[e];
                if (pe > 0.0f && fb_better(pe, e, bv, bi)) {
                    bv = pe;
                    bi = e;
                }
            }
        }
        fb_warp_best(bv, bi);
        const float ov = all_scores[orig];
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
    for (int a = 1; a < nc; a++) { /* stable insertion by ratio descending (src/car.c:168-176) */
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
    if (lane == 0) {
        for (int c = 0; c < nc; c++) {
            const int r = c_idx[c];
            W->ci[r] = c_best[c];
            W->cv[r] = A.car_dampen ? __fmul_rn(W->cv[r], c_ratio[c]) : c_score[c];
        }
        if (nc > 0 && !A.car_dampen) {
            float s2 = 0.0f;
            for (int r = 0; r < k; r++) s2 = __fadd_rn(s2, W->cv[r]);
            if (s2 > 0.0f) {
                const float i2 = __fdiv_rn(1.0f, s2);
                for (int r = 0; r < k; r++) W->cv[r] = __fmul_rn(W->cv[r], i2);
            }
        }
    }
    n_subs = nc;
    __syncwarp();
    return n_subs;
}

/* Must be called by all 512 threads of the block.  Outputs (shared memory): ids[n_slots], scores[n_slots],
 * ids_orig[top_k], slot_rec[n_slots], all_scores[n_experts].  `leader` updates the global counters;
 * `shared_score` is the weight of the shared expert's slot; `rec` (leader only, may be NULL) receives the decision
 * for the routing trace. */
__device__ void fb_block_select(const fb_args_t &A, fb_sel_smem_t *W, const float *h_smem, float *all_scores, int *ids,
                                int *ids_orig, float *scores, const uint8_t **slot_rec, bool leader,
                                float shared_score = 1.0f, fb_route_rec_t *rec = nullptr) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nE = A.n_experts, k = A.top_k, kk = min(k + 1, nE);
    float lg = (tid < nE) ? __ldcg(A.logits + tid) : -INFINITY;

    for (int pass = 0; pass < 2; pass++) {
        float v = lg;
        int id = (tid < nE) ? tid : 0x7fffffff;
        fb_sort32(v, id, lane);
        if (lane < 16) {
            W->lv[0][warp][lane] = v;
            W->li[0][warp][lane] = id;
        }
        __syncthreads();
        /* merge by rank: candidate p of warp list w has p better entries in its own list; a 5-step binary search
         * in each of the other 15 sorted lists counts the rest.  Ranks below 16 are the block's best 16, in order. */
        if (tid < 256) {
            const int w = tid >> 4, p = tid & 15;
            const float mv = W->lv[0][w][p];
            const int mi = W->li[0][w][p];
            int rank = p;
#pragma unroll /* fully unrolled on purpose: the fifteen searches overlap; unrolled by three the selection took 0.4 us longer */
            for (int o = 1; o < 16; o++) {
                const int w2 = (w + o) & 15;
                int pos = 0;
#pragma unroll
                for (int st = 8; st > 0; st >>= 1)
                    if (fb_better(W->lv[0][w2][pos + st - 1], W->li[0][w2][pos + st - 1], mv, mi)) pos += st;
                if (fb_better(W->lv[0][w2][pos], W->li[0][w2][pos], mv, mi)) pos++;
                rank += pos;
            }
            if (rank < 16) {
                W->lv[1][0][rank] = mv;
                W->li[1][0][rank] = mi;
            }
        }
        __syncthreads();
        /* best 16 now in lv[1][0][*] */
        if (pass == 1) break;
        uint32_t flag = 0;
        for (int r = 0; r + 1 < kk; r++) {
            const float a = W->lv[1][0][r], b = W->lv[1][0][r + 1];
            if (a - b <= FB_TIE_TOL * fmaxf(1.0f, fabsf(a))) flag |= (1u << r) | (1u << (r + 1));
        }
        if (!flag) break;
        bool mine = false;
        for (int r = 0; r < kk; r++)
            if (((flag >> r) & 1u) && W->li[1][0][r] == tid) mine = true;
        if (mine) lg = fb_exact_logit(A, h_smem, tid);
        __syncthreads();
    }

    /* softmax: the maximum is the best candidate's logit */
    const float mx = W->lv[1][0][0];
    float p = (tid < nE) ? expf(lg - mx) : 0.0f;
    float ps = p;
    for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(FULL, ps, o);
    if (lane == 0) W->psum[warp] = ps;
    if (tid < 16) {
        W->ci[tid] = W->li[1][0][tid];
    }
    __syncthreads();
    float sum = 0.0f;
#pragma unroll
    for (int w = 0; w < 16; w++) sum += W->psum[w];
    p = __fmul_rn(p, __fdiv_rn(1.0f, sum));
    if (tid < nE) all_scores[tid] = p;
    __syncthreads();

    if (warp == 0) {
        /* lane r holds candidate r.  Equal probabilities order by index like the CPU (src/tensor.c:226-252):
         * the list is already in logit order, so only an exact tie of the rounded probabilities can be out of place */
        int ci = (lane < kk) ? W->ci[lane] : 0x7fffffff;
        float cv = (lane < kk) ? all_scores[ci] : -1.0f;
        {
            const float nv = __shfl_down_sync(FULL, cv, 1);
            const int ni = __shfl_down_sync(FULL, ci, 1);
            const bool bad = (lane + 1 < kk) && fb_better(nv, ni, cv, ci);
            if (__ballot_sync(FULL, bad)) { /* rare: stable insertion by (score desc, index asc) on one lane */
                W->cv[lane & 15] = cv;
                W->ci[lane & 15] = ci;
                __syncwarp();
                if (lane == 0) {
                    for (int a = 1; a < kk; a++) {
                        const float tv = W->cv[a];
                        const int ti = W->ci[a];
                        int b = a - 1;
                        while (b >= 0 && fb_better(tv, ti, W->cv[b], W->ci[b])) {
                            W->cv[b + 1] = W->cv[b];
                            W->ci[b + 1] = W->ci[b];
                            b--;
                        }
                        W->cv[b + 1] = tv;
                        W->ci[b + 1] = ti;
                    }
                }
                __syncwarp();
                cv = (lane < kk) ? W->cv[lane] : -1.0f;
                ci = (lane < kk) ? W->ci[lane] : 0x7fffffff;
            }
        }
        float ssum = 0.0f; /* renormalise: sequential sum in list order (src/inference.c:496-502) */
        for (int r = 0; r < k; r++) ssum = __fadd_rn(ssum, __shfl_sync(FULL, cv, r));
        if (ssum > 0.0f) cv = __fmul_rn(cv, __fdiv_rn(1.0f, ssum));
        if (lane < 16) {
            W->cv[lane] = cv;
            W->ci[lane] = ci;
        }
        if (lane < k) {
            ids_orig[lane] = ci;
            if (rec) { /* routing log: the decision before cache-aware routing */
                rec->ids_orig[lane] = ci;
                rec->scores_orig[lane] = cv;
            }
        }
        __syncwarp();
        if (leader && A.freq && lane < k) atomicAdd(A.freq + W->ci[lane], 1u);

        /* ---- CAR ---- */
        int n_subs = 0;
        if (A.resident && A.car_threshold > 0.0f && A.car_threshold < 1.0f) n_subs = fb_select_car(A, W, all_scores, lane);
        if (lane < k) {
            int e = W->ci[lane];
            if (e < 0 || e >= nE) {
                atomicExch(A.status, FB_ST_BAD_ID);
                e = 0;
            }
            ids[lane] = e;
            scores[lane] = W->cv[lane];
            slot_rec[lane] = A.table_layer + (uint64_t)e * A.rec_bytes;
            if (rec) {
                rec->ids[lane] = e;
                rec->scores[lane] = W->cv[lane];
            }
        }
        if (lane == 0) {
            if (A.has_shared) {
                ids[k] = nE;
                scores[k] = shared_score; /* 1, or the shared expert's scalar gate */
                slot_rec[k] = A.table_layer + (uint64_t)nE * A.rec_bytes;
            }
            if (leader && n_subs) atomicAdd(A.counters + FB_CNT_SUBS, (unsigned)n_subs);
        }
    }
    __syncthreads();
}
