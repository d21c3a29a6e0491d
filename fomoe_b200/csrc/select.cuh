/*
 * select.cuh -- block-wide routing decision for the persistent stack kernel (512 threads, one per expert).
 *
 * Same result as route.cuh's single-warp routine, built for latency:
 *   1. every warp sorts its 32 (logit, expert) pairs with a shuffle bitonic network, best first;
 *   2. the best 16 of each warp are merged pairwise (bitonic merges that keep the better half) down to the block's
 *      best 16;
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

/* One level of the merge tree: warp w < NL takes sorted lists 2w and 2w+1 (16 entries each, best first) from `sv/si`,
 * lays them out as one bitonic run (the second list reversed into lanes 16..31), sorts it with the five
 * compare-exchange steps of a bitonic merge and leaves its best 16 as list w of `dv/di`. */
template <int NL>
__device__ __forceinline__ void fb_merge_level(const float (*sv)[16], const int (*si)[16], float (*dv)[16],
                                               int (*di)[16], int warp, int lane) {
    if (warp < NL) {
        const int src = 2 * warp + (lane >> 4), pos = (lane < 16) ? lane : 31 - lane;
        float v = sv[src][pos];
        int id = si[src][pos];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) fb_cmpx(v, id, d, (lane & d) == 0);
        if (lane < 16) {
            dv[warp][lane] = v;
            di[warp][lane] = id;
        }
    }
    __syncthreads();
}

/* The block's best 16 of one (value, id) pair per thread, in order (value descending, lower id first), left in
 * W->lv[1][slot][*] / W->li[1][slot][*].  Every warp sorts its 32 pairs with a shuffle network; the sixteen lists of
 * 16 are then halved four times (8, 4, 2, 1 warps), each step a 5-stage bitonic merge of two lists that keeps the
 * better half, ping-ponging between W->lv[0] and rows 4..11 of W->lv[1].  (Ranking all 256 candidates at once by
 * binary search in the other lists took one barrier instead of four but 900 instructions per thread: twice as
 * long.)  Called by all 512 threads.  Out of line and shared by the selection proper, its repeat after the near-tie
 * arbiter and cache-aware routing: one copy of this code stays in the instruction cache from layer to layer
 * (inlined at each use the stack kernel's hot path outgrew the cache, and every phase of every layer slowed down
 * by a third). */
static __device__ __noinline__ void fb_block_best16(fb_sel_smem_t *W, float v, int id, int slot) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    fb_sort32(v, id, lane);
    if (lane < 16) {
        W->lv[0][warp][lane] = v;
        W->li[0][warp][lane] = id;
    }
    __syncthreads();
    fb_merge_level<8>(W->lv[0], W->li[0], W->lv[1] + 4, W->li[1] + 4, warp, lane);
    fb_merge_level<4>(W->lv[1] + 4, W->li[1] + 4, W->lv[0], W->li[0], warp, lane);
    fb_merge_level<2>(W->lv[0], W->li[0], W->lv[1] + 4, W->li[1] + 4, warp, lane);
    fb_merge_level<1>(W->lv[1] + 4, W->li[1] + 4, W->lv[1] + slot, W->li[1] + slot, warp, lane);
}

/* Cache-aware routing over one residency tier (src/car.c:36-264; classify as src/gpu_kernels.hip:7097-7149) on the
 * renormalised selection in W->ci / W->cv.  The CPU walks the uncached positions in list order and, for each, scans
 * all experts for the best-scoring resident one that is neither selected nor already taken as a substitute; it is
 * accepted (and from then on taken) when its score is at least `threshold` times the original's.  A rejected
 * candidate stays available, so position after position meets the SAME ordered list of resident, unselected experts
 * and moves one entry down it per acceptance: the list's first top_k entries are all that can ever be used.  The
 * block forms that list once (every thread offers its expert's probability if it is resident, not selected and
 * positive; best 16 by (probability descending, lower index first), the CPU's scan order) and one thread walks it.
 * Substitutions touch only their own slot, so the order in which the CPU applies them (by ratio) does not matter
 * while its per-token budgets are off, as they are by default.  Called by all threads; returns (in warp 0) the
 * number of substitutions. */
__device__ __forceinline__ int fb_select_car(const fb_args_t &A, fb_sel_smem_t *W, const float *all_scores, float my_p,
                                             uint32_t my_resident_word) {
    const int tid = threadIdx.x, nE = A.n_experts, k = A.top_k;
    bool eligible = tid < nE && ((my_resident_word >> (tid & 31)) & 1u) && my_p > 0.0f;
    for (int r = 0; r < k; r++)
        if (W->ci[r] == tid) eligible = false;
    /* warp w holds mask word w: parked in shared memory for the walk below (a global load per position costs a
     * trip to L2 each) */
    if ((tid & 31) == 0) W->li[1][3][tid >> 5] = (int)my_resident_word;
    fb_block_best16(W, eligible ? my_p : -INFINITY, eligible ? tid : 0x7fffffff, 1);
    int nc = 0;
    if (tid == 0) {
        int next = 0;
        bool any = false;
        for (int r = 0; r < k && next < 16; r++) {
            const int orig = W->ci[r];
            if (((uint32_t)W->li[1][3][orig >> 5] >> (orig & 31)) & 1u) continue; /* cached */
            const float bv = W->lv[1][1][next];
            const int bi = W->li[1][1][next];
            if (bi == 0x7fffffff) break; /* no resident expert left to offer */
            const float ov = all_scores[orig];
            const float ratio = (ov > 0.0f) ? __fdiv_rn(bv, ov) : 0.0f;
            if (ratio >= A.car_threshold) {
                W->ci[r] = bi;
                W->cv[r] = A.car_dampen ? __fmul_rn(W->cv[r], ratio) : bv;
                next++; /* taken: later positions see the next entry */
                nc++;
                any = true;
            }
        }
        if (any && !A.car_dampen) {
            float s2 = 0.0f;
            for (int r = 0; r < k; r++) s2 = __fadd_rn(s2, W->cv[r]);
            if (s2 > 0.0f) {
                const float i2 = __fdiv_rn(1.0f, s2);
                for (int r = 0; r < k; r++) W->cv[r] = __fmul_rn(W->cv[r], i2);
            }
        }
        W->li[1][2][0] = nc;
    }
    __syncthreads();
    return W->li[1][2][0];
}

/* Must be called by all 512 threads of the block.  Outputs (shared memory): ids[n_slots], scores[n_slots],
 * ids_orig[top_k], slot_rec[n_slots], all_scores[n_experts].  `leader` updates the global counters;
 * `shared_score` is the weight of the shared expert's slot; `rec` (leader only, may be NULL) receives the decision
 * for the routing trace; `logit(expert)` fetches a router logit; `early(const int *candidates)` is called by every
 * thread as soon as the selected ids are known. */
template <class Logit, class Early>
__device__ void fb_block_select(const fb_args_t &A, fb_sel_smem_t *W, const float *h_smem, float *all_scores, int *ids,
                                int *ids_orig, float *scores, const uint8_t **slot_rec, bool leader, float shared_score,
                                fb_route_rec_t *rec, Logit logit, Early early) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nE = A.n_experts, k = A.top_k, kk = min(k + 1, nE);
    float lg = (tid < nE) ? logit(tid) : -INFINITY;
    /* cache-aware routing on for this layer?  (the same for every thread; its mask word is requested now) */
    const bool car_on = A.resident && A.car_threshold > 0.0f && A.car_threshold < 1.0f;
    const uint32_t res_word = car_on ? __ldg(A.resident + (tid >> 5)) : 0u;

#pragma unroll 1
    for (int pass = 0; pass < 2; pass++) {
        fb_block_best16(W, lg, (tid < nE) ? tid : 0x7fffffff, 0);
        /* best 16 now in lv[1][0][*] */
        if (pass == 1) break;
        /* lane r compares candidates r and r+1 (every warp does the same, so the flags need no broadcast) */
        const float ca = W->lv[1][0][lane & 15], cb = W->lv[1][0][(lane + 1) & 15];
        const uint32_t close = __ballot_sync(FULL, lane + 1 < kk && ca - cb <= FB_TIE_TOL * fmaxf(1.0f, fabsf(ca)));
        const uint32_t flag = close | (close << 1);
        if (!flag) break;
        bool mine = false;
        for (int r = 0; r < kk; r++)
            if (((flag >> r) & 1u) && W->li[1][0][r] == tid) mine = true;
        if (mine) lg = fb_exact_logit(A, h_smem, tid);
        __syncthreads();
    }

    /* The selected experts are known now, as W->li[1][0][0..k-1]; only their weights (and, rarely, their order or a
     * cache-aware substitute) are still to come.  The caller may start fetching what it will read first. */
    early(W->li[1][0]);

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
    }

    /* ---- CAR (all threads) ---- */
    int n_subs = 0;
    if (car_on) {
        __syncthreads(); /* warp 0 has left the selection before substitution in W->ci / W->cv */
        n_subs = fb_select_car(A, W, all_scores, p, res_word);
    }

    if (warp == 0) {
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
