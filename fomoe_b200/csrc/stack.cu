/*
 * stack.cu -- the whole decode stack as ONE persistent kernel (sm_100a).
 *
 * One block per SM stays resident for every layer of every token of a run and walks the
 * phases of a routed-MoE layer itself, so nothing returns to the host between the router
 * and the experts (the reference synchronises with the host once per layer to classify
 * and run car_evaluate, src/gpu_kernels.hip:6984, 7097-7187) and no kernel boundary drains
 * the memory pipeline:
 *
 *   P0  every block, redundantly: x += moe_out(prev) + resid; h = rmsnorm(x) * w; q8h = Q8_K(h)
 *       (x lives in registers, 8 elements per thread; src/tensor.c:175-184, src/quant.c:343-375)
 *   P1  router rows are dealt round-robin to the blocks; each thread multiplies its 8 columns of a
 *       row (prefetched into registers before the previous layer's barrier) and the block reduces
 *   --- logits exchanged as {generation, value} words, polled by the threads that rank them ---
 *   SEL every block, redundantly: ordered top-k, softmax, renormalise, CAR (select.cuh); as soon as
 *       the ids are known every warp requests the weights of its first gate/up task
 *   P2  gate/up Q4_K dequant-matvec + SwiGLU: (expert, 32-block group) tasks dealt to 16 warps per
 *       block, weights streamed by bulk copies into per-warp shared-memory rings (stream.cuh)
 *   --- grid barrier (activations) --- the first down groups are already in flight
 *   P3  down Q4_K/Q6_K dequant-matvec over (row group, expert) tasks, then the experts of each row group are
 *       combined in list order with their routing weights into moe_out
 *   --- grid barrier (moe_out), joined at the top of the next layer after its router rows
 *       have been requested ---
 *
 * Grid barriers are an arrival counter plus a generation word in global memory; every
 * spin is bounded and, when a limit runs out, the block raises an abort flag that releases all
 * other blocks, records FB_ST_WAIT_TIMEOUT and returns.  The kernel needs all blocks co-resident:
 * it is launched cooperatively with one block per SM.
 */
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "dots.cuh"
#include "launch.h"
#include "route.cuh"
#include "select.cuh"
#include "stream.cuh"

#define SK_THREADS 512
#ifndef SK_EARLY_ROUNDS
#define SK_EARLY_ROUNDS 0
#endif
#ifndef SK_EARLY_COPY
#define SK_EARLY_COPY 1
#endif
#define SK_WARPS 16
#define SK_DOWN_WARPS 13                              /* warps that run down tasks: 38 tasks per block at the 397B shape = 3 rounds */
#define SK_DN_SLOTS 12                                /* expert slots the down phase can serve */
#define SK_RING_BYTES (SK_DOWN_WARPS * 3 * FB_Q4K_GROUP) /* 179,712 B: 13 warps x 3 stages x 4608 or x 2 stages x 6720 (174,720); gate/up uses 16 x 2 x 4608 of it */
#define SK_RING_BYTES_TP (SK_DOWN_WARPS * 2 * FB_Q6K_GROUP) /* tensor-parallel instances: two stages of up to 6720 bytes */
#define SK_MAX_Q8A 48                                 /* n_slots * down blocks per row */
#define SK_MAX_RG 8                                   /* row groups one block's run of down tasks can touch */
#define SK_BAR_THREAD (SK_THREADS - 32) /* lane 0 of the last warp runs the grid barrier; it issues no copies */

struct sk_smem_t {
    fb_args_t A2[2];                     /* this layer's arguments and, fetched during the down phase, the next layer's */
    fb_q8_entry_t q8h[16];               /* quantised hidden state */
    fb_q8_entry_t q8a[SK_MAX_Q8A];       /* quantised activations of every slot */
    float dots[SK_MAX_RG][SK_DN_SLOTS][32]; /* per-expert down outputs of this block's row groups */
    float red[6][SK_WARPS];             /* four router rows, the shared expert's gate vector, the sum of squares */
    float shared_gate;
    float all_scores[FB_MAX_EXPERTS];
    fb_sel_smem_t sel;
    int ids[FB_MAX_SLOTS], ids_orig[FB_MAX_SLOTS];
    float scores[FB_MAX_SLOTS];
    const uint8_t *slot_rec[FB_MAX_SLOTS];
    int ok;
    uint64_t full[SK_WARPS][3];          /* ring stages */
};

struct sk_bar_t {
    unsigned long long *ctr;  /* [0] arrivals, [16] generation of the last completed barrier */
    int *abort_flag;
    int *status;
    int *host_flags;          /* mapped host memory: the host learns of a given-up wait without a copy */
    unsigned grid;
    unsigned long long base;  /* arrivals before this launch */
    unsigned limit;           /* polls before a wait is given up */
    unsigned epoch;           /* barriers this block has arrived at in this launch */
};

__device__ __forceinline__ int ld_volatile_s32(const int *p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

/* A wait ran out: release every other block (abort flag), record why for fomoe_b200_status, and tell the host,
 * which reads the mapped word after its synchronise and reports the call as failed. */
__device__ __forceinline__ void sk_give_up(const sk_bar_t &B) {
    atomicExch(B.abort_flag, 1);
    atomicExch(B.status, FB_ST_WAIT_TIMEOUT);
    if (B.host_flags) {
        asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(B.host_flags), "r"((int)FB_ST_WAIT_TIMEOUT) : "memory");
    }
}

/* Grid barrier.  Arrivals are counted on one cache line (an atomic that returns the count, so the last block
 * knows it is last); the last block then publishes the barrier's generation number on ANOTHER line, which is the
 * only one the waiting blocks poll, one thread per block.  Measured alternatives were slower: a counter that all
 * blocks poll (3-5 us per barrier), per-block flag words polled by a warp of every block (4-6 us), and exchanging
 * the data itself as {generation, value} words polled by their consumers (5 us for the 512 logits): on this chip
 * many pollers on few L2 lines delay the very stores they wait for.  Both words only ever grow; the host tells the
 * kernel where they stand when a launch starts. */
__device__ __forceinline__ void sk_arrive(sk_bar_t &B, sk_smem_t *S, bool fenced = true) {
    __syncthreads();
    B.epoch++;
    if (threadIdx.x == SK_BAR_THREAD) {
        unsigned long long old;
        /* Release only: what the block wrote is made visible at GPU scope before its arrival counts.  The generation
         * word is then a plain strong store with no fence of its own.  By then every block's data has been visible
         * at GPU scope since before that block's own arrival was counted (its release), the count this thread got
         * back shows all of those arrivals performed, and the store is issued only after that count has returned;
         * the waiting side reads the word with an acquire load and fetches the data from L2 afterwards.  A second
         * fence here (st.release) orders nothing that is not ordered already and cost 0.45 us per barrier, 1.35 us
         * per layer; an acquire on the arrival cost another 0.05.  (Build with -DSK_FENCED_GENERATION for the
         * textbook pattern.) */
#ifdef SK_FENCED_GENERATION
        asm volatile("atom.add.acq_rel.gpu.global.u64 %0, [%1], %2;" : "=l"(old) : "l"(B.ctr), "l"(1ULL) : "memory");
#else
        if (fenced)
            asm volatile("atom.add.release.gpu.global.u64 %0, [%1], %2;" : "=l"(old) : "l"(B.ctr), "l"(1ULL) : "memory");
        else /* everything the block publishes at this barrier validates itself ({generation, value} words) */
            asm volatile("atom.add.relaxed.gpu.global.u64 %0, [%1], %2;" : "=l"(old) : "l"(B.ctr), "l"(1ULL) : "memory");
#endif
        const unsigned long long gen = B.base / B.grid + B.epoch;
        if (old + 1ULL == gen * B.grid) {
#ifdef SK_FENCED_GENERATION
            asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(B.ctr + 16), "l"(gen) : "memory");
#else
            asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(B.ctr + 16), "l"(gen) : "memory");
#endif
        }
    }
}

/* wait: returns false (for every thread of the block) when the wait was given up */
__device__ __forceinline__ bool sk_wait(const sk_bar_t &B, sk_smem_t *S) {
    if (threadIdx.x == SK_BAR_THREAD) {
        const unsigned long long gen = B.base / B.grid + B.epoch;
        int ok = 1;
        unsigned n = 0;
        while (ld_acquire_u64(B.ctr + 16) < gen) {
            if (++n > B.limit || ((n & 63u) == 0 && ld_volatile_s32(B.abort_flag))) {
                ok = 0;
                break;
            }
        }
        if (!ok) sk_give_up(B);
        S->ok = ok;
    }
    __syncthreads();
    return S->ok != 0;
}

/* {generation, fp32 value} in one 8-byte word: data and flag cannot be seen apart, so a hand-over needs no fence */
typedef unsigned long long sk_word_t;

__device__ __forceinline__ void sk_put(sk_word_t *p, float v, uint32_t gen) {
    const sk_word_t w = ((sk_word_t)gen << 32) | (sk_word_t)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

__device__ __forceinline__ sk_word_t sk_get1(const sk_word_t *p) {
    sk_word_t a;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
    return a;
}

/* system scope: the word is written by, or meant for, another GPU; 16 bytes = two words in one load */
__device__ __forceinline__ void sk_get2_sys(const sk_word_t *p, sk_word_t &a, sk_word_t &b) {
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

__device__ __forceinline__ void sk_put_sys(sk_word_t *p, float v, uint32_t gen) {
    const sk_word_t w = ((sk_word_t)gen << 32) | (sk_word_t)__float_as_uint(v);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

/* Tensor-parallel output exchange, receiving side.  Every rank's combine step has stored its partial block output
 * into slot `src` of EVERY rank's receive buffer ([2][tp_size][n_embd] words in this GPU's own memory; the words of
 * generation g lie in half g & 1).  A thread polls its 8 elements of every slot until all carry `gen`, then adds the
 * partials in rank order, so all ranks form bit-identical sums (the reference's tp_allreduce_sum,
 * src/tp.hip:85-124, has the same meaning: out = p_0 + p_1 on both ranks).  false = gave up.
 *
 * Why two halves: a rank may store generation g+1 as soon as it has gathered g from everyone, which does not mean
 * that every block of every peer has read ITS g yet.  With the halves, g+2 is the first generation that reuses
 * g's words, and a rank stores g+2 only after gathering g+1 from every peer; a peer stores g+1 only after all its
 * blocks have passed the grid barriers of that layer, i.e. after all of them have read g. */
__device__ __forceinline__ bool sk_gather8(const sk_word_t *recv, int tp, int n, int e0, uint32_t gen, float (&v)[8],
                                           const int *abort_flag, unsigned limit) {
    recv += (size_t)(gen & 1u) * tp * n;
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = 0.0f;
    for (int src = 0; src < tp; src++) { /* rank order: every rank forms the same sum */
        const sk_word_t *p = recv + (size_t)src * n + e0;
        bool got = false;
        for (unsigned nsp = 0; nsp < limit && !got; nsp++) {
            sk_word_t w[8];
#pragma unroll
            for (int k = 0; k < 4; k++) sk_get2_sys(p + 2 * k, w[2 * k], w[2 * k + 1]);
            got = true;
#pragma unroll
            for (int k = 0; k < 8; k++) got = got && ((uint32_t)(w[k] >> 32) == gen);
            if (got) {
#pragma unroll
                for (int k = 0; k < 8; k++) v[k] = __fadd_rn(v[k], __uint_as_float((uint32_t)w[k]));
            } else if ((nsp & 255u) == 255u && ld_volatile_s32(abort_flag))
                break;
        }
        if (!got) return false;
    }
    return true;
}

/* The same exchange in two steps, for many ranks: polling tp slots one after the other costs tp dependent trips to
 * L2 in every thread of every block.  Step 1: one warp per 32 elements (128 warps on the whole GPU for n = 4096)
 * polls ALL ranks' words of its elements at once -- one word per rank and lane, so few registers -- adds them in rank
 * order and publishes the sum as a {generation, value} word in xsum (this GPU's memory).  Step 2: every thread reads
 * its 8 elements from xsum.  Two dependent trips whatever the number of ranks, and tp x fewer words polled. */
__device__ __forceinline__ bool sk_reduce_elem(const sk_word_t *recv, sk_word_t *xsum, int tp, int n, int e, uint32_t gen,
                                               const int *abort_flag, unsigned limit) {
    const sk_word_t *p = recv + (size_t)(gen & 1u) * tp * n + e;
    float s = 0.0f;
    for (int s0 = 0; s0 < tp; s0 += 4) { /* four ranks at a time: eight registers of words in flight */
        sk_word_t w[4];
        unsigned need = (tp - s0 >= 4) ? 15u : ((1u << (tp - s0)) - 1u);
        for (unsigned nsp = 0; nsp < limit && need; nsp++) {
#pragma unroll
            for (int k = 0; k < 4; k++)
                if ((need >> k) & 1u)
                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w[k]) : "l"(p + (size_t)(s0 + k) * n) : "memory");
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (((need >> k) & 1u) && (uint32_t)(w[k] >> 32) == gen) need &= ~(1u << k);
            if (need && (nsp & 255u) == 255u && ld_volatile_s32(abort_flag)) break;
        }
        if (need) return false;
#pragma unroll
        for (int k = 0; k < 4; k++)
            if (s0 + k < tp) s = __fadd_rn(s, __uint_as_float((uint32_t)w[k]));
    }
    sk_put(xsum + e, s, gen);
    return true;
}

__device__ __forceinline__ bool sk_gather8_local(const sk_word_t *xsum, int e0, uint32_t gen, float (&v)[8],
                                                 const int *abort_flag, unsigned limit) {
    for (unsigned nsp = 0; nsp < limit; nsp++) {
        sk_word_t w[8];
#pragma unroll
        for (int k = 0; k < 4; k++)
            asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(w[2 * k]), "=l"(w[2 * k + 1]) : "l"(xsum + e0 + 2 * k) : "memory");
        bool got = true;
#pragma unroll
        for (int k = 0; k < 8; k++) got = got && ((uint32_t)(w[k] >> 32) == gen);
        if (got) {
#pragma unroll
            for (int k = 0; k < 8; k++) v[k] = __uint_as_float((uint32_t)w[k]);
            return true;
        }
        if ((nsp & 255u) == 255u && ld_volatile_s32(abort_flag)) break;
    }
    return false;
}

__device__ __forceinline__ unsigned long long sk_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

/* phase stamps of block `trace_cta` (of every block when trace_cta < 0; trace_cap is then per block), in
 * nanoseconds of %globaltimer, 9 per layer, for profiling only */
#define SK_STAMP(idx)                                                                             \
    do {                                                                                          \
        if (TRACE && trace_p && trace_n < K.trace_cap)                                            \
            trace_p[trace_n++] = ((unsigned long long)(idx) << 56) | (sk_now() & 0x00ffffffffffffffULL); \
    } while (0)

/* TP: tensor-parallel exchange compiled in.  DM: which down-projection formats the instance carries -- the kernel is
 * instantiated per format family so that a run executes (and keeps in the instruction cache) only the dot products
 * it needs: the hot path is large, and code that is merely present between the hot instructions cost 1.7 us per layer
 * on the benchmark's Q4_K/Q6_K stack when all formats shared one instance.  TRACE: the phase stamps (another 0.4 us
 * per layer when compiled in and switched off). */
#define SK_DM_WHOLE 0    /* whole super-blocks, Q4_K and Q6_K */
#define SK_DM_WHOLE_Q5 1 /* ... and Q5_K */
#define SK_DM_HALF 2     /* half super-blocks (Q4_K, Q6_K): twice as many ranks as activation windows */

template <bool TP, int DM, bool TRACE>
__global__ void __launch_bounds__(SK_THREADS, 1) k_stack(fb_stack_args_t K) {
    extern __shared__ __align__(128) uint8_t dsm[];
    uint8_t *ring = dsm;
    sk_smem_t *S = reinterpret_cast<sk_smem_t *>(dsm + (TP ? SK_RING_BYTES_TP : SK_RING_BYTES));
    /* the normalised hidden state in fp32 (the near-tie arbiter re-sums router rows from it) lives in the first
     * 16 KB of the ring: it is written in P0 and last read in SEL, the ring is filled from P2 to the end of P3 */
    float *h_sm = reinterpret_cast<float *>(ring);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, G = gridDim.x;
    const bool leader = (cta == 0);
    sk_bar_t B = {K.bar, K.abort_flag, K.status, K.host_flags, (unsigned)G, K.bar_base, K.spin_limit, 0u};

    const uint32_t full_u = fb_smem_u32(&S->full[warp][0]);
    if (tid == 0) {
        for (int w = 0; w < SK_WARPS; w++)
            for (int s = 0; s < 3; s++) fb_mbar_init(fb_smem_u32(&S->full[w][s]), 1);
        fb_mbar_init_fence();
    }
    __syncthreads();
    uint32_t full_par = 0; /* bit s: parity of the completed phases of this warp's stage barrier s */

    const unsigned tok_first = (unsigned)K.tok_first;
    int trace_n = 0;
    /* where this thread records its stamps: thread 0 of the traced block (of every block when trace_cta < 0) */
    unsigned long long *trace_p = nullptr;
    if (TRACE && K.trace && tid == 0 && (K.trace_cta < 0 || cta == K.trace_cta))
        trace_p = K.trace + (K.trace_cta < 0 ? (size_t)cta * K.trace_cap : 0);
    bool alive = true;
    bool pending_join = false; /* a barrier has been arrived at but not yet waited for */

    /* the first layer's arguments; every later layer's are fetched by an idle warp during the layer before it */
    {
        const uint32_t *src = reinterpret_cast<const uint32_t *>(K.layers);
        uint32_t *dst = reinterpret_cast<uint32_t *>(&S->A2[0]);
        for (int i = tid; i < (int)(sizeof(fb_args_t) / 4); i += SK_THREADS) dst[i] = src[i];
        __syncthreads();
    }
    int cur = 0; /* which of the two argument buffers holds the current layer */
    for (int tk = 0; tk < K.tok_count && alive; tk++) {
        const unsigned tok = tok_first + (unsigned)tk;
        float x[8];
        for (int l = 0; l < K.n_layers && alive; l++, cur ^= 1) {
            const fb_args_t &A = S->A2[cur];
            const int n = A.n_embd, e0 = 8 * tid;
            const bool own = e0 < n;

            /* ---- router rows of this block: request them now, they depend on nothing */
            float4 wr[4][2];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int row = cta + j * G;
                if (own && row < A.n_experts) {
                    const float4 *p = reinterpret_cast<const float4 *>(A.router_w + (size_t)row * n + e0);
                    wr[j][0] = __ldg(p);
                    wr[j][1] = __ldg(p + 1);
                } else {
                    wr[j][0] = wr[j][1] = make_float4(0, 0, 0, 0);
                }
            }
            float4 r0 = make_float4(0, 0, 0, 0), r1 = r0, w0 = make_float4(1, 1, 1, 1), w1 = w0;
            if (own) { /* residual and norm weight of this layer: constants, requested before the join as well */
                const float4 *r = reinterpret_cast<const float4 *>(A.resid + e0);
                const float4 *wp = reinterpret_cast<const float4 *>(A.normw + e0);
                r0 = __ldg(r);
                r1 = __ldg(r + 1);
                w0 = __ldg(wp);
                w1 = __ldg(wp + 1);
            }
            if (A.has_shared && lane == 0) {
                /* the shared expert runs in every layer: its gate and up shards (the first bytes HBM has to deliver
                 * once the routing is known) are pulled into L2 now, while the chip waits on exchanges; 16 x 148
                 * slices, one per warp */
                const uint64_t tot = A.down_off; /* gate + up bytes of a record */
                const uint64_t csz = ((tot + (uint64_t)G * SK_WARPS - 1) / ((uint64_t)G * SK_WARPS) + 15ull) & ~15ull;
                const uint64_t off = ((uint64_t)cta * SK_WARPS + warp) * csz;
                if (off < tot)
                    fb_prefetch_l2(A.table_layer + (uint64_t)A.n_experts * A.rec_bytes + off, (uint32_t)min(csz, tot - off));
            }
            SK_STAMP(0);
            /* ---- the previous layer's block output: one GPU joins the barrier that publishes moe_out; tensor-parallel
             *      ranks gather the partial outputs of all ranks from their receive slots (that wait is the sync) */
            const uint32_t gen = K.gen_base + (uint32_t)(tk * K.n_layers + l) + 1u; /* this layer-token's generation */
            float mo[8];
            if (TP) {
                bool got = true;
                if (l > 0 && K.tp_two_stage) {
                    /* the ranks' words were added up by one warp per 32 elements while the previous layer's down
                     * phase was still streaming (see there): what is left is to fetch the sums */
                    if (own) got = sk_gather8_local(K.tp_xsum, e0, gen - 1u, mo, K.abort_flag, K.spin_limit);
                } else if (l > 0 && own)
                    got = sk_gather8(K.tp_recv, K.tp_size, n, e0, gen - 1u, mo, K.abort_flag, K.spin_limit);
                if (!__syncthreads_and(got ? 1 : 0)) {
                    if (tid == 0) sk_give_up(B);
                    alive = false;
                    break;
                }
            } else if (pending_join) {
                alive = sk_wait(B, S);
                pending_join = false;
                if (!alive) break;
            }

            SK_STAMP(1);
            /* ---- P0: residual stream, RMSNorm, Q8_K */
            float ss = 0.0f;
            if (own) {
                float4 v0, v1;
                if (l == 0) {
                    const float4 *p = reinterpret_cast<const float4 *>(K.tok_in + (size_t)tok * n + e0);
                    v0 = p[0];
                    v1 = p[1];
                } else {
                    if (!TP) {
                        const float4 *m = reinterpret_cast<const float4 *>(A.moe_out + e0);
                        const float4 m0 = __ldcg(m), m1 = __ldcg(m + 1);
                        mo[0] = m0.x; mo[1] = m0.y; mo[2] = m0.z; mo[3] = m0.w;
                        mo[4] = m1.x; mo[5] = m1.y; mo[6] = m1.z; mo[7] = m1.w;
                    }
                    v0 = make_float4(__fadd_rn(x[0], mo[0]), __fadd_rn(x[1], mo[1]), __fadd_rn(x[2], mo[2]), __fadd_rn(x[3], mo[3]));
                    v1 = make_float4(__fadd_rn(x[4], mo[4]), __fadd_rn(x[5], mo[5]), __fadd_rn(x[6], mo[6]), __fadd_rn(x[7], mo[7]));
                }
                x[0] = __fadd_rn(v0.x, r0.x); x[1] = __fadd_rn(v0.y, r0.y); x[2] = __fadd_rn(v0.z, r0.z); x[3] = __fadd_rn(v0.w, r0.w);
                x[4] = __fadd_rn(v1.x, r1.x); x[5] = __fadd_rn(v1.y, r1.y); x[6] = __fadd_rn(v1.z, r1.z); x[7] = __fadd_rn(v1.w, r1.w);
#pragma unroll
                for (int i = 0; i < 8; i++) ss = __fmaf_rn(x[i], x[i], ss);
            }
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(FULL, ss, o);
            if (lane == 0) S->red[5][warp] = ss;
            __syncthreads();
            float h[8];
            {
                /* every thread adds the sixteen partial sums itself, in the same order: no second barrier */
                float t = 0.0f;
#pragma unroll
                for (int w = 0; w < SK_WARPS; w++) t += S->red[5][w];
                const float sc = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)n), A.rms_eps)));
                const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int i = 0; i < 8; i++) h[i] = own ? __fmul_rn(__fmul_rn(x[i], sc), wv[i]) : 0.0f;
            }
            if (warp < n / FB_QK) fb_warp_quantize(h, &S->q8h[warp], lane);
            if (own) {
                float4 *hp = reinterpret_cast<float4 *>(h_sm + e0);
                hp[0] = make_float4(h[0], h[1], h[2], h[3]);
                hp[1] = make_float4(h[4], h[5], h[6], h[7]);
                /* these bytes are later overwritten by bulk copies (async proxy); block barriers follow before then */
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }

            SK_STAMP(2);
            /* ---- P1: router logits of this block's rows */
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float p = 0.0f;
                p = fmaf(wr[j][0].x, h[0], p); p = fmaf(wr[j][0].y, h[1], p); p = fmaf(wr[j][0].z, h[2], p); p = fmaf(wr[j][0].w, h[3], p);
                p = fmaf(wr[j][1].x, h[4], p); p = fmaf(wr[j][1].y, h[5], p); p = fmaf(wr[j][1].z, h[6], p); p = fmaf(wr[j][1].w, h[7], p);
                for (int o = 16; o > 0; o >>= 1) p += __shfl_xor_sync(FULL, p, o);
                if (lane == 0) S->red[j][warp] = p;
            }
            if (A.shared_gate_w) { /* scalar gate of the shared expert: sigmoid(h . w) (src/inference.c:586-592) */
                float p = 0.0f;
                if (own) {
                    const float4 *q = reinterpret_cast<const float4 *>(A.shared_gate_w + e0);
                    const float4 a0 = __ldg(q), a1 = __ldg(q + 1);
                    p = fmaf(a0.x, h[0], p); p = fmaf(a0.y, h[1], p); p = fmaf(a0.z, h[2], p); p = fmaf(a0.w, h[3], p);
                    p = fmaf(a1.x, h[4], p); p = fmaf(a1.y, h[5], p); p = fmaf(a1.z, h[6], p); p = fmaf(a1.w, h[7], p);
                }
                for (int o = 16; o > 0; o >>= 1) p += __shfl_xor_sync(FULL, p, o);
                if (lane == 0) S->red[4][warp] = p;
            }
            __syncthreads();
            if (tid < 4) {
                const int row = cta + tid * G;
                if (row < A.n_experts) {
                    float t = 0.0f;
                    for (int w = 0; w < SK_WARPS; w++) t += S->red[tid][w];
                    A.logits[row] = t; /* for inspection from the host */
                    sk_put(K.ll_logits + row, t, gen);
                }
            } else if (tid == 32) {
                float t = 0.0f;
                if (A.shared_gate_w)
                    for (int w = 0; w < SK_WARPS; w++) t += S->red[4][w];
                S->shared_gate = A.shared_gate_w ? __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-t))) : 1.0f;
            }
            for (int row = cta + 4 * G; row < A.n_experts; row += G) { /* more than 4 rows per block: rare shapes */
                float p = 0.0f;
                if (own) {
                    const float4 *q = reinterpret_cast<const float4 *>(A.router_w + (size_t)row * n + e0);
                    const float4 a0 = __ldg(q), a1 = __ldg(q + 1);
                    p = fmaf(a0.x, h[0], p); p = fmaf(a0.y, h[1], p); p = fmaf(a0.z, h[2], p); p = fmaf(a0.w, h[3], p);
                    p = fmaf(a1.x, h[4], p); p = fmaf(a1.y, h[5], p); p = fmaf(a1.z, h[6], p); p = fmaf(a1.w, h[7], p);
                }
                for (int o = 16; o > 0; o >>= 1) p += __shfl_xor_sync(FULL, p, o);
                __syncthreads();
                if (lane == 0) S->red[0][warp] = p;
                __syncthreads();
                if (tid == 0) {
                    float t = 0.0f;
                    for (int w = 0; w < SK_WARPS; w++) t += S->red[0][w];
                    A.logits[row] = t;
                    sk_put(K.ll_logits + row, t, gen);
                }
            }
            SK_STAMP(3);
            /* The logits travel as {generation, value} words; every thread polls the one word it ranks, and a word
             * of this layer-token cannot be mistaken for an older one.  (A block can only write the next
             * layer-token's word after barrier 2 of this one, which every block reaches after it has read its
             * logits.)  On one GPU that is the whole exchange: no grid barrier, 1.5 us per layer less than arrival,
             * release and a load behind it.  Tensor-parallel ranks keep a barrier (an arrival without a fence: the
             * words validate themselves): their blocks come out of the join as the peers' words arrive, up to
             * microseconds apart, and that many threads polling for that long slowed the whole layer by 1 - 4.5 us. */
            if (TP) {
                sk_arrive(B, S, false);
                alive = sk_wait(B, S);
                if (!alive) break;
            }

            /* ---- SEL: routing, redundantly in every block (results identical by construction) */
            if (leader && own) {
                /* the hidden state is kept in global memory as well, for inspection from the host.  Written here and
                 * not where it is formed: 16 KB of stores ahead of barrier 1 made block 0's arrival (a release) the
                 * last of every layer, by 0.45 us; ahead of barrier 2 they have the whole gate/up phase to drain */
                const float4 *hp = reinterpret_cast<const float4 *>(h_sm + e0);
                float4 *gp = reinterpret_cast<float4 *>(A.h + e0);
                gp[0] = hp[0];
                gp[1] = hp[1];
            }
            /* As soon as the ids are known, each warp starts the copies of its first gate/up task into its ring
             * stages: the softmax, renormalisation and hand-over that follow (about 1 us, more with cache-aware
             * routing) then overlap with HBM's start-up instead of preceding it.  The hidden state that shares the
             * ring's first bytes is dead by then.  When the final list differs in that slot (order changed by an
             * exact tie of probabilities, a cache-aware substitute) the stale copy is awaited and the right one
             * requested, which costs what starting late costs. */
            const int gu_total = A.n_slots * A.gate_groups;
            const int t0 = (int)(((long long)cta * gu_total) / G), t1 = (int)(((long long)(cta + 1) * gu_total) / G);
            const uint32_t ring_u = fb_smem_u32(ring) + warp * 2 * FB_Q4K_GROUP;
            auto issue = [&](const uint8_t *recp, int g, int which) {
                const uint8_t *src = recp + (which ? A.up_off : 0) + (uint64_t)g * FB_Q4K_GROUP;
                fb_mbar_expect_tx(full_u + 8 * which, FB_Q4K_GROUP);
                fb_bulk_g2s(ring_u + which * FB_Q4K_GROUP, src, FB_Q4K_GROUP, full_u + 8 * which);
            };
            int early_e = -1; /* the expert whose groups were requested early (the same in every lane) */
            auto early = [&](const int *cand) {
                SK_STAMP(5); /* the gate/up phase is timed from its first request */
                const int t = t0 + warp;
                if (t >= t1) return;
                const int slot = t / A.gate_groups, g = t - slot * A.gate_groups;
                const int e = slot < A.top_k ? cand[slot] : A.n_experts;
                if (e < 0 || e > A.n_experts) return;
                /* under cache-aware routing an expert that is not resident may still be replaced: it is left for
                 * the start of the phase proper (a resident one, and the shared expert, stay where they are) */
                if (slot < A.top_k && A.resident && A.car_threshold > 0.0f && A.car_threshold < 1.0f &&
                    !((__ldg(A.resident + (e >> 5)) >> (e & 31)) & 1u))
                    return;
#if SK_EARLY_COPY
                early_e = e;
                if (lane == 0) {
                    const uint8_t *recp = A.table_layer + (uint64_t)e * A.rec_bytes;
                    issue(recp, g, 0);
                    issue(recp, g, 1);
                }
#else
                if (lane == 0 && slot < A.top_k) {
                    const uint8_t *src = A.table_layer + (uint64_t)e * A.rec_bytes + (uint64_t)g * FB_Q4K_GROUP;
                    fb_prefetch_l2(src, FB_Q4K_GROUP);
                    fb_prefetch_l2(src + A.up_off, FB_Q4K_GROUP);
                }
#endif
#if SK_EARLY_ROUNDS
                const int tb = t + SK_WARPS;
                if (lane == 0 && tb < t1) {
                    const int sb = tb / A.gate_groups, gb = tb - sb * A.gate_groups;
                    const int eb = sb < A.top_k ? cand[sb] : -1;
                    if (eb >= 0 && eb < A.n_experts) {
                        const uint8_t *src = A.table_layer + (uint64_t)eb * A.rec_bytes + (uint64_t)gb * FB_Q4K_GROUP;
                        fb_prefetch_l2(src, FB_Q4K_GROUP);
                        fb_prefetch_l2(src + A.up_off, FB_Q4K_GROUP);
                    }
                }
#endif
            };
            /* the wait for the logits: a word is read again until it carries this layer-token's generation (bounded) */
            bool logits_ok = true;
            auto logit = [&](int e) -> float {
                sk_word_t w = sk_get1(K.ll_logits + e);
                for (unsigned nsp = 0; (uint32_t)(w >> 32) != gen; nsp++) {
                    if (nsp >= K.spin_limit || ((nsp & 255u) == 255u && ld_volatile_s32(K.abort_flag))) {
                        logits_ok = false;
                        break;
                    }
                    w = sk_get1(K.ll_logits + e);
                }
                SK_STAMP(4); /* thread 0's word has arrived */
                return __uint_as_float((uint32_t)w);
            };
            fb_block_select(A, &S->sel, h_sm, S->all_scores, S->ids, S->ids_orig, S->scores, S->slot_rec, leader,
                            S->shared_gate,
                            (leader && A.route_log) ? A.route_log + (size_t)tok * A.route_stride : nullptr, logit, early);
            if (!__all_sync(FULL, logits_ok)) { /* the block barrier that ends gate/up gives up */
                if (lane == 0) sk_give_up(B);
                alive = false;
            }
            if (leader) {
                if (tid < A.n_slots) {
                    A.ids[tid] = S->ids[tid];
                    A.scores[tid] = S->scores[tid];
                    if (tid < A.top_k) A.ids_orig[tid] = S->ids_orig[tid];
                }
                for (int e = tid; e < A.n_experts; e += SK_THREADS) A.all_scores[e] = S->all_scores[e];
            }

            /* ---- P2: gate/up + SwiGLU.  Tasks = (expert slot, 32-block group) in slot-major order; every block owns
             *      a contiguous, equally long run of them (so all SMs stream the same number of bytes) and deals
             *      its run round-robin to its 16 warps. */
            {
                const int bpr = A.gate_bpr, rpg = 32 / bpr;
                if (t0 + warp < t1) {
                    const int slot = (t0 + warp) / A.gate_groups, g = (t0 + warp) - slot * A.gate_groups;
                    if (early_e != S->ids[slot]) {
                        if (early_e >= 0) { /* a stale copy is on its way into the stages: take it off the barriers */
                            if (!fb_mbar_wait(full_u, full_par & 1) || !fb_mbar_wait(full_u + 8, (full_par >> 1) & 1))
                                alive = false;
                            full_par ^= 3u;
                            __syncwarp();
                        }
                        if (alive && lane == 0) {
                            issue(S->slot_rec[slot], g, 0);
                            issue(S->slot_rec[slot], g, 1);
                        }
                    }
                }
                const uint32_t a_u = fb_smem_u32(&S->q8h[lane % bpr]);
                for (int t = t0 + warp; t < t1 && alive; t += SK_WARPS) {
                    float f[2];
                    if (!fb_mbar_wait(full_u, full_par & 1) || !fb_mbar_wait(full_u + 8, (full_par >> 1) & 1)) {
                        alive = false;
                        break;
                    }
                    full_par ^= 3u;
                    /* both groups are read where they lie, sharing every activation load between gate and up */
                    fb_dot2_q4k_sm(ring_u + 16 * lane, ring_u + FB_Q4K_GROUP + 16 * lane, a_u, f[0], f[1]);
                    __syncwarp();
                    if (lane == 0 && t + SK_WARPS < t1) {
                        const int tn = t + SK_WARPS, sn = tn / A.gate_groups;
                        issue(S->slot_rec[sn], tn - sn * A.gate_groups, 0);
                        issue(S->slot_rec[sn], tn - sn * A.gate_groups, 1);
                    }
                    const float fg = fb_span_sum(f[0], bpr), fu = fb_span_sum(f[1], bpr);
                    const int slot = t / A.gate_groups, g = t - slot * A.gate_groups;
                    const int row = g * rpg + lane / bpr;
                    if (lane % bpr == 0 && row < A.inter_local) {
                        const float sl = __fdiv_rn(fg, __fadd_rn(1.0f, expf(-fg)));
                        A.act[slot * A.inter_local + row] = __fmul_rn(sl, fu);
                    }
                }
                if (!__syncthreads_and(alive ? 1 : 0)) {
                    if (tid == 0) sk_give_up(B);
                    alive = false;
                    break;
                }
            }

            SK_STAMP(6);
            /* ---- barrier (activations); this block's first down groups are requested while it completes.
             *      P3 tasks = (row group, expert slot) in row-group-major order, again one contiguous, equally
             *      long run per block dealt round-robin to 12 warps (two ring stages of one group each). */
            sk_arrive(B, S);
            const int ns = A.n_slots, dbpr = A.down_bpr, drpg = 32 / dbpr;
            const uint32_t GB = (DM == SK_DM_HALF) ? (A.down_type == FB_TYPE_Q4_K ? FB_Q4K_HGROUP : A.down_type == FB_TYPE_Q5_K ? FB_Q5K_HGROUP : FB_Q6K_HGROUP)
                                : (A.down_type == FB_TYPE_Q4_K) ? FB_Q4K_GROUP
                                : (DM == SK_DM_WHOLE_Q5 && A.down_type == FB_TYPE_Q5_K) ? FB_Q5K_GROUP : FB_Q6K_GROUP;
            const int dtotal = A.down_groups * ns;
            const int d0 = (int)(((long long)cta * dtotal) / G), d1 = (int)(((long long)(cta + 1) * dtotal) / G);
            /* the run [d0, d1): its last row group continues in the next block when d1 is not a multiple of ns;
             * those n_tail tasks run first.  Row groups owned here: those whose last slot lies in the run. */
            const int n_tail = (d1 > d0 && d1 % ns != 0) ? min(d1 - d0, d1 % ns) : 0;
            const int rg_first = d0 / ns;
            const int n_own_rg = (d1 > d0) ? (d1 / ns - rg_first) : 0;
            const uint32_t hand_gen = gen; /* tags this layer-token's hand-over words */
            auto dtask = [&](int j) { return j < n_tail ? d1 - n_tail + j : d0 + (j - n_tail); };
            /* on one GPU, groups of up to 4608 bytes (Q4_K) get three stages per warp, so that all three rounds of
             * the 397B shape are requested up front; larger ones two.  A tensor-parallel rank has at most two rounds
             * and keeps two stages (the third cost its instances registers, and with them 0.6 us per layer). */
            const int nst = (!TP && GB <= FB_Q4K_GROUP) ? 3 : 2;
            const uint32_t dstride = (!TP && GB <= FB_Q4K_GROUP) ? FB_Q4K_GROUP : FB_Q6K_GROUP;
            const uint32_t dring_u = fb_smem_u32(ring) + warp * nst * dstride;
            auto dissue = [&](int t, int s) {
                const int rg = t / ns, slot = t - rg * ns;
                fb_mbar_expect_tx(full_u + 8 * s, GB);
                fb_bulk_g2s(dring_u + s * dstride, S->slot_rec[slot] + A.down_off + (uint64_t)rg * GB, GB, full_u + 8 * s);
            };
            /* one group per warp now; the second follows the barrier and the (small, latency-critical) activation
             * loads, which would otherwise queue behind 175 KB of weights on their way into this SM */
            if (warp < SK_DOWN_WARPS && lane == 0 && warp < d1 - d0) dissue(dtask(warp), 0);
            alive = sk_wait(B, S);
            if (!alive) break;
            SK_STAMP(7);

            /* ---- P3: down + combine */
            {   /* quantise the activations of every slot (src/cpu_expert.c:109-110): all loads first, then the math */
                float v[3][8];
#pragma unroll
                for (int u = 0; u < 3; u++) {
                    const int wd = warp + u * SK_WARPS;
                    if (wd < ns * dbpr) {
                        const float4 *src = reinterpret_cast<const float4 *>(A.act + (wd / dbpr) * A.inter_local + (wd % dbpr) * FB_QK + 8 * lane);
                        const float4 p0 = __ldcg(src), p1 = __ldcg(src + 1);
                        v[u][0] = p0.x; v[u][1] = p0.y; v[u][2] = p0.z; v[u][3] = p0.w;
                        v[u][4] = p1.x; v[u][5] = p1.y; v[u][6] = p1.z; v[u][7] = p1.w;
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; i++) v[u][i] = 0.0f;
                    }
                }
                if (warp < SK_DOWN_WARPS && lane == 0) {
                    if (warp + SK_DOWN_WARPS < d1 - d0) dissue(dtask(warp + SK_DOWN_WARPS), 1);
                    if (nst == 3 && warp + 2 * SK_DOWN_WARPS < d1 - d0) dissue(dtask(warp + 2 * SK_DOWN_WARPS), 2);
                }
                /* the three windows' shuffle chains are independent: run them unconditionally so they interleave */
#pragma unroll
                for (int u = 0; u < 3; u++) {
                    const int wd = warp + u * SK_WARPS;
                    fb_warp_quantize(v[u], &S->q8a[min(wd, SK_MAX_Q8A - 1)], lane, wd < ns * dbpr);
                }
            }
            __syncthreads();
            /* Two-stage receive, first stage: under tensor parallelism the last warp of a block (it has no down
             * tasks) adds up, in rank order, the words all ranks store for the block's 32 output elements of THIS
             * layer as they arrive, and publishes the sums for the next layer's join.  It must not take part in the
             * block barrier before the combine: the words it waits for include the ones this very block's combine
             * sends.  The other fifteen warps meet at a barrier of their own; all sixteen meet again afterwards. */
            const bool early_reduce = TP && K.tp_two_stage && l + 1 < K.n_layers;
            const bool reducer = early_reduce && warp == SK_WARPS - 1;
            if (reducer) {
                bool got = true;
                for (int c = cta; c < n / 32 && got; c += G)
                    got = sk_reduce_elem(K.tp_recv, K.tp_xsum, K.tp_size, n, 32 * c + lane, gen, K.abort_flag, K.spin_limit);
                if (!__all_sync(FULL, got)) {
                    if (lane == 0) sk_give_up(B);
                    alive = false;
                }
            } else if (warp == SK_DOWN_WARPS) {
                /* a warp without down tasks fetches the next layer's arguments (the next token's first layer after
                 * the last one) into the other buffer; the block barriers below publish them */
                const int ln = (l + 1 < K.n_layers) ? l + 1 : 0;
                const uint32_t *src = reinterpret_cast<const uint32_t *>(K.layers + ln);
                uint32_t *dst = reinterpret_cast<uint32_t *>(&S->A2[cur ^ 1]);
                for (int i = lane; i < (int)(sizeof(fb_args_t) / 4); i += 32) dst[i] = src[i];
                /* its residency mask (64 bytes, long evicted by the expert stream) is asked back into L2: the
                 * selection reads it right after barrier 1 and would otherwise wait for HBM there */
                if (lane == 0) {
                    const uint32_t *rp = K.layers[ln].resident;
                    if (rp) {
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(rp));
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(rp + (FB_MAX_EXPERTS / 32 - 1)));
                    }
                }
            } else if (warp < SK_DOWN_WARPS) {
                int it = 0;
                for (int j = warp; j < d1 - d0; j += SK_DOWN_WARPS, it++) {
                    const int s = (nst == 2) ? (it & 1) : (it % 3);
                    if (!fb_mbar_wait(full_u + 8 * s, (full_par >> s) & 1u)) {
                        alive = false;
                        break;
                    }
                    full_par ^= 1u << s;
                    const int t = dtask(j);
                    const int rg = t / ns, slot = t - rg * ns;
                    const uint32_t st = dring_u + s * dstride + 16 * lane;
                    const uint32_t a_u = fb_smem_u32(&S->q8a[slot * dbpr + lane % dbpr]);
                    float f;
                    if (DM == SK_DM_HALF && A.down_type == FB_TYPE_Q4_K) { /* half super-blocks (layout.h) */
                        const uint4 hd = fb_lds128(st);
                        uint4 q[4];
#pragma unroll
                        for (int k = 0; k < 4; k++) q[k] = fb_lds128(st + 512 * (k + 1));
                        __syncwarp();
                        if (lane == 0 && j + nst * SK_DOWN_WARPS < d1 - d0) dissue(dtask(j + nst * SK_DOWN_WARPS), s);
                        f = fb_dot_q4k_half_sm(hd, q, a_u, A.down_half);
                    } else if (DM == SK_DM_HALF && A.down_type == FB_TYPE_Q5_K) {
                        const uint4 hd = fb_lds128(st), h0 = fb_lds128(st + 512), h1 = fb_lds128(st + 1024);
                        uint4 q[4];
#pragma unroll
                        for (int k = 0; k < 4; k++) q[k] = fb_lds128(st + 512 * (k + 3));
                        __syncwarp();
                        if (lane == 0 && j + nst * SK_DOWN_WARPS < d1 - d0) dissue(dtask(j + nst * SK_DOWN_WARPS), s);
                        f = fb_dot_q5k_half_sm(hd, h0, h1, q, a_u, A.down_half);
                    } else if (DM == SK_DM_HALF) {
                        uint4 ql[4], qh[2];
#pragma unroll
                        for (int k = 0; k < 4; k++) ql[k] = fb_lds128(st + 512 * k);
#pragma unroll
                        for (int k = 0; k < 2; k++) qh[k] = fb_lds128(st + 512 * (4 + k));
                        const uint2 sc = fb_lds64_a(dring_u + s * dstride + FB_Q6K_HOFF_SC + 8 * lane);
                        uint32_t d16;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(d16) : "r"(dring_u + s * dstride + FB_Q6K_HOFF_D + 2 * lane));
                        __syncwarp();
                        if (lane == 0 && j + nst * SK_DOWN_WARPS < d1 - d0) dissue(dtask(j + nst * SK_DOWN_WARPS), s);
                        f = fb_dot_q6k_half_sm(ql, qh, sc, d16, a_u, A.down_half);
                    } else if (A.down_type == FB_TYPE_Q4_K) {
                        const uint4 hd = fb_lds128(st);
                        uint4 q[8];
#pragma unroll
                        for (int k = 0; k < 8; k++) q[k] = fb_lds128(st + 512 * (k + 1));
                        __syncwarp();
                        if (lane == 0 && j + nst * SK_DOWN_WARPS < d1 - d0) dissue(dtask(j + nst * SK_DOWN_WARPS), s);
                        f = fb_dot_q4k_sm(hd, q, a_u);
                    } else if (DM == SK_DM_WHOLE_Q5 && A.down_type == FB_TYPE_Q5_K) {
                        const uint4 hd = fb_lds128(st), h0 = fb_lds128(st + 512), h1 = fb_lds128(st + 1024);
                        uint4 q[8];
#pragma unroll
                        for (int k = 0; k < 8; k++) q[k] = fb_lds128(st + 512 * (k + 3));
                        __syncwarp();
                        if (lane == 0 && j + nst * SK_DOWN_WARPS < d1 - d0) dissue(dtask(j + nst * SK_DOWN_WARPS), s);
                        f = fb_dot_q5k_sm(hd, h0, h1, q, a_u);
                    } else {
                        uint4 ql[8], qh[4];
#pragma unroll
                        for (int k = 0; k < 8; k++) ql[k] = fb_lds128(st + 512 * k);
#pragma unroll
                        for (int k = 0; k < 4; k++) qh[k] = fb_lds128(st + 512 * (8 + k));
                        const uint4 sc = fb_lds128(st + 512 * 12);
                        uint32_t d16;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(d16) : "r"(dring_u + s * dstride + FB_Q6K_OFF_D + 2 * lane));
                        __syncwarp();
                        if (lane == 0 && j + nst * SK_DOWN_WARPS < d1 - d0) dissue(dtask(j + nst * SK_DOWN_WARPS), s);
                        f = fb_dot_q6k_sm(ql, qh, sc, d16, a_u);
                    }
                    f = fb_span_sum(f, dbpr);
                    if (j < n_tail) {
                        /* a row group that continues in the next block: hand this slot's rows over through global
                         * memory right away (the owner combines at the end of its own run) */
                        const int r = rg * drpg + lane / dbpr;
                        if (lane % dbpr == 0 && r < n) sk_put(K.ll_dots + slot * n + r, f, hand_gen);
                    } else if (lane % dbpr == 0) {
                        S->dots[rg - rg_first][slot][lane / dbpr] = f;
                    }
                }
            }
            bool go;
            if (early_reduce) {
                go = alive;
                if (!reducer) {
                    uint32_t all;
                    asm volatile(
                        "{\n"
                        ".reg .pred p, q;\n"
                        "setp.ne.b32 p, %1, 0;\n"
                        "barrier.cta.red.and.pred q, 2, %2, p;\n"
                        "selp.u32 %0, 1, 0, q;\n"
                        "}\n"
                        : "=r"(all)
                        : "r"((uint32_t)alive), "n"(SK_THREADS - 32)
                        : "memory");
                    go = all != 0;
                }
            } else {
                go = __syncthreads_and(alive ? 1 : 0) != 0;
            }
            /* combine: partial += score * down in list order (src/cpu_expert.c:114-115), shared expert added after
             * (src/inference.c:595).  The block that ran a row group's LAST slot owns it; slots that ran in earlier
             * blocks arrive through global memory (those blocks ran them first, so the wait is normally over). */
            for (int q = warp; q < n_own_rg && go && !reducer; q += early_reduce ? SK_WARPS - 1 : SK_WARPS) {
                const int rg = rg_first + q;
                const int s_lo = max(d0, rg * ns) - rg * ns; /* slots below s_lo ran elsewhere */
                const int r = rg * drpg + lane;
                const bool row_ok = lane < drpg && r < n;
                if (s_lo > 0) {
                    /* slots below s_lo were run by the previous block(s): the warp fetches their s_lo x drpg words
                     * with all lanes, four requests per lane in flight, and parks the values beside its own */
                    const int nw = s_lo * drpg, dsh = __ffs(drpg) - 1;
                    bool ok = true;
                    for (int base = 0; base < nw && ok; base += 128) {
                        unsigned need = 0;
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int idx = base + 32 * u + lane;
                            if (idx < nw && rg * drpg + (idx & (drpg - 1)) < n) need |= 1u << u;
                        }
                        for (unsigned nsp = 0; nsp < K.spin_limit && need; nsp++) {
                            sk_word_t w[4];
#pragma unroll
                            for (int u = 0; u < 4; u++) {
                                const int idx = base + 32 * u + lane;
                                if ((need >> u) & 1u) w[u] = sk_get1(K.ll_dots + (idx >> dsh) * n + rg * drpg + (idx & (drpg - 1)));
                            }
#pragma unroll
                            for (int u = 0; u < 4; u++) {
                                const int idx = base + 32 * u + lane;
                                if (((need >> u) & 1u) && (uint32_t)(w[u] >> 32) == hand_gen) {
                                    S->dots[q][idx >> dsh][idx & (drpg - 1)] = __uint_as_float((uint32_t)w[u]);
                                    need &= ~(1u << u);
                                }
                            }
                            if (need && (nsp & 255u) == 255u && ld_volatile_s32(K.abort_flag)) break;
                        }
                        ok = need == 0u;
                    }
                    if (!__all_sync(FULL, ok)) {
                        if (lane == 0) sk_give_up(B);
                        break; /* the grid barrier that follows sees the abort flag */
                    }
                    __syncwarp();
                }
                if (row_ok) {
                    float acc = 0.0f;
                    for (int s = 0; s < A.top_k; s++) acc = __fmaf_rn(S->scores[s], S->dots[q][s][lane], acc);
                    if (A.has_shared) {
                        const float sh = S->dots[q][A.top_k][lane];
                        acc = __fadd_rn(acc, A.shared_gate_w ? __fmul_rn(sh, S->scores[A.top_k]) : sh);
                    }
                    if (TP) {
                        /* fused all-reduce, sending side: the partial goes straight into slot tp_rank of every
                         * rank's receive buffer over NVLink (plain peer stores of {generation, value} words) */
                        const size_t at = ((size_t)(gen & 1u) * K.tp_size + K.tp_rank) * n + r;
                        for (int p = 0; p < K.tp_size; p++) sk_put_sys(K.tp_peer[p] + at, acc, gen);
                    } else {
                        A.moe_out[r] = acc;
                    }
                }
            }
            /* everybody agrees on whether the layer succeeded (the reducing warp included) */
            if (early_reduce) go = __syncthreads_and((alive && go) ? 1 : 0) != 0;
            if (!go) {
                if (tid == 0) sk_give_up(B);
                alive = false;
                break;
            }
            SK_STAMP(8);
            if (!TP) {
                sk_arrive(B, S);
                pending_join = true;
            }
        } /* layers */
        if (!alive) break;
        /* ---- end of token: the last layer's block output, x += moe_out, publish */
        float mo[8];
        {
            const fb_args_t &A = S->A2[cur ^ 1]; /* the last layer's (cur has moved on) */
            const int e0 = 8 * tid;
            if (TP) {
                bool got = true;
                if (leader && e0 < A.n_embd)
                    got = sk_gather8(K.tp_recv, K.tp_size, A.n_embd, e0, K.gen_base + (uint32_t)((tk + 1) * K.n_layers), mo, K.abort_flag, K.spin_limit);
                if (!__syncthreads_and(got ? 1 : 0)) {
                    if (tid == 0) sk_give_up(B);
                    alive = false;
                    break;
                }
            } else {
                alive = sk_wait(B, S);
                pending_join = false;
                if (!alive) break;
                if (leader && e0 < A.n_embd) {
                    const float4 *m = reinterpret_cast<const float4 *>(A.moe_out + e0);
                    const float4 m0 = __ldcg(m), m1 = __ldcg(m + 1);
                    mo[0] = m0.x; mo[1] = m0.y; mo[2] = m0.z; mo[3] = m0.w;
                    mo[4] = m1.x; mo[5] = m1.y; mo[6] = m1.z; mo[7] = m1.w;
                }
            }
            if (leader && e0 < A.n_embd) {
                /* a host-to-host call lets the last token's result go straight to the caller's pinned buffer */
                float4 *o = (K.out_host && tk == K.tok_count - 1)
                                ? reinterpret_cast<float4 *>(K.out_host + e0)
                                : reinterpret_cast<float4 *>(K.tok_out + (size_t)tok * A.n_embd + e0);
                o[0] = make_float4(__fadd_rn(x[0], mo[0]), __fadd_rn(x[1], mo[1]), __fadd_rn(x[2], mo[2]), __fadd_rn(x[3], mo[3]));
                o[1] = make_float4(__fadd_rn(x[4], mo[4]), __fadd_rn(x[5], mo[5]), __fadd_rn(x[6], mo[6]), __fadd_rn(x[7], mo[7]));
                float4 *xo = reinterpret_cast<float4 *>(A.x + e0);
                xo[0] = o[0];
                xo[1] = o[1];
            }
        }
        __syncthreads(); /* the token is complete in this block before the next one starts */
    }
    if (!alive) {
        /* A block that gave up may still have bulk copies on their way into its ring (groups are requested ahead of
         * the barriers and waits that can run out).  They land within microseconds; the block stays for a bounded
         * grace period, far longer than that, before its shared memory is released. */
        const unsigned long long t_end = sk_now() + 100000ull; /* 100 us of %globaltimer */
        for (int i = 0; i < 4096 && sk_now() < t_end; i++) __nanosleep(256);
    }
    if (leader && tid == 0 && alive) *K.tok_ctr = tok_first + (unsigned)K.tok_count;
}

extern "C" int fb_stack_smem_bytes(void) { return (int)(SK_RING_BYTES + sizeof(sk_smem_t)); }

extern "C" int fb_stack_supported(const fb_args_t *a, int grid) {
    const int dtotal = a->down_groups * a->n_slots;
    const int run = (dtotal + grid - 1) / grid;                       /* longest run of down tasks of one block */
    const int max_rg = (run + a->n_slots - 2) / a->n_slots + 2;       /* row groups such a run can touch */
    if (a->down_half >= 0 && a->down_type != FB_TYPE_Q4_K && a->down_type != FB_TYPE_Q5_K && a->down_type != FB_TYPE_Q6_K) return 0;
    if (a->gate_type != FB_TYPE_Q4_K) return 0;
    return a->n_embd <= 4096 && a->n_slots <= SK_DN_SLOTS && a->n_slots * a->down_bpr <= SK_MAX_Q8A &&
           a->n_embd / FB_QK <= 16 && a->tp_size <= FB_MAX_TP && a->inter_local % FB_QK == 0 && max_rg <= SK_MAX_RG;
}

template <bool TP, int DM, bool TRACE>
static int sk_launch2(fb_stack_args_t &kk, int grid, int sm, int dev, void *stream) {
    static unsigned char configured[64]; /* the attribute holds for one device: one flag per device ordinal and instance */
    if (!configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(k_stack<TP, DM, TRACE>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = 1;
    }
    void *params[] = {&kk};
    return (int)cudaLaunchCooperativeKernel((const void *)k_stack<TP, DM, TRACE>, dim3(grid), dim3(SK_THREADS), params,
                                            (size_t)sm, (cudaStream_t)stream);
}

template <bool TP, int DM>
static int sk_launch(fb_stack_args_t &kk, int grid, int sm, int dev, void *stream) {
    return (kk.trace && kk.trace_cap > 0) ? sk_launch2<TP, DM, true>(kk, grid, sm, dev, stream)
                                          : sk_launch2<TP, DM, false>(kk, grid, sm, dev, stream);
}

extern "C" int fb_launch_stack(const fb_stack_args_t *k, int grid, void *stream) {
    const int sm = fb_stack_smem_bytes();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    fb_stack_args_t kk = *k;
    const bool tp = kk.tp_size > 1;
    switch (kk.down_mode) {
        case SK_DM_WHOLE: return tp ? sk_launch<true, SK_DM_WHOLE>(kk, grid, sm, dev, stream) : sk_launch<false, SK_DM_WHOLE>(kk, grid, sm, dev, stream);
        case SK_DM_WHOLE_Q5: return tp ? sk_launch<true, SK_DM_WHOLE_Q5>(kk, grid, sm, dev, stream) : sk_launch<false, SK_DM_WHOLE_Q5>(kk, grid, sm, dev, stream);
        case SK_DM_HALF: return tp ? sk_launch<true, SK_DM_HALF>(kk, grid, sm, dev, stream) : (int)cudaErrorInvalidValue;
    }
    return (int)cudaErrorInvalidValue;
}
