/*
 * batch.cu -- the routed-expert FFN for MANY tokens per call (prefill / batched decode) on the 5th-generation tensor
 * cores of sm_100a: tcgen05.mma with accumulators in tensor memory.
 *
 * Per layer:   prologue (residual, RMSNorm, Q8_K of every token)  ->  route (softmax, ordered top-k)  ->  bucket the
 * (token, slot) pairs by expert  ->  grouped GEMM gate+up with SwiGLU epilogue  ->  Q8_K of the activations  ->
 * grouped GEMM down  ->  combine in slot order.
 *
 * The definition computed is src/cpu_expert.c applied token by token: activations quantised to Q8_K per 256
 * (src/quant.c:343-375), products against the Q4_K weights (src/quant.c:405-476), silu(g)*u with expf
 * (src/cpu_expert.c:103-106), partial += score * down in list order (114-115), shared expert added last.  What changes
 * is how the products are formed.  Both operands are turned into fp16 and multiplied on the tensor cores with fp32
 * accumulation in tensor memory:
 *     A[row][k] = fp16( d*sc_j*q - dmin*m_j )              the dequantised weight (src/quant.c:82-105), one rounding
 *     B[k][pair] = fp16( q8_k * (yd_block / ymax_row) )     the Q8_K-quantised activation, relative to the row's
 *                                                           largest block scale; ymax_row multiplies the result
 * so the int8 rounding of the activations -- what separates this definition from the fp32-activation one by 2e-2 --
 * is reproduced exactly, and what differs from the CPU is two fp16 roundings per product (2^-12 each, random sign):
 * about 2e-4 relative on a layer output, inside the 1e-3 bound, stated in the tests.
 *
 * Grouped GEMM kernel (kb_gemm), one persistent CTA per SM, warp-specialised:
 *   warps 5..12 (256 threads)  producers: each thread owns one Q4_K block row of the tile, loads its 144 raw bytes
 *                              with coalesced 128-bit loads from the batched layout (batch_launch.h), dequantises 64
 *                              weights per 32 bytes with two-at-a-time fp16 arithmetic (nibble | 0x6400 = 1024 + q,
 *                              minus 1024, times d*sc minus dmin*m) and stores them into the 128-byte-swizzled,
 *                              K-major operand tile in shared memory; the same threads copy the activation rows
 *   warp 4, one thread         issues tcgen05.mma (M = 128 weight rows, N = pairs rounded up to 16, K = 16 per
 *                              instruction) and commits each pipeline stage / each finished tile to an mbarrier
 *   warps 0..3                 epilogue: tcgen05.ld of the accumulator (lane = weight row, column = pair), row scale,
 *                              SwiGLU (two matrices) or plain store (down), coalesced along the rows
 * The accumulators are double-buffered in tensor memory (2 x 2 x 128 columns of the 512), so the epilogue of one
 * tile overlaps the main loop of the next.  Every wait is bounded; a wait that runs out sets the status word, and the
 * CTA frees its tensor memory and returns.
 *
 * K' order.  The contraction does not care in which order k runs as long as A and B agree, so the operand tiles use
 * the order that makes the dequantisation cheapest: inside a 256-block, 64-wide atom c = ggml chunk c; its first
 * four 16-byte pieces hold the low nibbles (sub-block 2c), the last four the high nibbles (sub-block 2c+1); piece p
 * covers bytes 8p..8p+7 of the chunk in the order 0,2,1,3,4,6,5,7 (what the two-at-a-time extraction yields).
 */
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "batch_launch.h"
#include "dots.cuh"
#include "launch.h"
#include "route.cuh"
#include "stream.cuh"
#include "synth.h"

#define KB_THREADS 448
#define KB_COPY_WARP 13 /* one thread of it fetches the raw weight units */
#define KB_PROD_WARP0 5
#define KB_PROD_THREADS 256
#define KB_ATOM_BYTES 16384u /* 128 rows x 64 fp16 */
#define KB_WAIT_LIMIT (1u << 22)

/* position p (0..255) of the operand order inside a block -> the ggml index k it holds */
__host__ __device__ __forceinline__ int kb_kprime_to_k(int p) {
    const int cc = p >> 6, ch = (p >> 3) & 7, e = p & 7;
    const int hi = ch >> 2, wp = ch & 3;
    const int j = 2 * wp + (e >> 2);
    const int b = ((e & 3) == 1) ? 2 : ((e & 3) == 2) ? 1 : (e & 3);
    return 64 * cc + 32 * hi + 4 * j + b;
}

/* ------------------------------------------------------------------ table: generate / repack / export */
__device__ __forceinline__ uint8_t *kb_unit(uint8_t *mat, int K, int row, int kb) {
    return mat + ((uint64_t)(row >> 7) * (K / 256) + kb) * KB_TILE_BYTES;
}

/* A shard of a matrix: local block (row, kb) is block (row0 + row, kb0 + kb) of the full matrix, whose rows hold
 * bpr_full blocks; the synthetic generator and the ggml source are indexed by the full matrix's block number. */
__global__ void k_kb_gen(uint8_t *dst0, uint64_t rec_bytes, uint64_t mat_off, int M, int K, uint64_t seed, uint32_t layer,
                         uint32_t matrix, int row0, int bpr_full, int kb0) {
    const uint32_t e = blockIdx.y;
    uint8_t *mat = dst0 + (uint64_t)e * rec_bytes + mat_off;
    const uint64_t key = fsyn_key(seed, layer, e, matrix);
    const int bpr = K / 256, n = M * bpr;
    for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < n; b += gridDim.x * blockDim.x) {
        const int row = b / bpr, kb = b - row * bpr;
        uint32_t w[36];
        fsyn_q4k_block(key, (uint64_t)(row0 + row) * bpr_full + (kb0 + kb), w);
        uint4 *u = reinterpret_cast<uint4 *>(kb_unit(mat, K, row, kb)) + (row & 127);
#pragma unroll
        for (int p = 0; p < 9; p++) u[128 * p] = make_uint4(w[4 * p], w[4 * p + 1], w[4 * p + 2], w[4 * p + 3]);
    }
}

__global__ void k_kb_repack(uint8_t *mat, const uint8_t *src, int M, int K, int to_ggml, int row0, int bpr_full, int kb0) {
    const int bpr = K / 256, n = M * bpr;
    for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < n; b += gridDim.x * blockDim.x) {
        const int row = b / bpr, kb = b - row * bpr;
        uint4 *u = reinterpret_cast<uint4 *>(kb_unit(mat, K, row, kb)) + (row & 127);
        uint4 *g = reinterpret_cast<uint4 *>(const_cast<uint8_t *>(src) + ((uint64_t)(row0 + row) * bpr_full + (kb0 + kb)) * 144);
        for (int p = 0; p < 9; p++) {
            if (to_ggml) g[p] = u[128 * p];
            else u[128 * p] = g[p];
        }
    }
}

__global__ void k_kb_gen_f32(float *dst, uint64_t n, uint64_t key, float mean, float std) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        dst[i] = fsyn_f32(key, i, mean, std);
}

/* ------------------------------------------------------------------ prologue / activation quantiser
 * One block per row.  Optional glue first (x += resid; h = x * s * w with s = 1/sqrt(mean(x^2) + eps),
 * src/tensor.c:175-184).  Then quantize_row_q8_K per 256 (src/quant.c:343-375: amax, iscale = 127/amax, roundf, clamp,
 * d = 1/iscale; an all-zero block gives zeros) and the row goes out as fp16( q * d_block / d_max ) in K' order. */
#define KBQ_THREADS 256
#define KBQ_MAX_K 8192

__global__ void __launch_bounds__(KBQ_THREADS) k_kb_rows(float *x, const float *src, const float *resid, const float *normw,
                                                        float rms_eps, int n, float *h_out, uint16_t *xh, float *xscale,
                                                        int16_t *xbs, int exact) {
    __shared__ float s_red[KBQ_THREADS / 32];
    __shared__ float s_scale, s_dmax;
    __shared__ float s_d[KBQ_MAX_K / 256];
    extern __shared__ __align__(16) uint8_t dyn[];
    float *s_h = reinterpret_cast<float *>(dyn);       /* [n] */
    int8_t *s_q = reinterpret_cast<int8_t *>(s_h + n); /* [n] */
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = n / 256;
    if (x) { /* glue */
        float ss = 0.0f;
        for (int i = tid; i < n; i += KBQ_THREADS) {
            float v = x[(size_t)row * n + i];
            if (resid) v = __fadd_rn(v, resid[i]);
            x[(size_t)row * n + i] = v;
            s_h[i] = v;
            ss = __fmaf_rn(v, v, ss);
        }
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_red[warp] = ss;
        __syncthreads();
        if (tid == 0) {
            float t = 0.0f;
            for (int w = 0; w < KBQ_THREADS / 32; w++) t += s_red[w];
            s_scale = normw ? __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)n), rms_eps))) : 1.0f;
        }
        __syncthreads();
        const float sc = s_scale;
        for (int i = tid; i < n; i += KBQ_THREADS) {
            const float h = normw ? __fmul_rn(__fmul_rn(s_h[i], sc), normw[i]) : s_h[i];
            s_h[i] = h;
            if (h_out) h_out[(size_t)row * n + i] = h;
        }
    } else {
        for (int i = tid; i < n; i += KBQ_THREADS) s_h[i] = src[(size_t)row * n + i];
    }
    __syncthreads();
    for (int b = warp; b < nb; b += KBQ_THREADS / 32) { /* one warp per 256-block, 8 values per lane */
        float v[8], amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            v[i] = s_h[b * 256 + 8 * lane + i];
            amax = fmaxf(amax, fabsf(v[i]));
        }
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float d = 0.0f;
        int q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (amax != 0.0f) {
            const float iscale = __fdiv_rn(127.0f, amax);
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = max(-127, min(127, (int)roundf(__fmul_rn(iscale, v[i]))));
            d = __fdiv_rn(1.0f, iscale);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) s_q[b * 256 + 8 * lane + i] = (int8_t)q[i];
        if (lane == 0) s_d[b] = d;
    }
    __syncthreads();
    if (tid == 0) {
        float m = 0.0f;
        for (int b = 0; b < nb; b++) m = fmaxf(m, s_d[b]);
        s_dmax = m;
        if (!exact) xscale[row] = m;
    }
    if (exact) { /* block scales and the sums over the 32-wide sub-blocks (the bsums pairs of src/quant.c:368-372) */
        for (int b = tid; b < nb; b += KBQ_THREADS) xscale[(size_t)row * nb + b] = s_d[b];
        for (int i = tid; i < nb * 8; i += KBQ_THREADS) {
            int sum = 0;
            for (int k = 0; k < 32; k++) sum += s_q[i * 32 + k];
            xbs[(size_t)row * nb * 8 + i] = (int16_t)sum; /* at most 32 * 127 */
        }
    }
    __syncthreads();
    const float dmax = s_dmax;
    uint4 *out = reinterpret_cast<uint4 *>(xh + (size_t)row * n);
    for (int c = tid; c < n / 8; c += KBQ_THREADS) { /* 8 fp16 = one 16-byte piece */
        const int b = c >> 5, p0 = (c & 31) * 8;
        const float r = exact ? 1.0f : (dmax > 0.0f ? __fdiv_rn(s_d[b], dmax) : 0.0f);
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
            const float a0 = __fmul_rn((float)s_q[b * 256 + kb_kprime_to_k(p0 + e)], r);
            const float a1 = __fmul_rn((float)s_q[b * 256 + kb_kprime_to_k(p0 + e + 1)], r);
            const __half2 hh = __floats2half2_rn(a0, a1);
            w[e >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
        }
        out[c] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

/* ------------------------------------------------------------------ route: one warp per token
 * softmax over all experts (src/tensor.c:186-200), top-k by (probability descending, lower index first)
 * (src/tensor.c:226-252), weights renormalised with the sum taken in list order (src/inference.c:496-502). */
__global__ void k_kb_route(const float *logits, int n_tokens, int n_experts, int top_k, int *ids, float *scores,
                           int *status) {
    const int lane = threadIdx.x & 31, tok = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (tok >= n_tokens) return;
    const float *lg = logits + (size_t)tok * n_experts;
    float v[16];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int e = j * 32 + lane;
        v[j] = e < n_experts ? lg[e] : -INFINITY;
        mx = fmaxf(mx, v[j]);
    }
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, o));
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        v[j] = (j * 32 + lane < n_experts) ? expf(v[j] - mx) : 0.0f;
        sum += v[j];
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(FULL, sum, o);
    const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = (j * 32 + lane < n_experts) ? __fmul_rn(v[j], inv) : -1.0f;
    uint32_t taken = 0;
    float my_score = 0.0f;
    int my_id = 0;
    for (int r = 0; r < top_k; r++) {
        float bv = -1.0f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const int e = j * 32 + lane;
            if (e < n_experts && !((taken >> j) & 1u) && fb_better(v[j], e, bv, bi)) {
                bv = v[j];
                bi = e;
            }
        }
        fb_warp_best(bv, bi);
        if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
        if (lane == r) {
            my_score = bv;
            my_id = bi;
        }
    }
    float ssum = 0.0f;
    for (int r = 0; r < top_k; r++) ssum = __fadd_rn(ssum, __shfl_sync(FULL, my_score, r));
    if (lane < top_k) {
        if (my_id < 0 || my_id >= n_experts) {
            atomicExch(status, FB_ST_BAD_ID);
            my_id = 0;
        }
        ids[(size_t)tok * top_k + lane] = my_id;
        scores[(size_t)tok * top_k + lane] = ssum > 0.0f ? __fmul_rn(my_score, __fdiv_rn(1.0f, ssum)) : my_score;
    }
}

/* ------------------------------------------------------------------ bucket: pairs by expert + work items (one block) */
#define KBB_THREADS 1024
#define KBB_MAX_E 513

__global__ void __launch_bounds__(KBB_THREADS) k_kb_bucket(const int *ids, int n_tokens, int n_experts, int top_k,
                                                          int has_shared, int m_gu, int m_dn, int *counts, int *pairs,
                                                          kb_item_t *items_gu, int *n_items_gu, kb_item_t *items_dn,
                                                          int *n_items_dn) {
    __shared__ int cnt[KBB_MAX_E], off[KBB_MAX_E + 1], cur[KBB_MAX_E], coff[2][KBB_MAX_E + 1];
    const int tid = threadIdx.x, nE = n_experts + (has_shared ? 1 : 0), np = n_tokens * top_k;
    for (int e = tid; e < nE; e += KBB_THREADS) cnt[e] = cur[e] = 0;
    __syncthreads();
    for (int p = tid; p < np; p += KBB_THREADS) atomicAdd(&cnt[ids[p]], 1);
    __syncthreads();
    if (tid == 0) {
        if (has_shared) cnt[n_experts] = n_tokens;
        int o = 0, c0 = 0, c1 = 0;
        for (int e = 0; e < nE; e++) {
            off[e] = o;
            coff[0][e] = c0;
            coff[1][e] = c1;
            o += cnt[e];
            c0 += (cnt[e] + KB_GU_N - 1) / KB_GU_N;
            c1 += (cnt[e] + KB_TILE_N - 1) / KB_TILE_N;
        }
        off[nE] = o;
        coff[0][nE] = c0;
        coff[1][nE] = c1;
        *n_items_gu = c0 * m_gu;
        *n_items_dn = c1 * m_dn;
    }
    __syncthreads();
    for (int p = tid; p < np; p += KBB_THREADS) {
        const int e = ids[p];
        pairs[off[e] + atomicAdd(&cur[e], 1)] = p;
    }
    if (has_shared)
        for (int t = tid; t < n_tokens; t += KBB_THREADS) pairs[off[n_experts] + t] = np + t;
    for (int e = tid; e < nE; e += KBB_THREADS) {
        counts[e] = cnt[e];
        for (int pass = 0; pass < 2; pass++) {
            kb_item_t *items = pass ? items_dn : items_gu;
            const int mt = pass ? m_dn : m_gu, tn = pass ? KB_TILE_N : KB_GU_N;
            const int ch = coff[pass][e + 1] - coff[pass][e];
            for (int m = 0; m < mt; m++)
                for (int c = 0; c < ch; c++) {
                    kb_item_t it;
                    it.e = e;
                    it.m = m;
                    it.n0 = off[e] + c * tn;
                    it.n = min(tn, cnt[e] - c * tn);
                    items[mt * coff[pass][e] + m * ch + c] = it;
                }
        }
    }
}

/* ------------------------------------------------------------------ tcgen05 helpers */
__device__ __forceinline__ bool kb_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < KB_WAIT_LIMIT; i++) {
        if (fb_mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}

/* the same, adding the cycles waited to prof[slot] when profiling is on (block 0, one lane per warp) */
__device__ __forceinline__ bool kb_wait_p(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned long long *prof, int slot) {
    if (!prof) return kb_wait(bar, parity, abort_flag);
    const long long t0 = clock64();
    const bool r = kb_wait(bar, parity, abort_flag);
    if ((threadIdx.x & 31) == 0) atomicAdd(prof + slot, (unsigned long long)(clock64() - t0));
    return r;
}

/* shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart */
__device__ __forceinline__ uint64_t kb_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);        /* start address, bits [0,14) */
    d |= (uint64_t)1 << 16;                            /* leading byte offset (unused with swizzled K-major): 1 */
    d |= (uint64_t)(1024u >> 4) << 32;                 /* stride byte offset: 1024 bytes between 8-row groups */
    d |= (uint64_t)1 << 46;                            /* descriptor version of this architecture */
    d |= (uint64_t)2 << 61;                            /* layout type: 128-byte swizzle */
    return d;
}

/* instruction descriptor: fp16 x fp16 -> fp32, both operands K-major, M = 128, N = n */
__device__ __forceinline__ uint32_t kb_idesc(int n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void kb_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void kb_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void kb_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

/* 64 weights of one chunk (32 bytes = words w[0..7], low nibbles sub-block a, high nibbles sub-block b) -> fp16 into
 * row `row` of the atom at `atom_u`: pieces 0..3 low, 4..7 high, each piece at its swizzled place */
__device__ __forceinline__ void kb_dequant_atom(const uint4 &qa, const uint4 &qb, __half2 s_lo, __half2 b_lo, __half2 s_hi,
                                                __half2 b_hi, uint32_t atom_u, int row) {
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
    const uint32_t row_u = atom_u + (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
    const uint32_t sw = (uint32_t)(row & 7);
#pragma unroll
    for (int wp = 0; wp < 4; wp++) {
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t x = w[2 * wp + h];
            /* two nibbles at a time: (n | 0x6400) is the fp16 number 1024 + n */
            uint32_t l02 = (x & 0x000f000fu) | 0x64006400u, l13 = ((x >> 8) & 0x000f000fu) | 0x64006400u;
            uint32_t h02 = ((x >> 4) & 0x000f000fu) | 0x64006400u, h13 = ((x >> 12) & 0x000f000fu) | 0x64006400u;
            __half2 a = __hsub2(*reinterpret_cast<__half2 *>(&l02), k1024), b = __hsub2(*reinterpret_cast<__half2 *>(&l13), k1024);
            __half2 c = __hsub2(*reinterpret_cast<__half2 *>(&h02), k1024), d = __hsub2(*reinterpret_cast<__half2 *>(&h13), k1024);
            a = __hfma2(a, s_lo, b_lo);
            b = __hfma2(b, s_lo, b_lo);
            c = __hfma2(c, s_hi, b_hi);
            d = __hfma2(d, s_hi, b_hi);
            lo[2 * h] = *reinterpret_cast<uint32_t *>(&a);
            lo[2 * h + 1] = *reinterpret_cast<uint32_t *>(&b);
            hi[2 * h] = *reinterpret_cast<uint32_t *>(&c);
            hi[2 * h + 1] = *reinterpret_cast<uint32_t *>(&d);
        }
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(row_u + (((uint32_t)wp ^ sw) << 4)), "r"(lo[0]), "r"(lo[1]),
                     "r"(lo[2]), "r"(lo[3])
                     : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(row_u + (((uint32_t)(4 + wp) ^ sw) << 4)), "r"(hi[0]),
                     "r"(hi[1]), "r"(hi[2]), "r"(hi[3])
                     : "memory");
    }
}

/* ---- raw weight ring.  A (row tile, 256-block) unit of a matrix is 18,432 contiguous bytes, fetched by ONE bulk copy
 * (cp.async.bulk, completion counted in bytes on an mbarrier) into a ring of raw stages two 256-blocks deep, issued by
 * one producer thread two blocks ahead of the dequantisation: the HBM latency of the weights is off the producers'
 * path, and no registers are spent on prefetching.  A stage is released as soon as every producer warp has taken its
 * 144 bytes into registers. */
struct kb_cursor_t { /* which (work item, 256-block) the copy thread issues next */
    int it, kb;
};

/* the CTA's next block after (it, kb); false when the CTA's work ends */
__device__ __forceinline__ bool kb_cursor_next(kb_cursor_t &c, int kbs, int n_items, int stride) {
    if (++c.kb == kbs) {
        c.kb = 0;
        c.it += stride;
    }
    return c.it < n_items;
}

/* ------------------------------------------------------------------ down projection: one pass in fp16
 * (its result is not quantised again, so two fp16 roundings per product, about 2e-4 of the output, are inside the
 * bound).  A = fp16(d*sc*q - dmin*m), B = fp16(q8 * d_block / d_max), the row's d_max applied in the epilogue. */
#define KBD_STAGES 2
#define KBD_RAW 2
#define KBD_STAGE_BYTES (4u * KB_ATOM_BYTES) /* A: 2 atoms; B: 2 atoms of 128 rows */

struct kb_smem_ctl_t {
    uint64_t full[KBD_STAGES], empty[KBD_STAGES], acc_full[2], acc_empty[2], raw_full[KBD_RAW], raw_empty[KBD_RAW];
    uint32_t tmem_base;
    int abort_flag;
    int pair[2][KB_TILE_N], xrow[2][KB_TILE_N];
    float scale[2][KB_TILE_N];
};

__global__ void __launch_bounds__(KB_THREADS, 1) k_kb_down(kb_gemm_args_t P) {
    extern __shared__ uint8_t dyn_raw[];
    const uint32_t dyn_u = (fb_smem_u32(dyn_raw) + 1023u) & ~1023u; /* operand tiles: 1024-byte aligned */
    const uint32_t raw_u = dyn_u + KBD_STAGES * KBD_STAGE_BYTES;
    kb_smem_ctl_t *C = reinterpret_cast<kb_smem_ctl_t *>(dyn_raw + (raw_u - fb_smem_u32(dyn_raw)) + KBD_RAW * KB_TILE_BYTES);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_items = *P.n_items;
    const int kbs = P.K / 256, ksteps = P.K / 128;
    volatile int *abortp = &C->abort_flag;
    /* profiling aid: cycles block 0's roles wait -- [0] copy thread for a free raw stage, [1] producers for the pair
     * table's buffer, [2] for raw weights, [3] for a free operand stage, [4] MMA thread for a free accumulator,
     * [5] for a filled stage, [6] epilogue for a finished tile (sums over the waiting warps), [7] the block's run time */
    unsigned long long *prof = (blockIdx.x == 0) ? P.prof : nullptr;
    const long long t_start = clock64();

    if (tid == 0) {
        for (int s = 0; s < KBD_STAGES; s++) {
            fb_mbar_init(fb_smem_u32(&C->full[s]), KB_PROD_THREADS / 32);
            fb_mbar_init(fb_smem_u32(&C->empty[s]), 1);
        }
        for (int b = 0; b < 2; b++) {
            fb_mbar_init(fb_smem_u32(&C->acc_full[b]), 1);
            fb_mbar_init(fb_smem_u32(&C->acc_empty[b]), 4);
        }
        for (int r = 0; r < KBD_RAW; r++) {
            fb_mbar_init(fb_smem_u32(&C->raw_full[r]), 1);
            fb_mbar_init(fb_smem_u32(&C->raw_empty[r]), KB_PROD_THREADS / 32);
        }
        C->abort_flag = 0;
        fb_mbar_init_fence();
    }
    if (warp == 4) { /* tensor memory: two accumulator buffers of 128 columns */
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(fb_smem_u32(&C->tmem_base)), "r"(256u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = C->tmem_base;
    bool ok = true;

    if (warp == KB_COPY_WARP) {
        /* ---------------- copy thread: every 256-block of this CTA's tiles, in order, two blocks ahead of its use */
        if (lane == 0) {
            kb_cursor_t cur = {(int)blockIdx.x, -1};
            for (uint32_t blk = 0; kb_cursor_next(cur, kbs, n_items, gridDim.x); blk++) {
                const uint32_t r = blk % KBD_RAW, bar = fb_smem_u32(&C->raw_full[r]);
                if (blk >= KBD_RAW && !kb_wait_p(fb_smem_u32(&C->raw_empty[r]), ((blk / KBD_RAW) - 1) & 1, abortp, prof, 0)) { ok = false; break; }
                const kb_item_t J = P.items[cur.it];
                fb_mbar_expect_tx(bar, KB_TILE_BYTES);
                fb_bulk_g2s(raw_u + r * KB_TILE_BYTES,
                            P.w_layer + (uint64_t)J.e * P.rec_bytes + P.mat_off[0] + ((uint64_t)J.m * kbs + cur.kb) * KB_TILE_BYTES,
                            KB_TILE_BYTES, bar);
            }
        }
        __syncwarp();
    } else if (warp >= KB_PROD_WARP0) {
        /* ---------------- producers: dequantise A, copy B.  Thread (row, sel): row of the tile, and which of a step's
         * two atoms it dequantises. */
        const int pt = tid - KB_PROD_WARP0 * 32, row = pt & 127, sel = pt >> 7;
        uint32_t step = 0, cnt = 0, rb = 0; /* pipeline steps, tiles, 256-blocks so far */
        for (int it = blockIdx.x;; it += gridDim.x, cnt++) {
            /* All 256 producers meet here once per tile and leave together: a producer whose wait ran out arrives
             * with `false`, and nobody is left waiting at a barrier the others have abandoned. */
            const bool more = it < n_items;
            const int ab = cnt & 1;
            /* (the epilogue of the tile before last still reads this buffer's pair table) */
            bool w = ok && (!more || kb_wait_p(fb_smem_u32(&C->acc_empty[ab]), ((cnt >> 1) & 1) ^ 1, abortp, prof, 1));
            if (!w) C->abort_flag = 1;
            {
                uint32_t all;
                asm volatile(
                    "{\n"
                    ".reg .pred p, q;\n"
                    "setp.ne.b32 p, %1, 0;\n"
                    "barrier.cta.red.and.pred q, 1, %2, p;\n"
                    "selp.u32 %0, 1, 0, q;\n"
                    "}\n"
                    : "=r"(all)
                    : "r"((uint32_t)w), "n"(KB_PROD_THREADS)
                    : "memory");
                if (!all) {
                    ok = false;
                    break;
                }
            }
            if (!more) break;
            const kb_item_t I = P.items[it];
            if (pt < KB_TILE_N) {
                int p = 0, xr = 0;
                float sc = 0.0f;
                if (pt < I.n) {
                    p = P.pairs[I.n0 + pt];
                    const int npair = P.n_tokens * P.top_k;
                    xr = P.x_by_token ? (p < npair ? p / P.top_k : p - npair) : p;
                    sc = P.xscale[xr];
                }
                C->pair[ab][pt] = p;
                C->xrow[ab][pt] = xr;
                C->scale[ab][pt] = sc;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(KB_PROD_THREADS) : "memory");
            const int n_b = I.n * 16; /* 16-byte pieces of B per step: n rows x 2 atoms x 8 */
            for (int kb = 0; kb < kbs && ok; kb++, rb++) {
                const uint32_t r = rb % KBD_RAW;
                if (!__all_sync(0xffffffffu, kb_wait_p(fb_smem_u32(&C->raw_full[r]), (rb / KBD_RAW) & 1, abortp, prof, 2))) {
                    C->abort_flag = 1;
                    ok = false;
                    break;
                }
                const uint32_t u_u = raw_u + r * KB_TILE_BYTES + 16u * row;
                const uint4 hdr = fb_lds128(u_u);
                uint4 q[4]; /* the two chunks this thread dequantises: sel and 2 + sel */
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    q[2 * h] = fb_lds128(u_u + 2048u * (4 * h + 2 * sel + 1));
                    q[2 * h + 1] = fb_lds128(u_u + 2048u * (4 * h + 2 * sel + 2));
                }
                __syncwarp();
                if (lane == 0) fb_mbar_arrive(fb_smem_u32(&C->raw_empty[r]));
                const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffff)));
                const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
                /* 6-bit scales and mins of the 8 sub-blocks (src/quant.c:72-80), four to a word */
                const uint32_t sc_w[2] = {hdr.y & 0x3f3f3f3fu, (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4)};
                const uint32_t mn_w[2] = {hdr.z & 0x3f3f3f3fu, ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4)};
#pragma unroll
                for (int half = 0; half < 2; half++, step++) {
                    const int s = step % KBD_STAGES;
                    /* this thread's activation pieces of the step: requested before the stage is waited for */
                    uint4 bv[8];
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int i = pt + u * KB_PROD_THREADS;
                        if (i < n_b) {
                            const int rr = i >> 4, a = (i >> 3) & 1, ch = i & 7;
                            bv[u] = __ldg(reinterpret_cast<const uint4 *>(P.xh + (size_t)C->xrow[ab][rr] * P.K + kb * 256 + half * 128 + a * 64) + ch);
                        }
                    }
                    if (!__all_sync(0xffffffffu, kb_wait_p(fb_smem_u32(&C->empty[s]), ((step / KBD_STAGES) & 1) ^ 1, abortp, prof, 3))) {
                        C->abort_flag = 1; /* the whole warp stops producing; the tile barrier above ends the role */
                        ok = false;
                        break;
                    }
                    const uint32_t st_u = dyn_u + s * KBD_STAGE_BYTES;
                    {
                        const int a = sel; /* chunk = atom: sub-blocks 2cc (low nibbles), 2cc+1 (high) */
                        const float sl = (float)((sc_w[half] >> (16 * a)) & 0xff), sh = (float)((sc_w[half] >> (16 * a + 8)) & 0xff);
                        const float ml = (float)((mn_w[half] >> (16 * a)) & 0xff), mh = (float)((mn_w[half] >> (16 * a + 8)) & 0xff);
                        const __half2 s_lo = __float2half2_rn(__fmul_rn(d, sl)), b_lo = __float2half2_rn(-__fmul_rn(dmin, ml));
                        const __half2 s_hi = __float2half2_rn(__fmul_rn(d, sh)), b_hi = __float2half2_rn(-__fmul_rn(dmin, mh));
                        kb_dequant_atom(q[2 * half], q[2 * half + 1], s_lo, b_lo, s_hi, b_hi, st_u + a * KB_ATOM_BYTES, row);
                    }
                    const uint32_t b_u = st_u + 2 * KB_ATOM_BYTES;
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int i = pt + u * KB_PROD_THREADS;
                        if (i < n_b) {
                            const int rr = i >> 4, a = (i >> 3) & 1, ch = i & 7;
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(b_u + a * KB_ATOM_BYTES + (uint32_t)(rr >> 3) * 1024u + (uint32_t)(rr & 7) * 128u + (((uint32_t)ch ^ (uint32_t)(rr & 7)) << 4)),
                                         "r"(bv[u].x), "r"(bv[u].y), "r"(bv[u].z), "r"(bv[u].w)
                                         : "memory");
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); /* generic-proxy stores -> the tensor core's reads */
                    __syncwarp();
                    if (lane == 0) fb_mbar_arrive(fb_smem_u32(&C->full[s]));
                }
            }
        }
    } else if (warp == 4) {
        /* ---------------- MMA issue: one thread */
        if (lane == 0) {
            uint32_t step = 0, cnt = 0;
            for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, cnt++) {
                const kb_item_t I = P.items[it];
                const int ab = cnt & 1;
                const uint32_t idesc = kb_idesc((I.n + 15) & ~15);
                if (!kb_wait_p(fb_smem_u32(&C->acc_empty[ab]), ((cnt >> 1) & 1) ^ 1, abortp, prof, 4)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int ks = 0; ks < ksteps && ok; ks++, step++) {
                    const int s = step % KBD_STAGES;
                    if (!kb_wait_p(fb_smem_u32(&C->full[s]), (step / KBD_STAGES) & 1, abortp, prof, 5)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st_u = dyn_u + s * KBD_STAGE_BYTES, b_u = st_u + 2 * KB_ATOM_BYTES;
#pragma unroll
                    for (int a = 0; a < 2; a++)
#pragma unroll
                        for (int k16 = 0; k16 < 4; k16++)
                            kb_mma(tmem + (uint32_t)ab * KB_TILE_N, kb_smem_desc(st_u + a * KB_ATOM_BYTES + k16 * 32),
                                   kb_smem_desc(b_u + a * KB_ATOM_BYTES + k16 * 32), idesc, (ks | a | k16) ? 1u : 0u);
                    kb_commit(fb_smem_u32(&C->empty[s])); /* the stage is free once these MMAs have read it */
                }
                if (ok) kb_commit(fb_smem_u32(&C->acc_full[ab]));
            }
        }
        __syncwarp();
    } else {
        /* ---------------- epilogue: warp q reads accumulator lanes 32q .. 32q+31 = tile rows */
        uint32_t cnt = 0;
        for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, cnt++) {
            const kb_item_t I = P.items[it];
            const int ab = cnt & 1;
            if (!__all_sync(0xffffffffu, kb_wait_p(fb_smem_u32(&C->acc_full[ab]), (cnt >> 1) & 1, abortp, prof, 6))) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int grow = I.m * KB_TILE_M + warp * 32 + lane;
            const uint32_t t0 = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)ab * KB_TILE_N;
            for (int c0 = 0; c0 < I.n; c0 += 16) {
                uint32_t g[16];
                kb_tmem_ld16(t0 + c0, g);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; j++)
                    if (c0 + j < I.n)
                        P.out[(size_t)C->pair[ab][c0 + j] * P.M + grow] = __fmul_rn(__uint_as_float(g[j]), C->scale[ab][c0 + j]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) fb_mbar_arrive(fb_smem_u32(&C->acc_empty[ab]));
        }
    }
    if (!ok) { /* a wait ran out: tell the other roles and the host */
        C->abort_flag = 1;
        atomicExch(P.status, FB_ST_WAIT_TIMEOUT);
    }
    if (prof && tid == 0) atomicAdd(prof + 7, (unsigned long long)(clock64() - t_start));
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
    }
}

/* ------------------------------------------------------------------ gate + up + SwiGLU: exact integer products
 *
 * The activations of the down projection are quantised to int8 from the OUTPUT of this pass, so a relative error of
 * 2e-4 here moves several of the 1024 int8 values of a row by one step and costs 2e-3 of the layer output (measured
 * with the one-pass fp16 form on both projections).  This pass therefore keeps the reference's integer arithmetic
 * (src/quant.c:405-476) on the tensor cores: A = sc_j * q (at most 945) and B = the int8 activation are exact in
 * fp16, a 256-block's sum of products is an exact integer in the fp32 accumulator (below 2^24 in all but adversarial
 * data, 2^25 at most), and each 256-block's accumulator is read out and scaled on the CUDA cores:
 *     sum += (yd * d) * isum - (yd * dmin) * sum_j m_j * bs_j
 * with bs_j the activation's sub-block sums.  Accumulators are double-buffered per 256-block in tensor memory, so the
 * epilogue of one block overlaps the MMAs of the next; at most 32 pairs per pass keep the running sums (2 x 32 per
 * weight row) in registers.  Roles and pipeline as in k_kb_down. */
#define KBG_STAGES 2
#define KBG_RAW 2
#define KBG_B_ATOM ((uint32_t)KB_GU_N * 128u)
#define KBG_A_BYTES (4u * KB_ATOM_BYTES)
#define KBG_STAGE_BYTES (KBG_A_BYTES + 2u * KBG_B_ATOM)

struct kbg_ctl_t {
    uint64_t full[KBG_STAGES], empty[KBG_STAGES], blk_full[2], blk_empty[2], item_done[2], raw_full[KBG_RAW], raw_empty[KBG_RAW];
    uint32_t tmem_base;
    int abort_flag;
    int pair[2][KB_GU_N], xrow[2][KB_GU_N];
    /* activation side of a 256-block's scaling, per pair: {d, the eight sub-block sums, pad}; written by the producers
     * with the block's operand tiles, read by the epilogue.  Four blocks deep: the producers run at most two blocks
     * ahead of the MMAs, and the MMAs at most two ahead of the epilogue. */
    alignas(16) uint4 xt[4][KB_GU_N][2];  /* {d as float bits, -, -, -}, {eight int16 sums} */
};

__global__ void __launch_bounds__(KB_THREADS, 1) k_kb_gateup(kb_gemm_args_t P) {
    extern __shared__ uint8_t dyn_raw[];
    const uint32_t dyn_u = (fb_smem_u32(dyn_raw) + 1023u) & ~1023u;
    const uint32_t raw_u = dyn_u + KBG_STAGES * KBG_STAGE_BYTES; /* raw stage: gate unit, then up unit */
    kbg_ctl_t *C = reinterpret_cast<kbg_ctl_t *>(dyn_raw + (raw_u - fb_smem_u32(dyn_raw)) + KBG_RAW * 2 * KB_TILE_BYTES);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_items = *P.n_items;
    const int kbs = P.K / 256;
    volatile int *abortp = &C->abort_flag;
    /* profiling aid, as in k_kb_down, slots 8..15: copy thread, producers (pair table / raw weights / operand stage),
     * MMA thread (accumulator buffer / filled stage), epilogue (a block's sums), the block's run time */
    unsigned long long *prof = (blockIdx.x == 0 && P.prof) ? P.prof + 8 : nullptr;
    const long long t_start = clock64();

    if (tid == 0) {
        for (int s = 0; s < KBG_STAGES; s++) {
            fb_mbar_init(fb_smem_u32(&C->full[s]), KB_PROD_THREADS / 32);
            fb_mbar_init(fb_smem_u32(&C->empty[s]), 1);
        }
        for (int b = 0; b < 2; b++) {
            fb_mbar_init(fb_smem_u32(&C->blk_full[b]), 1);
            fb_mbar_init(fb_smem_u32(&C->blk_empty[b]), 4);
            fb_mbar_init(fb_smem_u32(&C->item_done[b]), 4);
        }
        for (int r = 0; r < KBG_RAW; r++) {
            fb_mbar_init(fb_smem_u32(&C->raw_full[r]), 1);
            fb_mbar_init(fb_smem_u32(&C->raw_empty[r]), KB_PROD_THREADS / 32);
        }
        C->abort_flag = 0;
        fb_mbar_init_fence();
    }
    if (warp == 4) { /* tensor memory: 2 buffers x {gate, up} x 32 columns */
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(fb_smem_u32(&C->tmem_base)), "r"(128u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = C->tmem_base;
    bool ok = true;

    if (warp == KB_COPY_WARP) {
        /* ---------------- copy thread: gate and up unit of every 256-block, two blocks ahead */
        if (lane == 0) {
            kb_cursor_t cur = {(int)blockIdx.x, -1};
            for (uint32_t blk = 0; kb_cursor_next(cur, kbs, n_items, gridDim.x); blk++) {
                const uint32_t r = blk % KBG_RAW, bar = fb_smem_u32(&C->raw_full[r]);
                if (blk >= KBG_RAW && !kb_wait_p(fb_smem_u32(&C->raw_empty[r]), ((blk / KBG_RAW) - 1) & 1, abortp, prof, 0)) { ok = false; break; }
                const kb_item_t J = P.items[cur.it];
                const uint8_t *rec = P.w_layer + (uint64_t)J.e * P.rec_bytes;
                const uint64_t off = ((uint64_t)J.m * kbs + cur.kb) * KB_TILE_BYTES;
                fb_mbar_expect_tx(bar, 2 * KB_TILE_BYTES);
                fb_bulk_g2s(raw_u + r * 2 * KB_TILE_BYTES, rec + P.mat_off[0] + off, KB_TILE_BYTES, bar);
                fb_bulk_g2s(raw_u + r * 2 * KB_TILE_BYTES + KB_TILE_BYTES, rec + P.mat_off[1] + off, KB_TILE_BYTES, bar);
            }
        }
        __syncwarp();
    } else if (warp >= KB_PROD_WARP0) {
        /* ---------------- producers: thread (mat, row) */
        const int pt = tid - KB_PROD_WARP0 * 32, mat = pt >> 7, row = pt & 127;
        uint32_t step = 0, cnt = 0, rb = 0;
        for (int it = blockIdx.x;; it += gridDim.x, cnt++) {
            const bool more = it < n_items;
            const int ab = cnt & 1;
            bool w = ok && (!more || kb_wait_p(fb_smem_u32(&C->item_done[ab]), ((cnt >> 1) & 1) ^ 1, abortp, prof, 1));
            if (!w) C->abort_flag = 1;
            {
                uint32_t all;
                asm volatile(
                    "{\n"
                    ".reg .pred p, q;\n"
                    "setp.ne.b32 p, %1, 0;\n"
                    "barrier.cta.red.and.pred q, 1, %2, p;\n"
                    "selp.u32 %0, 1, 0, q;\n"
                    "}\n"
                    : "=r"(all)
                    : "r"((uint32_t)w), "n"(KB_PROD_THREADS)
                    : "memory");
                if (!all) {
                    ok = false;
                    break;
                }
            }
            if (!more) break;
            const kb_item_t I = P.items[it];
            if (pt < KB_GU_N) {
                int p = 0, xr = 0;
                if (pt < I.n) {
                    p = P.pairs[I.n0 + pt];
                    const int npair = P.n_tokens * P.top_k;
                    xr = P.x_by_token ? (p < npair ? p / P.top_k : p - npair) : p;
                }
                C->pair[ab][pt] = p;
                C->xrow[ab][pt] = xr;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(KB_PROD_THREADS) : "memory");
            const int n_b = I.n * 16; /* at most 512: two pieces per thread */
            const __half2 zero2 = __float2half2_rn(0.0f);
            for (int kb = 0; kb < kbs && ok; kb++, rb++) {
                const uint32_t r = rb % KBG_RAW;
                if (!__all_sync(0xffffffffu, kb_wait_p(fb_smem_u32(&C->raw_full[r]), (rb / KBG_RAW) & 1, abortp, prof, 2))) {
                    C->abort_flag = 1;
                    ok = false;
                    break;
                }
                const uint32_t u_u = raw_u + (r * 2 + mat) * KB_TILE_BYTES + 16u * row;
                const uint4 hdr = fb_lds128(u_u);
                uint4 q[8];
#pragma unroll
                for (int p = 0; p < 8; p++) q[p] = fb_lds128(u_u + 2048u * (p + 1));
                __syncwarp();
                if (lane == 0) fb_mbar_arrive(fb_smem_u32(&C->raw_empty[r]));
                const uint32_t sc_w[2] = {hdr.y & 0x3f3f3f3fu, (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4)};
                /* this block's scale and sub-block sums of every pair: one pair per thread (the first n threads) */
                uint4 xv = make_uint4(0, 0, 0, 0);
                float xd = 0.0f;
                if (pt < I.n) {
                    const size_t xb = (size_t)C->xrow[ab][pt] * kbs + kb;
                    xv = __ldg(reinterpret_cast<const uint4 *>(P.xbs + xb * 8));
                    xd = __ldg(P.xscale + xb);
                }
#pragma unroll
                for (int half = 0; half < 2; half++, step++) {
                    const int s = step % KBG_STAGES;
                    uint4 bv[2];
#pragma unroll
                    for (int u = 0; u < 2; u++) {
                        const int i = pt + u * KB_PROD_THREADS;
                        if (i < n_b) {
                            const int rr = i >> 4, a = (i >> 3) & 1, ch = i & 7;
                            bv[u] = __ldg(reinterpret_cast<const uint4 *>(P.xh + (size_t)C->xrow[ab][rr] * P.K + kb * 256 + half * 128 + a * 64) + ch);
                        }
                    }
                    if (!__all_sync(0xffffffffu, kb_wait_p(fb_smem_u32(&C->empty[s]), ((step / KBG_STAGES) & 1) ^ 1, abortp, prof, 3))) {
                        C->abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t st_u = dyn_u + s * KBG_STAGE_BYTES;
#pragma unroll
                    for (int a = 0; a < 2; a++) { /* A = sc_j * q: small integers, exact in fp16 */
                        const int cc = 2 * half + a;
                        const __half2 s_lo = __float2half2_rn((float)((sc_w[half] >> (16 * a)) & 0xff));
                        const __half2 s_hi = __float2half2_rn((float)((sc_w[half] >> (16 * a + 8)) & 0xff));
                        kb_dequant_atom(q[2 * cc], q[2 * cc + 1], s_lo, zero2, s_hi, zero2, st_u + (mat * 2 + a) * KB_ATOM_BYTES, row);
                    }
                    const uint32_t b_u = st_u + KBG_A_BYTES;
#pragma unroll
                    for (int u = 0; u < 2; u++) {
                        const int i = pt + u * KB_PROD_THREADS;
                        if (i < n_b) {
                            const int rr = i >> 4, a = (i >> 3) & 1, ch = i & 7;
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(b_u + a * KBG_B_ATOM + (uint32_t)(rr >> 3) * 1024u + (uint32_t)(rr & 7) * 128u + (((uint32_t)ch ^ (uint32_t)(rr & 7)) << 4)),
                                         "r"(bv[u].x), "r"(bv[u].y), "r"(bv[u].z), "r"(bv[u].w)
                                         : "memory");
                        }
                    }
                    if (half == 0 && pt < I.n) {
                        C->xt[rb & 3][pt][0] = make_uint4(__float_as_uint(xd), 0, 0, 0);
                        C->xt[rb & 3][pt][1] = xv;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) fb_mbar_arrive(fb_smem_u32(&C->full[s]));
                }
            }
        }
    } else if (warp == 4) {
        /* ---------------- MMA issue */
        if (lane == 0) {
            uint32_t step = 0, bc = 0;
            for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
                const kb_item_t I = P.items[it];
                const uint32_t idesc = kb_idesc((I.n + 15) & ~15);
                for (int kb = 0; kb < kbs && ok; kb++, bc++) {
                    const int buf = bc & 1;
                    if (!kb_wait_p(fb_smem_u32(&C->blk_empty[buf]), ((bc >> 1) & 1) ^ 1, abortp, prof, 4)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (int half = 0; half < 2 && ok; half++, step++) {
                        const int s = step % KBG_STAGES;
                        if (!kb_wait_p(fb_smem_u32(&C->full[s]), (step / KBG_STAGES) & 1, abortp, prof, 5)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t st_u = dyn_u + s * KBG_STAGE_BYTES, b_u = st_u + KBG_A_BYTES;
#pragma unroll
                        for (int a = 0; a < 2; a++)
#pragma unroll
                            for (int k16 = 0; k16 < 4; k16++) {
                                const uint64_t bdesc = kb_smem_desc(b_u + a * KBG_B_ATOM + k16 * 32);
#pragma unroll
                                for (int m = 0; m < 2; m++)
                                    kb_mma(tmem + (uint32_t)(buf * 2 + m) * KB_GU_N,
                                           kb_smem_desc(st_u + (m * 2 + a) * KB_ATOM_BYTES + k16 * 32), bdesc, idesc,
                                           (half | a | k16) ? 1u : 0u);
                            }
                        kb_commit(fb_smem_u32(&C->empty[s]));
                    }
                    if (ok) kb_commit(fb_smem_u32(&C->blk_full[buf])); /* this 256-block's integer sums are complete */
                }
            }
        }
        __syncwarp();
    } else {
        /* ---------------- epilogue: scale every 256-block's sums, SwiGLU at the end */
        uint32_t cnt = 0, bc = 0;
        for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, cnt++) {
            const kb_item_t I = P.items[it];
            const int ab = cnt & 1;
            const int trow = warp * 32 + lane, grow = I.m * KB_TILE_M + trow;
            float accg[KB_GU_N], accu[KB_GU_N];
#pragma unroll
            for (int j = 0; j < KB_GU_N; j++) accg[j] = accu[j] = 0.0f;
            const uint8_t *wg = P.w_layer + (uint64_t)I.e * P.rec_bytes + P.mat_off[0];
            const uint8_t *wu = P.w_layer + (uint64_t)I.e * P.rec_bytes + P.mat_off[1];
            for (int kb = 0; kb < kbs && ok; kb++, bc++) {
                const int buf = bc & 1;
                /* this row's block headers: d, dmin and the eight 6-bit mins of gate and up */
                const uint4 hg = __ldg(reinterpret_cast<const uint4 *>(wg + ((uint64_t)I.m * kbs + kb) * KB_TILE_BYTES) + trow);
                const uint4 hu = __ldg(reinterpret_cast<const uint4 *>(wu + ((uint64_t)I.m * kbs + kb) * KB_TILE_BYTES) + trow);
                const float dg = __half2float(__ushort_as_half((unsigned short)(hg.x & 0xffff)));
                const float ng = __half2float(__ushort_as_half((unsigned short)(hg.x >> 16)));
                const float du = __half2float(__ushort_as_half((unsigned short)(hu.x & 0xffff)));
                const float nu = __half2float(__ushort_as_half((unsigned short)(hu.x >> 16)));
                const uint32_t mgw[2] = {hg.z & 0x3f3f3f3fu, ((hg.w >> 4) & 0x0f0f0f0fu) | (((hg.z >> 6) & 0x03030303u) << 4)};
                const uint32_t muw[2] = {hu.z & 0x3f3f3f3fu, ((hu.w >> 4) & 0x0f0f0f0fu) | (((hu.z >> 6) & 0x03030303u) << 4)};
                if (!__all_sync(0xffffffffu, kb_wait_p(fb_smem_u32(&C->blk_full[buf]), (bc >> 1) & 1, abortp, prof, 6))) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t t0 = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(buf * 2) * KB_GU_N;
#pragma unroll
                for (int c0 = 0; c0 < KB_GU_N; c0 += 16) { /* 16 pairs at a time: the sums, their scaling */
                    if (c0 < I.n) {
                        uint32_t ig[16], iu[16];
                        kb_tmem_ld16(t0 + c0, ig);
                        kb_tmem_ld16(t0 + KB_GU_N + c0, iu);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            if (c0 + j < I.n) {
                                const float yd = __uint_as_float(C->xt[bc & 3][c0 + j][0].x);
                                const uint4 bs = C->xt[bc & 3][c0 + j][1]; /* int16 pairs (bs_0, bs_1) .. (bs_6, bs_7) */
                                /* sum_j m_j * bs_j in exact integers, two terms per instruction (int16 pair x byte pair) */
                                int msg = fb_dp2a_lo_su(bs.x, mgw[0], 0), msu = fb_dp2a_lo_su(bs.x, muw[0], 0);
                                msg = fb_dp2a_hi_su(bs.y, mgw[0], msg);
                                msu = fb_dp2a_hi_su(bs.y, muw[0], msu);
                                msg = fb_dp2a_lo_su(bs.z, mgw[1], msg);
                                msu = fb_dp2a_lo_su(bs.z, muw[1], msu);
                                msg = fb_dp2a_hi_su(bs.w, mgw[1], msg);
                                msu = fb_dp2a_hi_su(bs.w, muw[1], msu);
                                accg[c0 + j] = __fmaf_rn(__fmul_rn(yd, dg), __uint_as_float(ig[j]), accg[c0 + j]);
                                accg[c0 + j] = __fmaf_rn(-__fmul_rn(yd, ng), (float)msg, accg[c0 + j]);
                                accu[c0 + j] = __fmaf_rn(__fmul_rn(yd, du), __uint_as_float(iu[j]), accu[c0 + j]);
                                accu[c0 + j] = __fmaf_rn(-__fmul_rn(yd, nu), (float)msu, accu[c0 + j]);
                            }
                        }
                    }
                }
                /* all of this block's sums have been read: its buffer can take the block after next */
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) fb_mbar_arrive(fb_smem_u32(&C->blk_empty[buf]));
            }
            if (!ok) break;
#pragma unroll
            for (int j = 0; j < KB_GU_N; j++)
                if (j < I.n) { /* silu(gate) * up, src/cpu_expert.c:103-106 */
                    const float g = accg[j];
                    P.out[(size_t)C->pair[ab][j] * P.M + grow] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), accu[j]);
                }
            __syncwarp();
            if (lane == 0) fb_mbar_arrive(fb_smem_u32(&C->item_done[ab])); /* the pair table of this buffer is free */
        }
    }
    if (!ok) {
        C->abort_flag = 1;
        atomicExch(P.status, FB_ST_WAIT_TIMEOUT);
    }
    if (prof && tid == 0) atomicAdd(prof + 7, (unsigned long long)(clock64() - t_start));
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
    }
}

/* x += y (the block output after the ranks' partial outputs have been summed) */
__global__ void k_kb_add(float *x, const float *y, uint64_t n4) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n4; i += (uint64_t)gridDim.x * blockDim.x) {
        float4 a = reinterpret_cast<float4 *>(x)[i];
        const float4 b = reinterpret_cast<const float4 *>(y)[i];
        a.x = __fadd_rn(a.x, b.x); a.y = __fadd_rn(a.y, b.y); a.z = __fadd_rn(a.z, b.z); a.w = __fadd_rn(a.w, b.w);
        reinterpret_cast<float4 *>(x)[i] = a;
    }
}

extern "C" int kb_launch_add(float *x, const float *y, uint64_t n, void *stream) {
    const uint64_t n4 = n / 4, g = (n4 + 255) / 256;
    k_kb_add<<<(int)(g > 1184 ? 1184 : (g < 1 ? 1 : g)), 256, 0, (cudaStream_t)stream>>>(x, y, n4);
    return (int)cudaGetLastError();
}

/* ------------------------------------------------------------------ combine */
__global__ void k_kb_combine(const float *dots, const float *scores, int n_tokens, int n_embd, int top_k, int has_shared,
                             float *out, float *x) {
    const int t = blockIdx.y;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_embd; i += gridDim.x * blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < top_k; s++) /* partial += score * down in list order, src/cpu_expert.c:114-115 */
            acc = __fmaf_rn(scores[(size_t)t * top_k + s], dots[((size_t)t * top_k + s) * n_embd + i], acc);
        if (has_shared) acc = __fadd_rn(acc, dots[((size_t)n_tokens * top_k + t) * n_embd + i]); /* src/inference.c:595 */
        if (out) out[(size_t)t * n_embd + i] = acc;
        if (x) x[(size_t)t * n_embd + i] = __fadd_rn(x[(size_t)t * n_embd + i], acc);
    }
}

/* ------------------------------------------------------------------ launchers */
extern "C" int kb_launch_gen(uint8_t *dst, uint64_t rec_bytes, int n_recs, uint64_t mat_off, int M, int K, uint64_t seed,
                             uint32_t layer, uint32_t matrix, int row0, int bpr_full, int kb0, void *stream) {
    const int n = M * (K / 256);
    dim3 grid((n + 127) / 128 > 256 ? 256 : (n + 127) / 128, n_recs);
    k_kb_gen<<<grid, 128, 0, (cudaStream_t)stream>>>(dst, rec_bytes, mat_off, M, K, seed, layer, matrix, row0, bpr_full, kb0);
    return (int)cudaGetLastError();
}

extern "C" int kb_launch_repack(uint8_t *dst, const uint8_t *src_ggml, int M, int K, int row0, int bpr_full, int kb0, void *stream) {
    const int n = M * (K / 256);
    k_kb_repack<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(dst, src_ggml, M, K, 0, row0, bpr_full, kb0);
    return (int)cudaGetLastError();
}

extern "C" int kb_launch_export(uint8_t *dst_ggml, const uint8_t *src, int M, int K, void *stream) {
    const int n = M * (K / 256);
    k_kb_repack<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(const_cast<uint8_t *>(src), dst_ggml, M, K, 1, 0, K / 256, 0);
    return (int)cudaGetLastError();
}

extern "C" int kb_launch_gen_f32(float *dst, uint64_t n, uint64_t seed, uint32_t layer, uint32_t stream_id, float mean,
                                 float std, void *stream) {
    const uint64_t key = fsyn_key(seed, layer, 0, stream_id);
    const uint64_t g = (n + 255) / 256;
    k_kb_gen_f32<<<(int)(g > 1184 ? 1184 : (g < 1 ? 1 : g)), 256, 0, (cudaStream_t)stream>>>(dst, n, key, mean, std);
    return (int)cudaGetLastError();
}

extern "C" int kb_launch_prologue(float *x, const float *resid, const float *normw, float rms_eps, int n_tokens, int n_embd,
                                  float *h_out, uint16_t *xh, float *xscale, int16_t *xbs, void *stream) {
    if (n_embd > KBQ_MAX_K || n_embd % 256) return (int)cudaErrorInvalidValue;
    k_kb_rows<<<n_tokens, KBQ_THREADS, (size_t)n_embd * 5, (cudaStream_t)stream>>>(x, nullptr, resid, normw, rms_eps, n_embd,
                                                                                  h_out, xh, xscale, xbs, 1);
    return (int)cudaGetLastError();
}

extern "C" int kb_launch_quant(const float *src, int rows, int n, int exact, uint16_t *xh, float *xscale, int16_t *xbs,
                               void *stream) {
    if (n > KBQ_MAX_K || n % 256 || (exact && !xbs)) return (int)cudaErrorInvalidValue;
    k_kb_rows<<<rows, KBQ_THREADS, (size_t)n * 5, (cudaStream_t)stream>>>(nullptr, src, nullptr, nullptr, 0.0f, n, nullptr, xh,
                                                                         xscale, xbs, exact);
    return (int)cudaGetLastError();
}

extern "C" int kb_launch_route(const float *logits, int n_tokens, int n_experts, int top_k, int *ids, float *scores,
                               int *status, void *stream) {
    if (n_experts > 512 || top_k > 32) return (int)cudaErrorInvalidValue;
    k_kb_route<<<(n_tokens + 7) / 8, 256, 0, (cudaStream_t)stream>>>(logits, n_tokens, n_experts, top_k, ids, scores, status);
    return (int)cudaGetLastError();
}

extern "C" int kb_launch_bucket(const int *ids, int n_tokens, int n_experts, int top_k, int has_shared, int m_tiles_gu,
                                int m_tiles_dn, int *counts, int *pairs, kb_item_t *items_gu, int *n_items_gu,
                                kb_item_t *items_dn, int *n_items_dn, void *stream) {
    if (n_experts + 1 > KBB_MAX_E) return (int)cudaErrorInvalidValue;
    k_kb_bucket<<<1, KBB_THREADS, 0, (cudaStream_t)stream>>>(ids, n_tokens, n_experts, top_k, has_shared, m_tiles_gu,
                                                            m_tiles_dn, counts, pairs, items_gu, n_items_gu, items_dn,
                                                            n_items_dn);
    return (int)cudaGetLastError();
}

extern "C" int kb_launch_down(const kb_gemm_args_t *a, int grid, void *stream) {
    static unsigned char configured[64]; /* the attribute holds for one device */
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    const int sm = 1024 + KBD_STAGES * (int)KBD_STAGE_BYTES + KBD_RAW * (int)KB_TILE_BYTES + (int)sizeof(kb_smem_ctl_t);
    if (!configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(k_kb_down, cudaFuncAttributeMaxDynamicSharedMemorySize, sm);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = 1;
    }
    k_kb_down<<<grid, KB_THREADS, sm, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int kb_launch_gateup(const kb_gemm_args_t *a, int grid, void *stream) {
    static unsigned char configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    const int sm = 1024 + KBG_STAGES * (int)KBG_STAGE_BYTES + KBG_RAW * 2 * (int)KB_TILE_BYTES + (int)sizeof(kbg_ctl_t);
    if (!configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(k_kb_gateup, cudaFuncAttributeMaxDynamicSharedMemorySize, sm);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = 1;
    }
    k_kb_gateup<<<grid, KB_THREADS, sm, (cudaStream_t)stream>>>(*a);
    return (int)cudaGetLastError();
}

extern "C" int kb_launch_combine(const float *dots, const float *scores, int n_tokens, int n_embd, int top_k, int has_shared,
                                 float *out, float *x, void *stream) {
    dim3 grid((n_embd + 255) / 256, n_tokens);
    k_kb_combine<<<grid, 256, 0, (cudaStream_t)stream>>>(dots, scores, n_tokens, n_embd, top_k, has_shared, out, x);
    return (int)cudaGetLastError();
}
