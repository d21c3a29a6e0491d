/*
 * batch_launch.h -- plain-C interface between the host library and the kernels of the BATCHED routed-expert FFN
 * (many tokens per call: prefill, or decode of many sequences), batch.cu.
 *
 * At batch 1 an expert FFN is a memory-bound matvec and runs on integer dot products (stack.cu, kernels.cu).  With
 * tokens-per-expert well above one it is a dense contraction: tokens are bucketed by expert on the device and each
 * (expert, 128-row tile) runs on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory), with
 * the Q4_K weights dequantised to fp16 on the way from HBM into the operand tiles.  The reference has no batched
 * expert path at all (its fused kernel is batch-1 only, src/gpu_kernels.hip:1320-1384, and gpu_expert_ffn takes one
 * hidden state, include/gpu.h:70-83); the definition computed is the same one: src/cpu_expert.c applied to every
 * token (activations quantised to Q8_K per 256, SwiGLU, down projection, weighted sum in list order).
 */
#ifndef FOMOE_B200_BATCH_LAUNCH_H
#define FOMOE_B200_BATCH_LAUNCH_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KB_TILE_M 128     /* weight rows per tile = MMA M */
#define KB_TILE_N 128     /* (token, expert) pairs per pass of the down projection = at most this many MMA columns */
#define KB_GU_N 32        /* the same for the gate/up pass, whose epilogue keeps 2 x 32 running sums in registers */
#define KB_TILE_BYTES (128u * 144u) /* one (row tile, 256-column block) unit of a matrix: 128 Q4_K blocks */

/* One unit of work of the grouped GEMM: rows [128 m, 128 m + 128) of expert e's matrices against n entries of the
 * expert's pair list starting at n0. */
typedef struct {
    int e, m, n0, n;
} kb_item_t;

typedef struct {
    /* weights: batched layout.  A matrix [M x K] is stored tile by tile, [M/128][K/256] units of 18,432 bytes; a unit
     * holds the 128 Q4_K blocks (row r of the tile, that 256-column block) as uint4 piece[9][128]: piece 0 = the
     * 16-byte header {d | dmin << 16, scales[12]}, pieces 1..8 = the 128 quant bytes, 16 at a time.  No padding: a
     * matrix takes its ggml size. */
    const uint8_t *w_layer;   /* record of expert e at w_layer + e * rec_bytes; the shared expert is index n_experts */
    uint64_t rec_bytes;
    uint64_t mat_off[2];      /* byte offsets inside a record of the matrices of this launch: {gate, up} or {down, -} */
    int M, K;                 /* rows and columns of each matrix */
    /* activations: fp16 rows in the K' order of the operand tiles (see batch.cu).
     * gate/up pass (exact): xh = the int8 Q8_K values as fp16 integers, xscale[row][K/256] = the blocks' d,
     *                       xbs[row][K/256][8] = the sums of the int8 values over each 32-wide sub-block;
     * down pass:            xh = q8 * d_block / d_max of the row, xscale[row] = d_max, xbs unused. */
    const uint16_t *xh;       /* [rows][K] */
    const float *xscale;
    const int16_t *xbs;
    int x_by_token;           /* 1: pair p reads row p / top_k (routed) or p - T top_k (shared); 0: row p */
    int top_k, n_tokens;
    /* work */
    const int *pairs;         /* expert-sorted pair ids */
    const kb_item_t *items;
    const int *n_items;       /* device word */
    float *out;               /* [pairs][M]: SwiGLU activations (two matrices) or down outputs (one) */
    int *status;
    /* optional profiling aid (NULL = off): block 0 adds the cycles its roles spent waiting, see batch.cu */
    unsigned long long *prof;
} kb_gemm_args_t;

/* M x K is this rank's shard: rows row0.. and 256-column blocks kb0.. of a matrix whose rows hold bpr_full blocks */
int kb_launch_gen(uint8_t *dst, uint64_t rec_bytes, int n_recs, uint64_t mat_off, int M, int K, uint64_t seed,
                  uint32_t layer, uint32_t matrix, int row0, int bpr_full, int kb0, void *stream);
int kb_launch_repack(uint8_t *dst, const uint8_t *src_ggml_full, int M, int K, int row0, int bpr_full, int kb0, void *stream);
int kb_launch_add(float *x, const float *y, uint64_t n, void *stream);
int kb_launch_export(uint8_t *dst_ggml, const uint8_t *src, int M, int K, void *stream);

/* x += resid (optional); h = rmsnorm(x) * normw (optional: else h = x); Q8_K of h per 256 (src/quant.c:343-375) written as
 * fp16 rows in K' order with one scale per row.  h_out (optional) receives h in fp32. */
int kb_launch_prologue(float *x, const float *resid, const float *normw, float rms_eps, int n_tokens, int n_embd,
                       float *h_out, uint16_t *xh, float *xscale, int16_t *xbs, void *stream);
/* the same quantiser on [rows][n] fp32 rows.  exact = 1: the form the gate/up pass reads (xbs must be given);
 * exact = 0: the form the down pass reads */
int kb_launch_quant(const float *src, int rows, int n, int exact, uint16_t *xh, float *xscale, int16_t *xbs, void *stream);
/* softmax over all experts, ordered top-k (value descending, lower index first), renormalised weights */
int kb_launch_route(const float *logits, int n_tokens, int n_experts, int top_k, int *ids, float *scores,
                    int *status, void *stream);
/* bucket the (token, slot) pairs by expert, append the shared expert's pairs, and list the work items */
int kb_launch_bucket(const int *ids, int n_tokens, int n_experts, int top_k, int has_shared, int m_tiles_gu,
                     int m_tiles_dn, int *counts, int *pairs, kb_item_t *items_gu, int *n_items_gu,
                     kb_item_t *items_dn, int *n_items_dn, void *stream);
/* gate + up + SwiGLU (exact integer products, scaled per 256-block) / down (one pass in fp16) */
int kb_launch_gateup(const kb_gemm_args_t *a, int grid, void *stream);
int kb_launch_down(const kb_gemm_args_t *a, int grid, void *stream);
/* out[t] = sum_s score[t][s] * dots[pair(t, s)] in slot order, shared expert added last; x += out when x != NULL */
int kb_launch_combine(const float *dots, const float *scores, int n_tokens, int n_embd, int top_k, int has_shared,
                      float *out, float *x, void *stream);
int kb_launch_gen_f32(float *dst, uint64_t n, uint64_t seed, uint32_t layer, uint32_t stream_id, float mean, float std,
                      void *stream);

#ifdef __cplusplus
}
#endif
#endif
