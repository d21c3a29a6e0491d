/*
 * launch.h -- the thin C-ABI between the C host library and the CUDA kernels.
 *
 * Everything here is plain C: device pointers travel as ordinary pointers, streams as
 * void*.  The host side (engine.c) owns all memory and ordering; the functions below
 * only enqueue kernels on the given stream and return the CUDA error code (0 = ok).
 */
#ifndef FOMOE_B200_LAUNCH_H
#define FOMOE_B200_LAUNCH_H

#include <stdint.h>

#include "layout.h"

#ifdef __cplusplus
extern "C" {
#endif

/* One quantised activation block as the kernels consume it (304 B, 16-byte aligned):
 * the reference's block_q8_K (include/quant.h:94-98) re-ordered so the 256 int8 values
 * come first.  19 uint4 per entry keeps 8 consecutive entries on distinct shared-memory
 * bank groups. */
typedef struct {
    int8_t qs[256];
    int16_t bsums[16];
    float d;
    uint32_t pad[3];
} __attribute__((aligned(16))) fb_q8_entry_t;

/* status word values written by kernels (0 = ok) */
#define FB_ST_OK 0
#define FB_ST_BAD_ID 1      /* router produced an expert id outside the table */
#define FB_ST_WAIT_TIMEOUT 2 /* a bounded wait ran out */

#define FB_MAX_TP 8 /* tensor-parallel ranks */

/* Routing decision of one layer-token as the kernels log it (when a log is attached): the top-k before cache-aware
 * routing with its renormalised weights, and what was used.  The host turns these into the reference's routing-trace
 * records (src/gpu_kernels.hip:451-484). */
typedef struct {
    int ids_orig[16];
    float scores_orig[16];
    int ids[16];
    float scores[16];
} fb_route_rec_t;

/* Argument block passed by value to every hot-path kernel. */
typedef struct {
    /* shapes */
    int n_embd, n_inter, inter_local, n_experts, top_k, n_slots, has_shared;
    int tp_rank, tp_size;
    int gate_bpr, down_bpr;       /* 256-column blocks per row in this rank's gate/up and down shards */
    int gate_type;                /* FB_TYPE_Q4_K, or FB_TYPE_Q6_K (per-phase kernels with plain loads only) */
    int gate_groups, down_groups; /* 32-block groups per shard */
    uint64_t up_off, down_off;    /* byte offsets of the up and down shards inside an expert record */
    float rms_eps, car_threshold;
    int car_dampen;
    /* this layer */
    const uint8_t *table_layer; /* record of expert e at table_layer + e * rec_bytes; shared expert = index n_experts */
    uint64_t rec_bytes;
    int down_type;
    int down_half;            /* -1: the down shard holds whole super-blocks; 0 / 1: that half of every super-block */
    const float *router_w;    /* [n_experts][n_embd] */
    const float *resid;       /* [n_embd] or NULL */
    const float *normw;       /* [n_embd] or NULL */
    const float *shared_gate_w; /* [n_embd] or NULL: the shared expert's output is scaled by sigmoid(h . w) */
    float *shared_gate;         /* that scalar, written by the prologue kernel (per-phase path) */
    const uint32_t *resident; /* [16] residency bit mask or NULL */
    uint32_t *freq;           /* [n_experts] selection histogram for this layer or NULL */
    /* state */
    float *x;       /* residual stream [n_embd] */
    float *h;       /* normalised hidden state [n_embd] */
    float *moe_out; /* MoE block output (this rank's partial under TP) [n_embd] */
    fb_q8_entry_t *q8h; /* [n_embd/256] */
    float *logits;      /* [n_experts] */
    float *all_scores;  /* [n_experts] softmax over all experts */
    int *ids;           /* [n_slots] selected expert ids (slot top_k = shared) */
    int *ids_orig;      /* [top_k] ids before CAR */
    float *scores;      /* [n_slots] routing weights */
    const uint8_t **slot_rec; /* [n_slots] record pointers */
    float *act;         /* [n_slots][inter_local] silu(gate)*up */
    fb_q8_entry_t *q8a; /* [n_slots][inter_local/256] */
    float *dots;        /* [n_slots][n_embd] per-expert down outputs */
    unsigned *counters; /* arrival counters: [0] router, [1] substitutions, then windows, then row groups */
    int *status;
    int accumulate;        /* 1: the combine adds onto moe_out instead of overwriting it */
    const float *tok_in;   /* device-resident token inputs [max_tokens][n_embd] */
    float *tok_out;        /* device-resident token outputs */
    unsigned *tok_ctr;     /* index of the token in flight */
    fb_route_rec_t *route_log; /* NULL, or this layer's record of token 0; token t's lies route_stride records on */
    int route_stride;
} fb_args_t;

#define FB_CNT_ROUTER 0
#define FB_CNT_SUBS 1
#define FB_CNT_WIN 8 /* first window counter; n_slots * (inter_local/256) of them, row groups follow */

/* prologue flags */
#define FB_PRO_ADD_PREV 1 /* x += moe_out */
#define FB_PRO_RESID 2    /* x += resid */
#define FB_PRO_NORM 4     /* h = rmsnorm(x) * normw (else h = x) */
#define FB_PRO_QUANT 8    /* q8h = Q8_K(h) */
#define FB_PRO_LOAD 16    /* x = tok_in[*tok_ctr] first */
#define FB_PRO_STORE 32   /* tok_out[*tok_ctr] = x at the end, then ++*tok_ctr */

int fb_launch_prologue(const fb_args_t *a, int flags, void *stream);
int fb_launch_router(const fb_args_t *a, int grid, void *stream);
/* route from host-provided ids/scores already in a->ids / a->scores: only fills slot_rec */
int fb_launch_set_slots(const fb_args_t *a, void *stream);
int fb_launch_gate_up(const fb_args_t *a, int grid, void *stream);
int fb_launch_down(const fb_args_t *a, int grid, void *stream);
/* the same two phases with fp32 activations (kernels_f32.cu) */
int fb_launch_gate_up_f32(const fb_args_t *a, int grid, void *stream);
int fb_launch_down_f32(const fb_args_t *a, int grid, void *stream);
/* same phases with weights streamed by bulk copies into per-warp shared-memory rings */
int fb_launch_gate_up_ring(const fb_args_t *a, int grid, void *stream);
int fb_launch_down_ring(const fb_args_t *a, int grid, void *stream);

/* ---- the persistent stack kernel: all layers of `tok_count` tokens in one launch ---- */
typedef struct {
    const fb_args_t *layers; /* device array, one entry per layer of the range to run */
    int n_layers;
    int down_mode;           /* down formats among the layers: 0 whole Q4_K/Q6_K, 1 whole incl. Q5_K, 2 half super-blocks */
    int tok_count;           /* tokens tok_first .. tok_first + tok_count - 1 */
    int tok_first;
    const float *tok_in;
    float *tok_out;
    float *out_host;         /* NULL, or mapped host memory that receives the LAST token's output instead of tok_out */
    unsigned *tok_ctr;       /* left at tok_first + tok_count for the per-phase path */
    unsigned long long *bar; /* grid barrier: [0] arrival counter, [16] generation of the last completed barrier */
    unsigned long long bar_base; /* arrivals before this launch (the host keeps count) */
    unsigned long long *ll_dots; /* [FB_MAX_SLOTS][n_embd] {generation, value} words: row groups split between blocks */
    unsigned long long *ll_logits; /* [FB_MAX_EXPERTS] {generation, value} words: the router logits of the layer-token in flight */
    unsigned gen_base;       /* layer-tokens run by earlier launches */
    unsigned spin_limit;     /* polls after which a wait on another block or rank is given up */
    int *abort_flag;         /* raised by a block that gave up a wait; cleared by the host before a launch */
    int *status;
    /* tensor parallelism: the combine step stores this rank's partial block output into slot tp_rank of every
     * rank's receive buffer ({generation, value} words, double-buffered by generation parity so that a fast rank can
     * never overwrite words a slow block of a peer still has to read); tp_peer[p] is rank p's buffer as mapped into
     * this process (tp_peer[tp_rank] == tp_recv, this GPU's own) */
    int tp_rank, tp_size;
    unsigned long long *tp_recv;     /* [2][tp_size][n_embd]: words of generation g lie in half g & 1 */
    unsigned long long *tp_peer[FB_MAX_TP];
    unsigned long long *tp_xsum;     /* [n_embd] {generation, value}: the rank-ordered sum, formed once per GPU */
    int tp_two_stage;                /* 1: a few warps add the ranks' partials up and publish the sum in tp_xsum,
                                        everyone else reads that; 0: every thread polls every rank's slot itself */
    int *host_flags;                 /* mapped host memory: [0] receives the status code of a block that gave up */
    unsigned long long *trace; /* optional phase stamps of one block (profiling), or NULL */
    int trace_cap, trace_cta;
} fb_stack_args_t;

int fb_stack_smem_bytes(void);
int fb_stack_supported(const fb_args_t *a, int grid);
int fb_launch_stack(const fb_stack_args_t *k, int grid, void *stream);

/* ---- table construction ---- */
typedef struct {
    int type;
    int rows_local, bpr_local; /* shard geometry */
    int row0, b0, bpr_full;    /* position of the shard inside the full matrix */
    int half;                  /* -1 whole super-blocks; 0 / 1: the shard holds that half of each of its blocks */
} fb_shard_geom_t;

/* generate expert `e`'s matrix stream (seed, layer, e, matrix) for e in [0, n_recs) straight into
 * the device layout; dst0 = first record's shard, rec_stride between experts */
int fb_launch_gen_shards(uint8_t *dst0, uint64_t rec_stride, int n_recs, uint64_t seed, uint32_t layer,
                         uint32_t matrix, fb_shard_geom_t g, void *stream);
int fb_launch_gen_f32(float *dst, uint64_t n, uint64_t seed, uint32_t layer, uint32_t stream_id, float mean,
                      float std, void *stream);
/* ggml-ordered bytes of the full matrix (device memory) -> this rank's shard */
int fb_launch_repack(uint8_t *dst, const uint8_t *src_ggml, fb_shard_geom_t g, void *stream);
/* shard -> ggml-ordered bytes of the shard's blocks, row-major (rows_local x bpr_local blocks) */
int fb_launch_export_ggml(uint8_t *dst_ggml, const uint8_t *shard, fb_shard_geom_t g, void *stream);
/* shard -> fp32 [rows_local][bpr_local*256] */
int fb_launch_dequant(float *dst, const uint8_t *shard, fb_shard_geom_t g, void *stream);

/* standalone matvec (microbenchmark / parity): out[rows_local] = shard . q8 (bpr_local entries) */
int fb_launch_matvec(float *out, const uint8_t *shard, fb_shard_geom_t g, const fb_q8_entry_t *q8, int grid,
                     void *stream);
int fb_launch_quantize(fb_q8_entry_t *dst, const float *src, int n_blocks, void *stream);
/* projections in 32-value blocks (Q8_0, MXFP4) on fp32 activations, weights in ggml order: proj32.cu */
int fb_launch_p32_matvec(int type, const uint8_t *w, int rows, int cols, const float *x, float *y, void *stream);
int fb_launch_p32_gate_up(int gate_type, const uint8_t *gate, int up_type, const uint8_t *up, int inter, int n_embd,
                          const float *h, float *act, void *stream);

#ifdef __cplusplus
}
#endif
#endif
