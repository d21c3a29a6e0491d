/*
 * batch_engine.c -- host side of the batched (many tokens per call) routed-expert FFN: owns the expert table in the
 * batched layout, the per-call work buffers and the launch sequence of batch.cu.  Plain C like the rest of the host
 * library; kernels are reached through batch_launch.h only.
 */
#include <cuda_runtime_api.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/fomoe_b200.h"
#include "batch_launch.h"
#include "launch.h"
#include "synth.h"

#define KB_STREAM_LOGITS 8u /* synthetic router logits: one stream per layer, element = token * n_experts + expert */

struct fomoe_b200_batch {
    fomoe_b200_batch_config_t cfg;
    int n_sm;
    cudaStream_t stream;
    cudaEvent_t ev0, ev1;
    int il, tp_rank, tp_size;  /* this rank's share of the intermediate dimension: rows of gate/up, columns of down */
    uint64_t mat_gu, mat_dn, rec_bytes, table_bytes; /* bytes of this rank's gate (or up) shard, down shard, record */
    uint64_t full_gu, full_dn;  /* the same for the whole matrices: a ggml record is 2 full_gu + full_dn */
    float *part;               /* [max_tokens][n_embd]: this rank's partial block output (tensor parallel only) */
    fomoe_b200_allreduce_fn allreduce;
    void *allreduce_user;
    uint8_t **table;       /* per layer: (n_experts + has_shared) records gate | up | down, batched layout */
    float **resid, **normw;
    float *logits;         /* [n_layers][max_tokens][n_experts] or NULL */
    /* work buffers for max_tokens tokens */
    float *x, *h, *lg, *scores, *act, *dots, *xs_h, *xs_a;
    int16_t *bs_h;
    uint16_t *xh_h, *xh_a;
    int *ids, *counts, *pairs, *n_items, *status;
    kb_item_t *items_gu, *items_dn;
    uint8_t *stage;
    unsigned long long *prof; /* wait-cycle counters of the GEMM kernels' block 0 while profiling, or NULL */
    uint64_t launches;
    char err[256];
};

static void berr(fomoe_b200_batch_t *b, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(b->err, sizeof(b->err), fmt, ap);
    va_end(ap);
    fprintf(stderr, "fomoe_b200 (batch): %s\n", b->err);
}

#define BCK(b, call)                                                                       \
    do {                                                                                   \
        cudaError_t e_ = (call);                                                           \
        if (e_ != cudaSuccess) {                                                           \
            berr((b), "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
            return -1;                                                                     \
        }                                                                                  \
    } while (0)

#define BCKL(b, call)                                                                      \
    do {                                                                                   \
        int e_ = (call);                                                                   \
        (b)->launches++;                                                                   \
        if (e_ != 0) {                                                                     \
            berr((b), "%s failed: %s (%s:%d)", #call, cudaGetErrorString((cudaError_t)e_), __FILE__, __LINE__); \
            return -1;                                                                     \
        }                                                                                  \
    } while (0)

void fomoe_b200_batch_destroy(fomoe_b200_batch_t *b) {
    if (!b) return;
    cudaSetDevice(b->cfg.device);
    if (b->stream) cudaStreamSynchronize(b->stream);
    for (int l = 0; l < b->cfg.n_layers; l++) {
        if (b->table) cudaFree(b->table[l]);
        if (b->resid) cudaFree(b->resid[l]);
        if (b->normw) cudaFree(b->normw[l]);
    }
    free(b->table); free(b->resid); free(b->normw);
    cudaFree(b->logits); cudaFree(b->x); cudaFree(b->h); cudaFree(b->lg); cudaFree(b->scores); cudaFree(b->act);
    cudaFree(b->dots); cudaFree(b->xs_h); cudaFree(b->xs_a); cudaFree(b->bs_h); cudaFree(b->xh_h); cudaFree(b->xh_a); cudaFree(b->ids);
    cudaFree(b->counts); cudaFree(b->pairs); cudaFree(b->n_items); cudaFree(b->status); cudaFree(b->items_gu);
    cudaFree(b->items_dn); cudaFree(b->stage); cudaFree(b->prof); cudaFree(b->part);
    if (b->ev0) cudaEventDestroy(b->ev0);
    if (b->ev1) cudaEventDestroy(b->ev1);
    if (b->stream) cudaStreamDestroy(b->stream);
    free(b);
}

static int balloc(fomoe_b200_batch_t *b, void **p, uint64_t bytes) {
    BCK(b, cudaMalloc(p, bytes ? bytes : 16));
    BCK(b, cudaMemset(*p, 0, bytes ? bytes : 16));
    return 0;
}

fomoe_b200_batch_t *fomoe_b200_batch_create(const fomoe_b200_batch_config_t *cfg) {
    int ndev = 0;
    if (!cfg) return NULL;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
        fprintf(stderr, "fomoe_b200 (batch): no CUDA device (this library has no CPU path)\n");
        return NULL;
    }
    fomoe_b200_batch_t *b = (fomoe_b200_batch_t *)calloc(1, sizeof(*b));
    if (!b) return NULL;
    b->cfg = *cfg;
    if (cfg->device < 0 || cfg->device >= ndev || cfg->n_layers < 1 || cfg->n_embd % 256 || cfg->n_embd < 256 ||
        cfg->n_embd > 8192 || cfg->n_embd % KB_TILE_M || cfg->n_inter % 256 || cfg->n_inter < 256 || cfg->n_inter > 8192 ||
        cfg->n_experts < 1 || cfg->n_experts > 512 || cfg->top_k < 1 || cfg->top_k > 16 || cfg->top_k > cfg->n_experts ||
        cfg->max_tokens < 1 || cfg->tp_size < 0 || cfg->tp_size > 8 || cfg->tp_rank < 0 ||
        cfg->tp_rank >= (cfg->tp_size ? cfg->tp_size : 1) || cfg->n_inter % (256 * (cfg->tp_size ? cfg->tp_size : 1))) {
        berr(b, "unsupported configuration");
        free(b);
        return NULL;
    }
    /* tensor parallel: rank r of N owns gate/up rows [r I/N, (r+1) I/N) and the same columns of down, whole 256-wide
     * activation windows, exactly as the decode path shards (src/tp.hip:85-124 sums the ranks' outputs) */
    b->tp_size = cfg->tp_size ? cfg->tp_size : 1;
    b->tp_rank = cfg->tp_rank;
    b->il = cfg->n_inter / b->tp_size;
    const int nl = cfg->n_layers, ne = cfg->n_embd, ni = b->il, T = cfg->max_tokens;
    const int nrec = cfg->n_experts + (cfg->has_shared ? 1 : 0);
    const uint64_t npairs = (uint64_t)T * cfg->top_k + (cfg->has_shared ? T : 0);
    b->mat_gu = (uint64_t)ni * (ne / 256) * 144;
    b->mat_dn = (uint64_t)ne * (ni / 256) * 144;
    b->rec_bytes = 2 * b->mat_gu + b->mat_dn;
    b->full_gu = b->mat_gu * (uint64_t)b->tp_size;
    b->full_dn = b->mat_dn * (uint64_t)b->tp_size;
    if (cudaSetDevice(cfg->device) != cudaSuccess) goto fail;
    {
        struct cudaDeviceProp prop;
        b->n_sm = cudaGetDeviceProperties(&prop, cfg->device) == cudaSuccess ? prop.multiProcessorCount : 148;
    }
    if (cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking) != cudaSuccess) goto fail;
    if (cudaEventCreate(&b->ev0) != cudaSuccess || cudaEventCreate(&b->ev1) != cudaSuccess) goto fail;
    b->table = (uint8_t **)calloc((size_t)nl, sizeof(void *));
    b->resid = (float **)calloc((size_t)nl, sizeof(void *));
    b->normw = (float **)calloc((size_t)nl, sizeof(void *));
    if (!b->table || !b->resid || !b->normw) goto fail;
    for (int l = 0; l < nl; l++) {
        if (cudaMalloc((void **)&b->table[l], b->rec_bytes * (uint64_t)nrec) != cudaSuccess) {
            berr(b, "cudaMalloc of %.2f GB for layer %d's experts failed", b->rec_bytes * (double)nrec / 1e9, l);
            goto fail;
        }
        b->table_bytes += b->rec_bytes * (uint64_t)nrec;
        if (balloc(b, (void **)&b->resid[l], sizeof(float) * ne) || balloc(b, (void **)&b->normw[l], sizeof(float) * ne)) goto fail;
    }
    /* worst case of work items: every expert holds at least one pair, plus the extra passes of crowded experts */
    const uint64_t max_chunks = (uint64_t)nrec + npairs / KB_TILE_N + 1, max_chunks_gu = (uint64_t)nrec + npairs / KB_GU_N + 1;
    if (balloc(b, (void **)&b->x, sizeof(float) * (uint64_t)T * ne) || balloc(b, (void **)&b->h, sizeof(float) * (uint64_t)T * ne) ||
        balloc(b, (void **)&b->lg, sizeof(float) * (uint64_t)T * cfg->n_experts) ||
        balloc(b, (void **)&b->scores, sizeof(float) * (uint64_t)T * cfg->top_k) ||
        balloc(b, (void **)&b->ids, sizeof(int) * (uint64_t)T * cfg->top_k) ||
        balloc(b, (void **)&b->act, sizeof(float) * npairs * ni) || balloc(b, (void **)&b->dots, sizeof(float) * npairs * ne) ||
        balloc(b, (void **)&b->xh_h, sizeof(uint16_t) * (uint64_t)T * ne) || balloc(b, (void **)&b->xs_h, sizeof(float) * (uint64_t)T * (ne / 256)) ||
        balloc(b, (void **)&b->bs_h, sizeof(int16_t) * (uint64_t)T * (ne / 256) * 8) ||
        balloc(b, (void **)&b->xh_a, sizeof(uint16_t) * npairs * ni) || balloc(b, (void **)&b->xs_a, sizeof(float) * npairs) ||
        balloc(b, (void **)&b->counts, sizeof(int) * (nrec + 1)) || balloc(b, (void **)&b->pairs, sizeof(int) * npairs) ||
        balloc(b, (void **)&b->n_items, sizeof(int) * 2) || balloc(b, (void **)&b->status, sizeof(int)) ||
        balloc(b, (void **)&b->items_gu, sizeof(kb_item_t) * max_chunks_gu * (ni / KB_TILE_M)) ||
        balloc(b, (void **)&b->items_dn, sizeof(kb_item_t) * max_chunks * (ne / KB_TILE_M)) ||
        balloc(b, (void **)&b->stage, 2 * b->full_gu + b->full_dn) ||
        (b->tp_size > 1 && balloc(b, (void **)&b->part, sizeof(float) * (uint64_t)T * ne)))
        goto fail;
    if (ni % KB_TILE_M) goto fail;
    return b;
fail:
    if (!b->err[0]) berr(b, "CUDA setup failed: %s", cudaGetErrorString(cudaGetLastError()));
    fomoe_b200_batch_destroy(b);
    return NULL;
}

const char *fomoe_b200_batch_last_error(fomoe_b200_batch_t *b) { return b ? b->err : "null context"; }
uint64_t fomoe_b200_batch_table_bytes(fomoe_b200_batch_t *b) { return b ? b->table_bytes : 0; }
uint64_t fomoe_b200_batch_kernel_launches(fomoe_b200_batch_t *b) { return b ? b->launches : 0; }

int fomoe_b200_batch_status(fomoe_b200_batch_t *b) {
    int st = -1;
    if (!b) return -1;
    cudaSetDevice(b->cfg.device);
    if (cudaStreamSynchronize(b->stream) != cudaSuccess) return -1;
    if (cudaMemcpy(&st, b->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (st) cudaMemset(b->status, 0, sizeof(int));
    return st;
}

int fomoe_b200_batch_generate(fomoe_b200_batch_t *b, uint64_t seed, int with_logits) {
    if (!b) return -1;
    BCK(b, cudaSetDevice(b->cfg.device));
    const fomoe_b200_batch_config_t *c = &b->cfg;
    const int nrec = c->n_experts + (c->has_shared ? 1 : 0);
    for (int l = 0; l < c->n_layers; l++) {
        const int row0 = b->tp_rank * b->il, kb0 = b->tp_rank * (b->il / 256);
        BCKL(b, kb_launch_gen(b->table[l], b->rec_bytes, nrec, 0, b->il, c->n_embd, seed, (uint32_t)l, FSYN_M_GATE, row0, c->n_embd / 256, 0, b->stream));
        BCKL(b, kb_launch_gen(b->table[l], b->rec_bytes, nrec, b->mat_gu, b->il, c->n_embd, seed, (uint32_t)l, FSYN_M_UP, row0, c->n_embd / 256, 0, b->stream));
        BCKL(b, kb_launch_gen(b->table[l], b->rec_bytes, nrec, 2 * b->mat_gu, c->n_embd, b->il, seed, (uint32_t)l, FSYN_M_DOWN, 0, c->n_inter / 256, kb0, b->stream));
        BCKL(b, kb_launch_gen_f32(b->resid[l], (uint64_t)c->n_embd, seed, (uint32_t)l, FSYN_M_RESID, 0.0f, FOMOE_RESID_STD, b->stream));
        BCKL(b, kb_launch_gen_f32(b->normw[l], (uint64_t)c->n_embd, seed, (uint32_t)l, FSYN_M_NORMW, FOMOE_NORMW_MEAN, FOMOE_NORMW_STD, b->stream));
    }
    if (with_logits) {
        const uint64_t per = (uint64_t)c->max_tokens * c->n_experts;
        if (!b->logits && balloc(b, (void **)&b->logits, sizeof(float) * per * c->n_layers)) return -1;
        for (int l = 0; l < c->n_layers; l++)
            BCKL(b, kb_launch_gen_f32(b->logits + per * l, per, seed, (uint32_t)l, KB_STREAM_LOGITS, 0.0f, 1.0f, b->stream));
    }
    BCK(b, cudaStreamSynchronize(b->stream));
    return 0;
}

int fomoe_b200_batch_upload(fomoe_b200_batch_t *b, int layer, int expert, const void *record) {
    if (!b || !record || layer < 0 || layer >= b->cfg.n_layers || expert < 0 ||
        expert >= b->cfg.n_experts + (b->cfg.has_shared ? 1 : 0))
        return -1;
    BCK(b, cudaSetDevice(b->cfg.device));
    uint8_t *dst = b->table[layer] + (uint64_t)expert * b->rec_bytes;
    /* the whole ggml record is staged; this rank's rows (gate, up) and column blocks (down) are cut out of it */
    const int row0 = b->tp_rank * b->il, kb0 = b->tp_rank * (b->il / 256);
    BCK(b, cudaMemcpyAsync(b->stage, record, 2 * b->full_gu + b->full_dn, cudaMemcpyDefault, b->stream));
    BCKL(b, kb_launch_repack(dst, b->stage, b->il, b->cfg.n_embd, row0, b->cfg.n_embd / 256, 0, b->stream));
    BCKL(b, kb_launch_repack(dst + b->mat_gu, b->stage + b->full_gu, b->il, b->cfg.n_embd, row0, b->cfg.n_embd / 256, 0, b->stream));
    BCKL(b, kb_launch_repack(dst + 2 * b->mat_gu, b->stage + 2 * b->full_gu, b->cfg.n_embd, b->il, 0, b->cfg.n_inter / 256, kb0, b->stream));
    BCK(b, cudaStreamSynchronize(b->stream));
    return 0;
}

int fomoe_b200_batch_export(fomoe_b200_batch_t *b, int layer, int expert, void *record_out) {
    if (!b || !record_out || layer < 0 || layer >= b->cfg.n_layers || expert < 0 ||
        expert >= b->cfg.n_experts + (b->cfg.has_shared ? 1 : 0))
        return -1;
    BCK(b, cudaSetDevice(b->cfg.device));
    const uint8_t *src = b->table[layer] + (uint64_t)expert * b->rec_bytes;
    BCKL(b, kb_launch_export(b->stage, src, b->il, b->cfg.n_embd, b->stream));
    BCKL(b, kb_launch_export(b->stage + b->mat_gu, src + b->mat_gu, b->il, b->cfg.n_embd, b->stream));
    BCKL(b, kb_launch_export(b->stage + 2 * b->mat_gu, src + 2 * b->mat_gu, b->cfg.n_embd, b->il, b->stream));
    BCK(b, cudaMemcpyAsync(record_out, b->stage, b->rec_bytes, cudaMemcpyDeviceToHost, b->stream));
    BCK(b, cudaStreamSynchronize(b->stream));
    return 0;
}

/* experts of one layer on the T hidden states already quantised in xh_h / xs_h, logits in `lg`: leaves the block
 * output in `out_dev` (may be NULL) and adds it to `x_dev` (may be NULL) */
static int enqueue_layer(fomoe_b200_batch_t *b, int layer, int T, const float *lg, float *out_dev, float *x_dev) {
    const fomoe_b200_batch_config_t *c = &b->cfg;
    const int m_gu = b->il / KB_TILE_M, m_dn = c->n_embd / KB_TILE_M;
    BCKL(b, kb_launch_route(lg, T, c->n_experts, c->top_k, b->ids, b->scores, b->status, b->stream));
    BCKL(b, kb_launch_bucket(b->ids, T, c->n_experts, c->top_k, c->has_shared, m_gu, m_dn, b->counts, b->pairs, b->items_gu,
                             b->n_items, b->items_dn, b->n_items + 1, b->stream));
    kb_gemm_args_t a;
    memset(&a, 0, sizeof(a));
    a.w_layer = b->table[layer];
    a.rec_bytes = b->rec_bytes;
    a.top_k = c->top_k;
    a.n_tokens = T;
    a.pairs = b->pairs;
    a.status = b->status;
    a.prof = b->prof;
    /* gate + up + SwiGLU */
    a.mat_off[0] = 0;
    a.mat_off[1] = b->mat_gu;
    a.M = b->il;
    a.K = c->n_embd;
    a.xh = b->xh_h;
    a.xscale = b->xs_h;
    a.xbs = b->bs_h;
    a.x_by_token = 1;
    a.items = b->items_gu;
    a.n_items = b->n_items;
    a.out = b->act;
    BCKL(b, kb_launch_gateup(&a, b->n_sm, b->stream));
    const int npairs = T * c->top_k + (c->has_shared ? T : 0);
    BCKL(b, kb_launch_quant(b->act, npairs, b->il, 0, b->xh_a, b->xs_a, NULL, b->stream));
    /* down */
    a.mat_off[0] = 2 * b->mat_gu;
    a.mat_off[1] = 0;
    a.M = c->n_embd;
    a.K = b->il;
    a.xh = b->xh_a;
    a.xscale = b->xs_a;
    a.xbs = NULL;
    a.x_by_token = 0;
    a.items = b->items_dn;
    a.n_items = b->n_items + 1;
    a.out = b->dots;
    BCKL(b, kb_launch_down(&a, b->n_sm, b->stream));
    if (b->tp_size == 1) {
        BCKL(b, kb_launch_combine(b->dots, b->scores, T, c->n_embd, c->top_k, c->has_shared, out_dev, x_dev, b->stream));
        return 0;
    }
    /* tensor parallel: this rank's partial block output, summed over the ranks by the caller's collective (in place,
     * on this stream), then handed on.  Without a collective installed the partial itself is the result. */
    BCKL(b, kb_launch_combine(b->dots, b->scores, T, c->n_embd, c->top_k, c->has_shared, b->part, NULL, b->stream));
    const uint64_t n = (uint64_t)T * c->n_embd;
    if (b->allreduce && b->allreduce(b->allreduce_user, b->part, (int)n, (void *)b->stream)) {
        berr(b, "the caller's all-reduce reported a failure at layer %d", layer);
        return -1;
    }
    if (out_dev) BCK(b, cudaMemcpyAsync(out_dev, b->part, sizeof(float) * n, cudaMemcpyDeviceToDevice, b->stream));
    if (x_dev) BCKL(b, kb_launch_add(x_dev, b->part, n, b->stream));
    return 0;
}

int fomoe_b200_batch_set_allreduce(fomoe_b200_batch_t *b, fomoe_b200_allreduce_fn fn, void *user) {
    if (!b) return -1;
    b->allreduce = fn;
    b->allreduce_user = user;
    return 0;
}

int fomoe_b200_batch_moe_layer(fomoe_b200_batch_t *b, int layer, int n_tokens, const float *h, const float *logits, float *out,
                               int *ids_out, float *scores_out) {
    if (!b || !h || !logits || !out || layer < 0 || layer >= b->cfg.n_layers || n_tokens < 1 || n_tokens > b->cfg.max_tokens)
        return -1;
    const fomoe_b200_batch_config_t *c = &b->cfg;
    BCK(b, cudaSetDevice(c->device));
    const size_t nb = sizeof(float) * (size_t)n_tokens * c->n_embd;
    BCK(b, cudaMemcpyAsync(b->h, h, nb, cudaMemcpyHostToDevice, b->stream));
    BCK(b, cudaMemcpyAsync(b->lg, logits, sizeof(float) * (size_t)n_tokens * c->n_experts, cudaMemcpyHostToDevice, b->stream));
    BCKL(b, kb_launch_quant(b->h, n_tokens, c->n_embd, 1, b->xh_h, b->xs_h, b->bs_h, b->stream));
    if (enqueue_layer(b, layer, n_tokens, b->lg, b->x, NULL)) return -1;
    BCK(b, cudaMemcpyAsync(out, b->x, nb, cudaMemcpyDeviceToHost, b->stream));
    if (ids_out)
        BCK(b, cudaMemcpyAsync(ids_out, b->ids, sizeof(int) * (size_t)n_tokens * c->top_k, cudaMemcpyDeviceToHost, b->stream));
    if (scores_out)
        BCK(b, cudaMemcpyAsync(scores_out, b->scores, sizeof(float) * (size_t)n_tokens * c->top_k, cudaMemcpyDeviceToHost, b->stream));
    BCK(b, cudaStreamSynchronize(b->stream));
    return 0;
}

int fomoe_b200_batch_tokens_upload(fomoe_b200_batch_t *b, int n_tokens, const float *x) {
    if (!b || !x || n_tokens < 1 || n_tokens > b->cfg.max_tokens) return -1;
    BCK(b, cudaSetDevice(b->cfg.device));
    BCK(b, cudaMemcpyAsync(b->x, x, sizeof(float) * (size_t)n_tokens * b->cfg.n_embd, cudaMemcpyHostToDevice, b->stream));
    BCK(b, cudaStreamSynchronize(b->stream));
    return 0;
}

int fomoe_b200_batch_tokens_download(fomoe_b200_batch_t *b, int n_tokens, float *x_out) {
    if (!b || !x_out || n_tokens < 1 || n_tokens > b->cfg.max_tokens) return -1;
    BCK(b, cudaSetDevice(b->cfg.device));
    BCK(b, cudaMemcpyAsync(x_out, b->x, sizeof(float) * (size_t)n_tokens * b->cfg.n_embd, cudaMemcpyDeviceToHost, b->stream));
    BCK(b, cudaStreamSynchronize(b->stream));
    return 0;
}

int fomoe_b200_batch_stack_run(fomoe_b200_batch_t *b, int n_tokens, int l0, int l1, float *elapsed_ms) {
    if (!b || n_tokens < 1 || n_tokens > b->cfg.max_tokens || l0 < 0 || l1 > b->cfg.n_layers || l0 >= l1) return -1;
    if (!b->logits) {
        berr(b, "stack_run needs the synthetic router logits (generate with with_logits = 1)");
        return -1;
    }
    const fomoe_b200_batch_config_t *c = &b->cfg;
    BCK(b, cudaSetDevice(c->device));
    BCK(b, cudaEventRecord(b->ev0, b->stream));
    for (int l = l0; l < l1; l++) {
        BCKL(b, kb_launch_prologue(b->x, b->resid[l], b->normw[l], c->rms_eps, n_tokens, c->n_embd, NULL, b->xh_h, b->xs_h, b->bs_h, b->stream));
        if (enqueue_layer(b, l, n_tokens, b->logits + (uint64_t)l * c->max_tokens * c->n_experts, NULL, b->x)) return -1;
    }
    BCK(b, cudaEventRecord(b->ev1, b->stream));
    BCK(b, cudaStreamSynchronize(b->stream));
    if (elapsed_ms) BCK(b, cudaEventElapsedTime(elapsed_ms, b->ev0, b->ev1));
    return 0;
}

int fomoe_b200_batch_get_routing(fomoe_b200_batch_t *b, int n_tokens, int *ids, float *scores, int *counts) {
    if (!b || n_tokens < 1 || n_tokens > b->cfg.max_tokens) return -1;
    BCK(b, cudaSetDevice(b->cfg.device));
    BCK(b, cudaStreamSynchronize(b->stream));
    if (ids) BCK(b, cudaMemcpy(ids, b->ids, sizeof(int) * (size_t)n_tokens * b->cfg.top_k, cudaMemcpyDeviceToHost));
    if (scores) BCK(b, cudaMemcpy(scores, b->scores, sizeof(float) * (size_t)n_tokens * b->cfg.top_k, cudaMemcpyDeviceToHost));
    if (counts)
        BCK(b, cudaMemcpy(counts, b->counts, sizeof(int) * (size_t)(b->cfg.n_experts + (b->cfg.has_shared ? 1 : 0)), cudaMemcpyDeviceToHost));
    return 0;
}

/* Profiling aid: on = 1 starts counting the cycles block 0 of the two GEMM kernels spends waiting, per role (out[0..7]
 * down pass, out[8..15] gate/up pass; see batch.cu for the slots); on = 0 reads the counters into out[16] and stops. */
int fomoe_b200_batch_wait_profile(fomoe_b200_batch_t *b, int on, unsigned long long *out) {
    if (!b) return -1;
    BCK(b, cudaSetDevice(b->cfg.device));
    BCK(b, cudaStreamSynchronize(b->stream));
    if (on) {
        if (!b->prof && balloc(b, (void **)&b->prof, sizeof(unsigned long long) * 16)) return -1;
        BCK(b, cudaMemset(b->prof, 0, sizeof(unsigned long long) * 16));
        return 0;
    }
    if (!b->prof || !out) return -1;
    BCK(b, cudaMemcpy(out, b->prof, sizeof(unsigned long long) * 16, cudaMemcpyDeviceToHost));
    cudaFree(b->prof);
    b->prof = NULL;
    return 0;
}

/* host copy of the synthetic router logits of one layer: [n_tokens][n_experts] */
void fomoe_b200_batch_synth_logits(uint64_t seed, int layer, int max_tokens, int n_experts, int n_tokens, float *out) {
    const uint64_t key = fsyn_key(seed, (uint32_t)layer, 0, KB_STREAM_LOGITS);
    (void)max_tokens;
    for (uint64_t i = 0; i < (uint64_t)n_tokens * n_experts; i++) out[i] = fsyn_f32(key, i, 0.0f, 1.0f);
}
