/*
 * engine.c -- host side of libfomoe_b200.so, in C like the reference's host code.
 *
 * Owns the CUDA context objects, the HBM-resident expert table and the per-token launch
 * sequence; calls the kernels only through the thin C-ABI of launch.h.  The reference
 * keeps experts in a VRAM LRU backed by pinned DRAM and NVMe (src/expert_cache.c,
 * src/expert_store.c, src/nvme_io.c) and returns to the host after the router of every
 * layer to classify and run car_evaluate (src/gpu_kernels.hip:6984, 7097-7187); here the
 * whole table is resident and routing stays on the device, so a token is one CUDA graph.
 */
#define _POSIX_C_SOURCE 200809L /* fseeko */
#define _FILE_OFFSET_BITS 64
#include <cuda_runtime_api.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/types.h>

#include "../../include/fomoe_b200.h"
#include "launch.h"
#include "synth.h"

#define FB_N_SM_DEFAULT 148

typedef struct {
    uint8_t *table;      /* (n_experts + has_shared) records of rec_bytes */
    uint64_t rec_bytes;  /* this rank's bytes per record in the device layout */
    uint64_t down_bytes;
    int down_type;
    float *router_w, *resid, *normw;
    uint32_t *mask; /* device copy of the residency mask */
    uint32_t mask_host[16];
    int mask_set;
    float *shared_gate_w; /* [n_embd] or NULL */
} fb_layer_t;

struct fomoe_b200_ctx {
    fomoe_b200_config_t cfg;
    int *down_types;
    int n_sm;
    cudaStream_t stream;
    cudaEvent_t ev0, ev1;
    fb_layer_t *layers;
    uint64_t table_bytes;
    /* geometry */
    int inter_local, gate_bpr, down_bpr, gate_groups, down_groups, n_slots;
    int gate_part;  /* which inter_local-row slice of gate/up this rank computes */
    int down_half;  /* -1, or which half of every down super-block this rank owns (twice as many ranks as windows) */
    uint64_t gate_bytes; /* bytes of one gate (or up) shard */
    /* state */
    float *x, *h, *moe_out, *logits, *all_scores, *scores, *act, *dots;
    int *ids, *ids_orig, *status;
    const uint8_t **slot_rec;
    fb_q8_entry_t *q8h, *q8a;
    unsigned *counters, *tok_ctr;
    float *shared_gate; /* scalar gate of the shared expert for the layer in flight */
    uint32_t *freq; /* [n_layers][n_experts] or NULL */
    float *tok_in, *tok_out;
    int max_tokens;
    /* staging */
    uint8_t *stage;       /* device staging for uploads / exports */
    uint64_t stage_bytes;
    /* record uploads of the operator surfaces: two staging buffers filled on a copy stream, so that the host never
     * waits between records and the copy of one record overlaps the regrouping of the one before */
    uint8_t *stage2;
    cudaStream_t copy_stream;
    cudaEvent_t ev_full[2], ev_free[2];
    int serial_upload;    /* 1: one record at a time with a synchronise after each (comparison arm) */
    float *pin;           /* pinned host scratch, 4 * n_embd floats + routing scratch (mapped into the device) */
    float *pin_dev;       /* the same memory as the device sees it */
    /* graphs */
    int use_graphs;
    fomoe_b200_allreduce_fn allreduce; /* caller's collective for the per-phase tensor-parallel path, or NULL */
    void *allreduce_user;
    cudaGraphExec_t graph_exec;
    int graph_nodes;
    uint64_t launches;
    int pin_busy; /* an un-synchronised call may still be reading the pinned scratch */
    /* per-kernel event timing (tokens_profile) */
    cudaEvent_t *pev;
    int *pev_phase;
    int pev_cap, pev_n, profiling;
    int variant; /* 0: per-phase kernels, plain loads; 1: per-phase kernels, bulk-copy rings; 2 (default): the
                    persistent stack kernel for whole-token runs, per-phase kernels (plain) elsewhere.
                    Environment override: FOMOE_B200_VARIANT */
    fb_args_t *d_layer_args; /* device copy of every layer's arguments for the stack kernel */
    int layer_args_valid;
    unsigned long long *d_trace, *d_ll_dots, *d_ll_logits;
    /* tensor parallelism: this rank's receive buffer and every rank's buffer as mapped here */
    unsigned long long *tp_recv, *tp_peer[FB_MAX_TP], *tp_xsum;
    int tp_connected, tp_two_stage;
    int *host_flags;      /* in the mapped pinned block: [0] = code of a stack launch that gave a wait up */
    int last_status;      /* what fomoe_b200_status reports next: the code of the most recent failed run */
    fb_route_rec_t *route_log; /* [max_tokens + 1][n_layers] routing decisions, or NULL */
    FILE *trace_fp;            /* routing-trace file being written, or NULL */
    uint32_t trace_tokens;     /* tokens written to it so far */
    unsigned long long *d_bar;     /* grid barrier words */
    unsigned long long bar_count;  /* arrivals all finished stack launches have added */
    unsigned gen_count;            /* layer-tokens of all finished stack launches */
    int trace_cap, trace_cta;
    int *d_abort;
    unsigned spin_limit; /* polls after which the stack kernel gives a wait up */
    int act_f32;         /* 1: experts run with fp32 activations (the reference's second definition) */
    char err[256];
};

static void set_err(fomoe_b200_ctx_t *c, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(c->err, sizeof(c->err), fmt, ap);
    va_end(ap);
    fprintf(stderr, "fomoe_b200: %s\n", c->err);
}

#define CK(c, call)                                                                      \
    do {                                                                                 \
        cudaError_t e_ = (call);                                                         \
        if (e_ != cudaSuccess) {                                                         \
            set_err((c), "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
            return -1;                                                                   \
        }                                                                                \
    } while (0)

#define CKL(c, call)                                                                     \
    do {                                                                                 \
        int e_;                                                                          \
        if ((c)->profiling) prof_mark((c), #call);                                       \
        e_ = (call);                                                                     \
        (c)->launches++;                                                                 \
        if (e_ != 0) {                                                                   \
            set_err((c), "%s failed: %s (%s:%d)", #call, cudaGetErrorString((cudaError_t)e_), __FILE__, __LINE__); \
            return -1;                                                                   \
        }                                                                                \
    } while (0)

static void prof_mark(struct fomoe_b200_ctx *c, const char *call);

static int is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

static uint64_t ggml_matrix_bytes(int type, int rows, int cols) {
    return (uint64_t)rows * (uint64_t)(cols / FB_QK) * fb_block_bytes(type);
}

static fb_shard_geom_t geom_gate(const fomoe_b200_ctx_t *c) {
    fb_shard_geom_t g;
    g.type = c->cfg.gate_type;
    g.rows_local = c->inter_local;
    g.bpr_local = g.bpr_full = c->gate_bpr;
    g.row0 = c->gate_part * c->inter_local;
    g.b0 = 0;
    g.half = -1;
    return g;
}

static fb_shard_geom_t geom_down(const fomoe_b200_ctx_t *c, int type) {
    fb_shard_geom_t g;
    g.type = type;
    g.rows_local = c->cfg.n_embd;
    g.bpr_local = c->down_bpr;
    g.bpr_full = c->cfg.n_inter / FB_QK;
    g.row0 = 0;
    g.b0 = c->gate_part * c->down_bpr;
    g.half = c->down_half;
    return g;
}

static void drop_graph(fomoe_b200_ctx_t *c) {
    c->layer_args_valid = 0;
    if (c->graph_exec) {
        cudaGraphExecDestroy(c->graph_exec);
        c->graph_exec = NULL;
    }
}

/* ------------------------------------------------------------------ create / destroy */
void fomoe_b200_destroy(fomoe_b200_ctx_t *c) {
    if (!c) return;
    cudaSetDevice(c->cfg.device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    drop_graph(c);
    if (c->layers) {
        for (int l = 0; l < c->cfg.n_layers; l++) {
            cudaFree(c->layers[l].table);
            cudaFree(c->layers[l].router_w);
            cudaFree(c->layers[l].resid);
            cudaFree(c->layers[l].normw);
            cudaFree(c->layers[l].mask);
            cudaFree(c->layers[l].shared_gate_w);
        }
        free(c->layers);
    }
    cudaFree(c->x); cudaFree(c->h); cudaFree(c->moe_out); cudaFree(c->logits); cudaFree(c->all_scores);
    cudaFree(c->scores); cudaFree(c->act); cudaFree(c->dots); cudaFree(c->ids); cudaFree(c->ids_orig);
    cudaFree(c->status); cudaFree((void *)c->slot_rec); cudaFree(c->q8h); cudaFree(c->q8a);
    cudaFree(c->counters); cudaFree(c->tok_ctr); cudaFree(c->shared_gate); cudaFree(c->freq); cudaFree(c->tok_in); cudaFree(c->tok_out);
    for (int p = 0; p < FB_MAX_TP; p++)
        if (c->tp_connected == 1 && c->tp_peer[p] && c->tp_peer[p] != c->tp_recv) cudaIpcCloseMemHandle(c->tp_peer[p]);
    cudaFree(c->tp_recv);
    cudaFree(c->tp_xsum);
    cudaFree(c->route_log);
    if (c->trace_fp) fclose(c->trace_fp);
    cudaFree(c->stage2);
    for (int i = 0; i < 2; i++) {
        if (c->ev_full[i]) cudaEventDestroy(c->ev_full[i]);
        if (c->ev_free[i]) cudaEventDestroy(c->ev_free[i]);
    }
    if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
    cudaFree(c->d_trace); cudaFree(c->stage); cudaFree(c->d_layer_args); cudaFree(c->d_bar); cudaFree(c->d_ll_dots); cudaFree(c->d_ll_logits); cudaFree(c->d_abort);
    if (c->pin) cudaFreeHost(c->pin);
    for (int i = 0; i < c->pev_cap; i++) cudaEventDestroy(c->pev[i]);
    free(c->pev);
    free(c->pev_phase);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    if (c->stream) cudaStreamDestroy(c->stream);
    free(c->down_types);
    free(c);
}

static int dev_alloc(fomoe_b200_ctx_t *c, void **p, uint64_t bytes) {
    CK(c, cudaMalloc(p, bytes ? bytes : 16));
    CK(c, cudaMemset(*p, 0, bytes ? bytes : 16));
    return 0;
}

fomoe_b200_ctx_t *fomoe_b200_create(const fomoe_b200_config_t *cfg) {
    if (!cfg) return NULL;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
        fprintf(stderr, "fomoe_b200: no CUDA device (this library has no CPU path)\n");
        return NULL;
    }
    fomoe_b200_ctx_t *c = (fomoe_b200_ctx_t *)calloc(1, sizeof(*c));
    if (!c) return NULL;
    c->cfg = *cfg;
    c->use_graphs = 1;
    c->spin_limit = 1u << 22; /* seconds: far beyond any legitimate wait, still bounded */
    c->variant = getenv("FOMOE_B200_VARIANT") ? atoi(getenv("FOMOE_B200_VARIANT")) : 2;
    const int N = cfg->tp_size > 0 ? cfg->tp_size : 1;
    c->cfg.tp_size = N;
    if (cfg->device < 0 || cfg->device >= ndev || cfg->n_layers < 1 || cfg->n_embd % FB_QK || cfg->n_embd > 8192 ||
        cfg->n_embd < FB_QK || cfg->n_inter % FB_QK || cfg->n_inter < FB_QK || N > FB_MAX_TP || cfg->n_experts < 1 ||
        cfg->n_experts > FB_MAX_EXPERTS || cfg->top_k < 1 || cfg->top_k > FB_MAX_TOPK || cfg->top_k > cfg->n_experts ||
        (cfg->gate_type != FB_TYPE_Q4_K && cfg->gate_type != FB_TYPE_Q6_K) || cfg->tp_rank < 0 || cfg->tp_rank >= N) {
        set_err(c, "unsupported configuration");
        free(c);
        return NULL;
    }
    /* Shards: N ranks over W = n_inter/256 activation windows.  N divides W: rank r owns W/N whole windows (gate/up
     * rows and down column blocks).  N == 2 W: the ranks 2p and 2p+1 share window p -- both compute its 256 gate/up
     * rows (quantising a window needs the maximum over all 256 values, src/quant.c:343-375, and recomputing the
     * partner's 128 rows is cheaper than exchanging maxima between GPUs in the middle of a layer) and each owns
     * one 128-column half of the down super-blocks of that window. */
    {
        const int W = cfg->n_inter / FB_QK;
        if (N <= W && W % N == 0) {
            c->inter_local = cfg->n_inter / N;
            c->gate_part = cfg->tp_rank;
            c->down_half = -1;
        } else if (N == 2 * W) {
            c->inter_local = FB_QK;
            c->gate_part = cfg->tp_rank >> 1;
            c->down_half = cfg->tp_rank & 1;
        } else {
            set_err(c, "tp_size %d does not divide the %d activation windows of n_inter %d (nor is it twice their number)", N,
                    W, cfg->n_inter);
            free(c);
            return NULL;
        }
    }
    c->gate_bpr = cfg->n_embd / FB_QK;
    c->down_bpr = c->inter_local / FB_QK;
    if (!is_pow2(c->gate_bpr) || !is_pow2(c->down_bpr) || c->gate_bpr > 32 || c->down_bpr > 32 ||
        c->inter_local / FB_QK > 32) {
        set_err(c, "blocks per row must be a power of two <= 32 (n_embd %d, local intermediate %d)", cfg->n_embd,
                c->inter_local);
        free(c);
        return NULL;
    }
    c->n_slots = cfg->top_k + (cfg->has_shared ? 1 : 0);
    c->gate_groups = (int)fb_n_groups((uint64_t)c->inter_local * c->gate_bpr);
    c->down_groups = (int)fb_n_groups((uint64_t)cfg->n_embd * c->down_bpr);
    c->gate_bytes = fb_shard_bytes(cfg->gate_type, (uint64_t)c->inter_local * c->gate_bpr);
    c->max_tokens = cfg->max_tokens > 0 ? cfg->max_tokens : 1;
    c->down_types = (int *)malloc(sizeof(int) * (size_t)cfg->n_layers);
    for (int l = 0; l < cfg->n_layers; l++) {
        c->down_types[l] = cfg->down_types ? cfg->down_types[l] : FB_TYPE_Q6_K;
        if (c->down_types[l] != FB_TYPE_Q4_K && c->down_types[l] != FB_TYPE_Q5_K && c->down_types[l] != FB_TYPE_Q6_K) {
            set_err(c, "layer %d: down type %d unsupported", l, c->down_types[l]);
            free(c->down_types);
            free(c);
            return NULL;
        }
    }
    c->cfg.down_types = c->down_types;

    if (cudaSetDevice(cfg->device) != cudaSuccess) goto fail;
    {
        struct cudaDeviceProp prop;
        c->n_sm = (cudaGetDeviceProperties(&prop, cfg->device) == cudaSuccess) ? prop.multiProcessorCount
                                                                                : FB_N_SM_DEFAULT;
    }
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) goto fail;
    if (cudaEventCreate(&c->ev0) != cudaSuccess || cudaEventCreate(&c->ev1) != cudaSuccess) goto fail;

    c->layers = (fb_layer_t *)calloc((size_t)cfg->n_layers, sizeof(fb_layer_t));
    const int n_recs = cfg->n_experts + (cfg->has_shared ? 1 : 0);
    uint64_t max_rec_ggml = 0;
    for (int l = 0; l < cfg->n_layers; l++) {
        fb_layer_t *L = &c->layers[l];
        L->down_type = c->down_types[l];
        L->down_bytes = fb_shard_bytes_h(L->down_type, c->down_half, (uint64_t)cfg->n_embd * c->down_bpr);
        L->rec_bytes = 2 * c->gate_bytes + L->down_bytes;
        const uint64_t tb = L->rec_bytes * (uint64_t)n_recs;
        if (cudaMalloc((void **)&L->table, tb) != cudaSuccess) {
            set_err(c, "cudaMalloc of %.2f GB for layer %d's experts failed", tb / 1e9, l);
            goto fail;
        }
        c->table_bytes += tb;
        if (dev_alloc(c, (void **)&L->router_w, sizeof(float) * (uint64_t)cfg->n_experts * cfg->n_embd)) goto fail;
        if (dev_alloc(c, (void **)&L->resid, sizeof(float) * cfg->n_embd)) goto fail;
        if (dev_alloc(c, (void **)&L->normw, sizeof(float) * cfg->n_embd)) goto fail;
        if (dev_alloc(c, (void **)&L->mask, sizeof(uint32_t) * 16)) goto fail;
        const uint64_t rg = fomoe_b200_record_bytes(c, l);
        if (rg > max_rec_ggml) max_rec_ggml = rg;
    }
    const int nl = cfg->n_layers, ne = cfg->n_embd;
    if (dev_alloc(c, (void **)&c->x, sizeof(float) * ne) || dev_alloc(c, (void **)&c->h, sizeof(float) * ne) ||
        dev_alloc(c, (void **)&c->moe_out, sizeof(float) * ne) ||
        dev_alloc(c, (void **)&c->logits, sizeof(float) * nl * FB_MAX_EXPERTS) ||
        dev_alloc(c, (void **)&c->all_scores, sizeof(float) * nl * FB_MAX_EXPERTS) ||
        dev_alloc(c, (void **)&c->scores, sizeof(float) * nl * FB_MAX_SLOTS) ||
        dev_alloc(c, (void **)&c->ids, sizeof(int) * nl * FB_MAX_SLOTS) ||
        dev_alloc(c, (void **)&c->ids_orig, sizeof(int) * nl * FB_MAX_SLOTS) ||
        dev_alloc(c, (void **)&c->slot_rec, sizeof(void *) * nl * FB_MAX_SLOTS) ||
        dev_alloc(c, (void **)&c->act, sizeof(float) * FB_MAX_SLOTS * c->inter_local) ||
        dev_alloc(c, (void **)&c->dots, sizeof(float) * FB_MAX_SLOTS * ne) ||
        dev_alloc(c, (void **)&c->q8h, sizeof(fb_q8_entry_t) * (ne / FB_QK)) ||
        dev_alloc(c, (void **)&c->q8a, sizeof(fb_q8_entry_t) * FB_MAX_SLOTS * (c->inter_local / FB_QK)) ||
        dev_alloc(c, (void **)&c->counters, sizeof(unsigned) * (FB_CNT_WIN + FB_MAX_SLOTS * 32 + c->down_groups)) ||
        dev_alloc(c, (void **)&c->status, sizeof(int)) || dev_alloc(c, (void **)&c->tok_ctr, sizeof(unsigned)) ||
        dev_alloc(c, (void **)&c->shared_gate, sizeof(float)) ||
        dev_alloc(c, (void **)&c->d_layer_args, sizeof(fb_args_t) * (uint64_t)nl) ||
        dev_alloc(c, (void **)&c->d_bar, 32 * sizeof(unsigned long long)) ||
        dev_alloc(c, (void **)&c->d_ll_dots, sizeof(unsigned long long) * FB_MAX_SLOTS * (uint64_t)ne) || dev_alloc(c, (void **)&c->d_ll_logits, sizeof(unsigned long long) * FB_MAX_EXPERTS) || dev_alloc(c, (void **)&c->d_abort, sizeof(int)) ||
        dev_alloc(c, (void **)&c->tok_in, sizeof(float) * (uint64_t)(c->max_tokens + 1) * ne) ||
        dev_alloc(c, (void **)&c->tok_out, sizeof(float) * (uint64_t)(c->max_tokens + 1) * ne))
        goto fail;
    if (N > 1) { /* [2][tp_size][n_embd] words; plain cudaMalloc so that it can be shared with the other ranks */
        if (cudaMalloc((void **)&c->tp_recv, sizeof(unsigned long long) * 2 * (size_t)N * ne) != cudaSuccess ||
            cudaMemset(c->tp_recv, 0, sizeof(unsigned long long) * 2 * (size_t)N * ne) != cudaSuccess ||
            dev_alloc(c, (void **)&c->tp_xsum, sizeof(unsigned long long) * (size_t)ne))
            goto fail;
        /* many ranks: add the partials up once per GPU instead of in every thread (stack.cu) */
        c->tp_two_stage = getenv("FOMOE_B200_TP_TWO_STAGE") ? atoi(getenv("FOMOE_B200_TP_TWO_STAGE")) : (N >= 4);
    }
    c->stage_bytes = max_rec_ggml > sizeof(float) * (uint64_t)ne * 1024 ? max_rec_ggml : sizeof(float) * (uint64_t)ne * 1024;
    if (cudaMalloc((void **)&c->stage, c->stage_bytes) != cudaSuccess) goto fail;
    if (cudaHostAlloc((void **)&c->pin, sizeof(float) * (4 * (size_t)ne + 4 * FB_MAX_EXPERTS), cudaHostAllocMapped) !=
        cudaSuccess)
        goto fail;
    if (cudaHostGetDevicePointer((void **)&c->pin_dev, c->pin, 0) != cudaSuccess) goto fail;
    memset(c->pin, 0, sizeof(float) * (4 * (size_t)ne + 4 * FB_MAX_EXPERTS));
    c->host_flags = (int *)(c->pin + 3 * (size_t)ne);
    return c;
fail:
    if (!c->err[0]) set_err(c, "CUDA setup failed: %s", cudaGetErrorString(cudaGetLastError()));
    fomoe_b200_destroy(c);
    return NULL;
}

const char *fomoe_b200_last_error(fomoe_b200_ctx_t *c) { return c ? c->err : "null context"; }

/* A stack launch that gave a wait up leaves its barrier words, hand-over words and abort flag in an unknown state:
 * clear them so that the next launch starts clean.  Generations are NOT reset: every launch, finished or not, has
 * advanced gen_count by its layer-tokens on every rank that made the call, so the ranks still agree, and no word
 * an aborted launch left behind (here or in a peer's receive buffer) can ever match a later generation. */
static void stack_recover(fomoe_b200_ctx_t *c) {
    cudaMemsetAsync(c->d_abort, 0, sizeof(int), c->stream);
    cudaMemsetAsync(c->d_bar, 0, 32 * sizeof(unsigned long long), c->stream);
    cudaMemsetAsync(c->status, 0, sizeof(int), c->stream);
    cudaStreamSynchronize(c->stream);
    c->bar_count = 0;
    c->host_flags[0] = 0;
}

/* after the synchronise that follows a stack launch: 0, or -1 when a block gave a wait up (the kernel said so in
 * mapped host memory; no copy is needed to find out) */
static int stack_finish(fomoe_b200_ctx_t *c) {
    const int code = c->host_flags[0];
    if (!code) return 0;
    c->last_status = code;
    stack_recover(c);
    set_err(c, "the stack kernel gave up a bounded wait (status %d): a peer rank did not deliver, or the wait limit is too "
               "short; results of this call are not valid", code);
    return -1;
}

int fomoe_b200_status(fomoe_b200_ctx_t *c) {
    int st = -1;
    if (!c) return -1;
    cudaSetDevice(c->cfg.device);
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) return -1;
    if (cudaMemcpy(&st, c->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (c->host_flags[0]) { /* a launch whose caller did not synchronise through this library */
        c->last_status = c->host_flags[0];
        stack_recover(c);
    }
    if (st != FB_ST_OK) cudaMemset(c->status, 0, sizeof(int));
    if (c->last_status) st = c->last_status;
    c->last_status = 0; /* reported once: a later successful run reads 0 again */
    return st;
}

uint64_t fomoe_b200_record_bytes(fomoe_b200_ctx_t *c, int layer) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers) return 0;
    return 2 * ggml_matrix_bytes(c->cfg.gate_type, c->cfg.n_inter, c->cfg.n_embd) +
           ggml_matrix_bytes(c->down_types[layer], c->cfg.n_embd, c->cfg.n_inter);
}

uint64_t fomoe_b200_table_bytes(fomoe_b200_ctx_t *c) { return c ? c->table_bytes : 0; }
const fomoe_b200_config_t *fomoe_b200_get_config(fomoe_b200_ctx_t *c) { return c ? &c->cfg : NULL; }
uint64_t fomoe_b200_kernel_launches(fomoe_b200_ctx_t *c) { return c ? c->launches : 0; }

uint64_t fomoe_b200_substitutions(fomoe_b200_ctx_t *c) {
    unsigned v = 0;
    if (!c) return 0;
    cudaSetDevice(c->cfg.device);
    cudaStreamSynchronize(c->stream);
    cudaMemcpy(&v, c->counters + FB_CNT_SUBS, sizeof(unsigned), cudaMemcpyDeviceToHost);
    return v;
}

/* Profiling aid: record %globaltimer stamps of block `cta` at the phase boundaries of the stack kernel
 * for the next run; cap = 0 switches it off.  fomoe_b200_trace_read copies them out: the top byte of each
 * word is the stamp index (0 layer top, 1 joined previous barrier, 2 after RMSNorm/Q8_K, 3 router rows done,
 * 4 logits barrier passed, 5 routing done, 6 gate/up done, 7 activation barrier passed, 8 down done). */
int fomoe_b200_trace_enable(fomoe_b200_ctx_t *c, int cap, int cta) {
    if (!c) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    CK(c, cudaStreamSynchronize(c->stream));
    cudaFree(c->d_trace);
    c->d_trace = NULL;
    c->trace_cap = 0;
    if (cap > 0) {
        const size_t words = (size_t)cap * (cta < 0 ? (size_t)c->n_sm : 1);
        CK(c, cudaMalloc((void **)&c->d_trace, sizeof(unsigned long long) * words));
        CK(c, cudaMemset(c->d_trace, 0, sizeof(unsigned long long) * words));
        c->trace_cap = cap;
        c->trace_cta = cta;
    }
    return 0;
}

int fomoe_b200_trace_read(fomoe_b200_ctx_t *c, unsigned long long *out, int n) {
    if (!c || !out || !c->d_trace || (size_t)n > (size_t)c->trace_cap * (c->trace_cta < 0 ? (size_t)c->n_sm : 1)) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    CK(c, cudaStreamSynchronize(c->stream));
    CK(c, cudaMemcpy(out, c->d_trace, sizeof(unsigned long long) * (size_t)n, cudaMemcpyDeviceToHost));
    return 0;
}

/* ---- tensor parallelism: one process per GPU; the ranks exchange the handle of their receive buffer (through
 * whatever channel the caller has, e.g. torch.distributed) and map each other's buffers.  The reference's
 * counterpart is tp_init / tp_allreduce_sum (include/tp.h:30-79), a host-staged copy between two GPUs of one
 * process; here the sum is fused into the stack kernel and travels as peer stores over NVLink. */
int fomoe_b200_tp_export(fomoe_b200_ctx_t *c, void *handle64) {
    if (!c || !handle64 || !c->tp_recv) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    cudaIpcMemHandle_t h;
    CK(c, cudaIpcGetMemHandle(&h, c->tp_recv));
    memcpy(handle64, &h, sizeof(h));
    return 0;
}

int fomoe_b200_tp_connect(fomoe_b200_ctx_t *c, const void *handles) {
    if (!c || !handles || !c->tp_recv) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    for (int p = 0; p < c->cfg.tp_size; p++) {
        if (p == c->cfg.tp_rank) {
            c->tp_peer[p] = c->tp_recv;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)p * sizeof(h), sizeof(h));
        void *ptr = NULL;
        CK(c, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        c->tp_peer[p] = (unsigned long long *)ptr;
    }
    c->tp_connected = 1;
    return 0;
}

int fomoe_b200_tp_connect_ptrs(fomoe_b200_ctx_t *c, void *const *recv_ptrs) {
    if (!c || !recv_ptrs || !c->tp_recv) return -1;
    for (int p = 0; p < c->cfg.tp_size; p++) {
        if (!recv_ptrs[p]) return -1;
        c->tp_peer[p] = (p == c->cfg.tp_rank) ? c->tp_recv : (unsigned long long *)recv_ptrs[p];
    }
    c->tp_connected = 2; /* nothing to close on destroy */
    return 0;
}

void *fomoe_b200_tp_recv_ptr(fomoe_b200_ctx_t *c) { return c ? (void *)c->tp_recv : NULL; }

int fomoe_b200_set_wait_limit(fomoe_b200_ctx_t *c, unsigned polls) {
    if (!c) return -1;
    c->spin_limit = polls ? polls : 1u << 22;
    return 0;
}

int fomoe_b200_set_allreduce(fomoe_b200_ctx_t *c, fomoe_b200_allreduce_fn fn, void *user) {
    if (!c) return -1;
    drop_graph(c);
    c->allreduce = fn;
    c->allreduce_user = user;
    return 0;
}

void *fomoe_b200_stream(fomoe_b200_ctx_t *c) { return c ? (void *)c->stream : NULL; }

int fomoe_b200_set_act_mode(fomoe_b200_ctx_t *c, int mode) {
    if (!c || (mode != FOMOE_B200_ACT_Q8K && mode != FOMOE_B200_ACT_F32)) return -1;
    if (c->stream) cudaStreamSynchronize(c->stream);
    drop_graph(c);
    c->act_f32 = mode == FOMOE_B200_ACT_F32;
    return 0;
}

int fomoe_b200_set_variant(fomoe_b200_ctx_t *c, int variant) {
    if (!c || variant < 0 || variant > 2) return -1;
    if (c->stream) cudaStreamSynchronize(c->stream);
    drop_graph(c);
    c->variant = variant;
    return 0;
}

int fomoe_b200_set_graphs(fomoe_b200_ctx_t *c, int enable) {
    if (!c) return -1;
    c->use_graphs = enable ? 1 : 0;
    if (!enable) drop_graph(c);
    return 0;
}

/* ------------------------------------------------------------------ routing trace, expert histogram
 * The reference writes one record per layer and token to the file named by QMOE_TRACE_FILE: a 32-byte header and
 * packed records of token id, layer id, the top-k before and after cache-aware routing with their weights, and
 * where each expert came from (src/gpu_kernels.hip:451-484, written at 6306-6340, read by tools/read_trace.py).
 * Here the kernels log every decision on the device (fb_route_rec_t) and the host appends the records after each
 * run.  Arrays hold top_k entries and the record is padded to a multiple of 8 bytes, which is what
 * tools/read_trace.py parses and, for top_k = 10, byte for byte the reference's 144-byte record.  Source codes: every
 * expert is in HBM here, so an expert the residency mask marks as cached (or any expert when no mask is set) is
 * "VRAM" (0), one it does not is what the reference would have fetched: "NVMe" (2); a substituted slot is "CAR" (3),
 * a slot whose weight ended at zero "DROP" (4). */
#define FB_TRACE_MAGIC 0x54524345u

int fomoe_b200_routing_trace_open(fomoe_b200_ctx_t *c, const char *path) {
    if (!c || !path) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    CK(c, cudaStreamSynchronize(c->stream));
    if (c->trace_fp) fclose(c->trace_fp);
    c->trace_fp = fopen(path, "wb");
    if (!c->trace_fp) {
        set_err(c, "cannot create routing trace %s", path);
        return -1;
    }
    if (!c->route_log) {
        if (dev_alloc(c, (void **)&c->route_log, sizeof(fb_route_rec_t) * (size_t)(c->max_tokens + 1) * c->cfg.n_layers)) return -1;
        drop_graph(c); /* the kernels' arguments change */
    }
    uint8_t hd[32];
    memset(hd, 0, sizeof(hd));
    const uint32_t magic = FB_TRACE_MAGIC, version = 1;
    const uint16_t nl = (uint16_t)c->cfg.n_layers, ne = (uint16_t)c->cfg.n_experts, tk = (uint16_t)c->cfg.top_k;
    memcpy(hd, &magic, 4);
    memcpy(hd + 4, &version, 4);
    memcpy(hd + 8, &nl, 2);
    memcpy(hd + 10, &ne, 2);
    memcpy(hd + 12, &tk, 2);
    c->trace_tokens = 0;
    return fwrite(hd, 1, 32, c->trace_fp) == 32 ? 0 : -1;
}

int fomoe_b200_routing_trace_close(fomoe_b200_ctx_t *c) {
    if (!c) return -1;
    int rc = 0;
    if (c->trace_fp) rc = fclose(c->trace_fp) ? -1 : 0;
    c->trace_fp = NULL;
    return rc;
}

/* records of tokens [first, first + count) x layers [l0, l1) from the device log to the file */
static int trace_append(fomoe_b200_ctx_t *c, int first, int count, int l0, int l1) {
    if (!c->trace_fp || !c->route_log) return 0;
    const int nl = c->cfg.n_layers, k = c->cfg.top_k;
    const size_t nrec = (size_t)count * nl;
    fb_route_rec_t *h = (fb_route_rec_t *)malloc(sizeof(fb_route_rec_t) * nrec);
    if (!h) return -1;
    if (cudaMemcpy(h, c->route_log + (size_t)first * nl, sizeof(fb_route_rec_t) * nrec, cudaMemcpyDeviceToHost) != cudaSuccess) {
        free(h);
        set_err(c, "routing trace: copy failed");
        return -1;
    }
    const size_t raw = 8 + (size_t)k * (2 + 4 + 2 + 4 + 1), rec_bytes = (raw + 7) & ~(size_t)7;
    uint8_t *buf = (uint8_t *)calloc(1, rec_bytes);
    int rc = buf ? 0 : -1;
    for (int t = 0; t < count && !rc; t++) {
        for (int l = l0; l < l1 && !rc; l++) {
            const fb_route_rec_t *r = &h[(size_t)t * nl + l];
            const fb_layer_t *L = &c->layers[l];
            memset(buf, 0, rec_bytes);
            const uint32_t tok = c->trace_tokens + (uint32_t)t;
            const uint16_t lid = (uint16_t)l;
            uint8_t n_subs = 0;
            uint8_t *o_ids = buf + 8, *o_sc = o_ids + 2 * k, *f_ids = o_sc + 4 * k, *f_sc = f_ids + 2 * k, *src = f_sc + 4 * k;
            for (int i = 0; i < k; i++) {
                const int16_t oi = (int16_t)r->ids_orig[i], fi = (int16_t)r->ids[i];
                memcpy(o_ids + 2 * i, &oi, 2);
                memcpy(o_sc + 4 * i, &r->scores_orig[i], 4);
                memcpy(f_ids + 2 * i, &fi, 2);
                memcpy(f_sc + 4 * i, &r->scores[i], 4);
                const int e = r->ids_orig[i];
                const int resident = !L->mask_set || ((L->mask_host[(e >> 5) & 15] >> (e & 31)) & 1u);
                uint8_t s = resident ? 0 : 2;
                if (r->ids[i] != r->ids_orig[i]) {
                    s = 3;
                    n_subs++;
                } else if (r->scores[i] == 0.0f)
                    s = 4;
                src[i] = s;
            }
            memcpy(buf, &tok, 4);
            memcpy(buf + 4, &lid, 2);
            buf[6] = (uint8_t)k;
            buf[7] = n_subs;
            if (fwrite(buf, 1, rec_bytes, c->trace_fp) != rec_bytes) rc = -1;
        }
    }
    c->trace_tokens += (uint32_t)count;
    free(buf);
    free(h);
    if (rc) set_err(c, "routing trace: write failed");
    return rc;
}

/* Histogram of the routed expert ids before substitution, [n_layers][n_experts] counters since it was enabled (the
 * reference: gpu_enable_expert_freq / gpu_get_expert_freq, include/gpu.h:50-57, counted at src/gpu_kernels.hip:7832-7835). */
int fomoe_b200_enable_expert_freq(fomoe_b200_ctx_t *c) {
    if (!c) return -1;
    if (c->freq) return 0;
    CK(c, cudaSetDevice(c->cfg.device));
    CK(c, cudaStreamSynchronize(c->stream));
    if (dev_alloc(c, (void **)&c->freq, sizeof(uint32_t) * (size_t)c->cfg.n_layers * c->cfg.n_experts)) return -1;
    drop_graph(c);
    return 0;
}

int fomoe_b200_get_expert_freq(fomoe_b200_ctx_t *c, uint32_t *out) {
    if (!c || !out || !c->freq) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    CK(c, cudaStreamSynchronize(c->stream));
    CK(c, cudaMemcpy(out, c->freq, sizeof(uint32_t) * (size_t)c->cfg.n_layers * c->cfg.n_experts, cudaMemcpyDeviceToHost));
    return 0;
}

/* Ranks in one process: let this context's device store into `peer_device`'s memory. */
int fomoe_b200_tp_enable_peer(fomoe_b200_ctx_t *c, int peer_device) {
    if (!c) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    if (peer_device == c->cfg.device) return 0;
    int can = 0;
    CK(c, cudaDeviceCanAccessPeer(&can, c->cfg.device, peer_device));
    if (!can) {
        set_err(c, "device %d cannot access device %d", c->cfg.device, peer_device);
        return -1;
    }
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
        set_err(c, "cudaDeviceEnablePeerAccess(%d): %s", peer_device, cudaGetErrorString(e));
        return -1;
    }
    cudaGetLastError();
    return 0;
}

/* Diagnostic stand-in for a rank: writes `partial` (n_embd floats, NULL = zeros) into this context's receive buffer
 * as rank src_rank's contribution to the layer-token that lies `ahead` layer-tokens after the last one launched
 * (ahead = 1: the first layer-token of the next call).  Lets a test, or a supervisor that has lost a rank, feed a
 * rank's share from the host instead of from a peer GPU. */
int fomoe_b200_tp_inject(fomoe_b200_ctx_t *c, int src_rank, const float *partial, unsigned ahead) {
    if (!c || !c->tp_recv || src_rank < 0 || src_rank >= c->cfg.tp_size || ahead < 1) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    CK(c, cudaStreamSynchronize(c->stream));
    const int n = c->cfg.n_embd;
    const uint32_t gen = c->gen_count + ahead;
    unsigned long long *w = (unsigned long long *)malloc(sizeof(unsigned long long) * (size_t)n);
    if (!w) return -1;
    for (int i = 0; i < n; i++) {
        uint32_t bits = 0;
        if (partial) memcpy(&bits, &partial[i], 4);
        w[i] = ((unsigned long long)gen << 32) | bits;
    }
    const cudaError_t e = cudaMemcpy(c->tp_recv + ((size_t)(gen & 1u) * c->cfg.tp_size + src_rank) * n, w,
                                     sizeof(unsigned long long) * (size_t)n, cudaMemcpyHostToDevice);
    free(w);
    if (e != cudaSuccess) {
        set_err(c, "tp_inject: %s", cudaGetErrorString(e));
        return -1;
    }
    return 0;
}

/* ------------------------------------------------------------------ table */
int fomoe_b200_table_generate(fomoe_b200_ctx_t *c, uint64_t seed) {
    if (!c) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    const int n_recs = c->cfg.n_experts + (c->cfg.has_shared ? 1 : 0);
    for (int l = 0; l < c->cfg.n_layers; l++) {
        fb_layer_t *L = &c->layers[l];
        fb_shard_geom_t gg = geom_gate(c), gd = geom_down(c, L->down_type);
        CKL(c, fb_launch_gen_shards(L->table, L->rec_bytes, n_recs, seed, (uint32_t)l, FSYN_M_GATE, gg, c->stream));
        CKL(c, fb_launch_gen_shards(L->table + c->gate_bytes, L->rec_bytes, n_recs, seed, (uint32_t)l, FSYN_M_UP, gg,
                                    c->stream));
        CKL(c, fb_launch_gen_shards(L->table + 2 * c->gate_bytes, L->rec_bytes, n_recs, seed, (uint32_t)l, FSYN_M_DOWN,
                                    gd, c->stream));
        CKL(c, fb_launch_gen_f32(L->router_w, (uint64_t)c->cfg.n_experts * c->cfg.n_embd, seed, (uint32_t)l,
                                 FSYN_M_ROUTER, 0.0f, FOMOE_ROUTER_STD, c->stream));
        CKL(c, fb_launch_gen_f32(L->resid, (uint64_t)c->cfg.n_embd, seed, (uint32_t)l, FSYN_M_RESID, 0.0f,
                                 FOMOE_RESID_STD, c->stream));
        CKL(c, fb_launch_gen_f32(L->normw, (uint64_t)c->cfg.n_embd, seed, (uint32_t)l, FSYN_M_NORMW, FOMOE_NORMW_MEAN,
                                 FOMOE_NORMW_STD, c->stream));
    }
    CK(c, cudaStreamSynchronize(c->stream));
    return 0;
}

static int check_rec(fomoe_b200_ctx_t *c, int layer, int expert) {
    const int n_recs = c->cfg.n_experts + (c->cfg.has_shared ? 1 : 0);
    if (layer < 0 || layer >= c->cfg.n_layers || expert < 0 || expert >= n_recs) {
        set_err(c, "layer %d / expert %d out of range", layer, expert);
        return -1;
    }
    return 0;
}

/* enqueue: H2D of one ggml record + repack of its three matrices into record slot `expert`.  down_type: 0 = the
 * layer's own; the one-layer engines behind the operator surfaces take whatever type a call brings (their record
 * slots are sized for the largest).  stage_idx < 0: the single staging buffer on the context's stream (the caller
 * synchronises before reusing it); >= 0: staging buffer stage_idx & 1, filled on the copy stream. */
static int upload_record(fomoe_b200_ctx_t *c, int layer, int expert, const void *record, int down_type, int stage_idx) {
    fb_layer_t *L = &c->layers[layer];
    const int dt = down_type ? down_type : L->down_type;
    const uint64_t gb = ggml_matrix_bytes(c->cfg.gate_type, c->cfg.n_inter, c->cfg.n_embd);
    const uint64_t rb = 2 * gb + ggml_matrix_bytes(dt, c->cfg.n_embd, c->cfg.n_inter);
    uint8_t *dst = L->table + (uint64_t)expert * L->rec_bytes;
    /* `record` may be a host pointer (the reference's callers, src/inference.c:538-549: staged through a device
     * buffer) or memory of this GPU (an expert that a caller already keeps in device memory: repacked where it lies) */
    const uint8_t *src = c->stage;
    struct cudaPointerAttributes at;
    int buf = -1;
    if (cudaPointerGetAttributes(&at, record) == cudaSuccess && at.type == cudaMemoryTypeDevice &&
        at.device == c->cfg.device) {
        src = (const uint8_t *)record;
    } else {
        cudaGetLastError(); /* an unregistered host pointer is not an error */
        if (rb > c->stage_bytes) {
            set_err(c, "record of %llu bytes exceeds the staging buffer", (unsigned long long)rb);
            return -1;
        }
        if (stage_idx < 0) {
            CK(c, cudaMemcpyAsync(c->stage, record, rb, cudaMemcpyDefault, c->stream));
        } else {
            buf = stage_idx & 1;
            if (!c->copy_stream) {
                CK(c, cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
                CK(c, cudaMalloc((void **)&c->stage2, c->stage_bytes));
                for (int i = 0; i < 2; i++) {
                    CK(c, cudaEventCreateWithFlags(&c->ev_full[i], cudaEventDisableTiming));
                    CK(c, cudaEventCreateWithFlags(&c->ev_free[i], cudaEventDisableTiming));
                }
            }
            uint8_t *stg = buf ? c->stage2 : c->stage;
            src = stg;
            CK(c, cudaStreamWaitEvent(c->copy_stream, c->ev_free[buf], 0)); /* its previous contents have been regrouped */
            CK(c, cudaMemcpyAsync(stg, record, rb, cudaMemcpyDefault, c->copy_stream));
            CK(c, cudaEventRecord(c->ev_full[buf], c->copy_stream));
            CK(c, cudaStreamWaitEvent(c->stream, c->ev_full[buf], 0));
        }
    }
    fb_shard_geom_t gd = geom_down(c, dt);
    CKL(c, fb_launch_repack(dst, src, geom_gate(c), c->stream));
    CKL(c, fb_launch_repack(dst + c->gate_bytes, src + gb, geom_gate(c), c->stream));
    CKL(c, fb_launch_repack(dst + 2 * c->gate_bytes, src + 2 * gb, gd, c->stream));
    if (buf >= 0) CK(c, cudaEventRecord(c->ev_free[buf], c->stream));
    return 0;
}

/* records [0, n) of layer 0 from the caller's buffers, without the host waiting in between */
static int upload_records(fomoe_b200_ctx_t *c, int n, void *const *records, const b200_expert_work_t *work, int down_type) {
    for (int e = 0; e < n; e++) {
        const void *r = records ? records[e] : work[e].expert_data;
        if (!r) return -1;
        if (c->serial_upload) {
            if (upload_record(c, 0, e, r, down_type, -1)) return -1;
            CK(c, cudaStreamSynchronize(c->stream));
        } else if (upload_record(c, 0, e, r, down_type, e))
            return -1;
    }
    return 0;
}

int fomoe_b200_table_upload(fomoe_b200_ctx_t *c, int layer, int expert, const void *record) {
    if (!c || !record || check_rec(c, layer, expert)) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    if (upload_record(c, layer, expert, record, 0, -1)) return -1;
    CK(c, cudaStreamSynchronize(c->stream)); /* the staging buffer is reused by the next call */
    return 0;
}

/* ---- expert store files of the reference (".qmoe", include/expert_store.h:9-40): a 64-byte header, a table of
 * 32-byte layer entries, then for each layer its experts at data_offset + e * stride, each expert gate | up | down in
 * ggml order (tools/prepare_experts.c:262-291).  The routed experts of store layers first_store_layer ..
 * first_store_layer + n_layers - 1 are read and repacked into the table; the shared expert is not part of such a
 * file.  Returns the number of experts loaded, or -1. */
typedef struct {
    uint32_t magic, version, n_moe_layers, n_experts, quant_type, alignment;
    uint64_t gate_size, up_size, down_size, stride;
} qmoe_head_t;
typedef struct {
    uint64_t data_offset, stride, down_size;
    uint32_t down_type, pad;
} qmoe_layer_t;

int fomoe_b200_table_load_qmoe(fomoe_b200_ctx_t *c, const char *path, int first_store_layer) {
    if (!c || !path || first_store_layer < 0) return -1;
    FILE *f = fopen(path, "rb");
    if (!f) {
        set_err(c, "cannot open expert store %s", path);
        return -1;
    }
    int rc = -1, loaded = 0;
    uint8_t *buf = NULL;
    qmoe_layer_t *idx = NULL;
    qmoe_head_t hd;
    if (fread(&hd, sizeof(hd), 1, f) != 1 || hd.magic != 0x454F4D51u || hd.version < 2) {
        set_err(c, "%s: not an expert store of version >= 2", path);
        goto done;
    }
    const uint64_t gb = ggml_matrix_bytes(c->cfg.gate_type, c->cfg.n_inter, c->cfg.n_embd);
    if ((int)hd.n_experts != c->cfg.n_experts || hd.gate_size != gb || hd.up_size != gb ||
        (uint64_t)first_store_layer + (uint64_t)c->cfg.n_layers > hd.n_moe_layers) {
        set_err(c, "%s: %u layers of %u experts, gate/up %llu/%llu bytes do not match the table (%d layers from %d, %d "
                   "experts, %llu bytes)", path, hd.n_moe_layers, hd.n_experts, (unsigned long long)hd.gate_size,
                (unsigned long long)hd.up_size, c->cfg.n_layers, first_store_layer, c->cfg.n_experts,
                (unsigned long long)gb);
        goto done;
    }
    idx = (qmoe_layer_t *)malloc(sizeof(qmoe_layer_t) * hd.n_moe_layers);
    if (!idx || fseek(f, 64, SEEK_SET) || fread(idx, sizeof(qmoe_layer_t), hd.n_moe_layers, f) != hd.n_moe_layers) {
        set_err(c, "%s: layer index unreadable", path);
        goto done;
    }
    for (int l = 0; l < c->cfg.n_layers; l++) {
        const qmoe_layer_t *e = &idx[first_store_layer + l];
        const uint64_t stride = e->stride ? e->stride : hd.stride, rb = fomoe_b200_record_bytes(c, l);
        if ((int)e->down_type != c->down_types[l] || e->down_size != rb - 2 * gb || stride < rb) {
            set_err(c, "%s: store layer %d has down type %u / %llu bytes, the table expects type %d / %llu bytes", path,
                    first_store_layer + l, e->down_type, (unsigned long long)e->down_size, c->down_types[l],
                    (unsigned long long)(rb - 2 * gb));
            goto done;
        }
        if (!buf) buf = (uint8_t *)malloc(c->stage_bytes);
        if (!buf) goto done;
        for (int x = 0; x < c->cfg.n_experts; x++) {
            if (fseeko(f, (off_t)(e->data_offset + (uint64_t)x * stride), SEEK_SET) || fread(buf, 1, rb, f) != rb) {
                set_err(c, "%s: short read at layer %d expert %d", path, first_store_layer + l, x);
                goto done;
            }
            if (fomoe_b200_table_upload(c, l, x, buf)) goto done;
            loaded++;
        }
    }
    rc = loaded;
done:
    free(buf);
    free(idx);
    fclose(f);
    return rc;
}

static int shard_of(fomoe_b200_ctx_t *c, int layer, int expert, int matrix, const uint8_t **shard,
                    fb_shard_geom_t *g) {
    if (check_rec(c, layer, expert) || matrix < 0 || matrix > 2) return -1;
    fb_layer_t *L = &c->layers[layer];
    const uint8_t *rec = L->table + (uint64_t)expert * L->rec_bytes;
    *shard = rec + (matrix == 0 ? 0 : matrix == 1 ? c->gate_bytes : 2 * c->gate_bytes);
    *g = matrix == 2 ? geom_down(c, L->down_type) : geom_gate(c);
    return 0;
}

int fomoe_b200_table_export(fomoe_b200_ctx_t *c, int layer, int expert, int matrix, void *out) {
    const uint8_t *shard;
    fb_shard_geom_t g;
    if (!c || !out || shard_of(c, layer, expert, matrix, &shard, &g)) return -1;
    if (g.half >= 0) {
        set_err(c, "table_export: a shard of half super-blocks has no ggml form (use table_dequant)");
        return -1;
    }
    CK(c, cudaSetDevice(c->cfg.device));
    const uint64_t bytes = (uint64_t)g.rows_local * g.bpr_local * fb_block_bytes(g.type);
    CKL(c, fb_launch_export_ggml(c->stage, shard, g, c->stream));
    CK(c, cudaMemcpyAsync(out, c->stage, bytes, cudaMemcpyDeviceToHost, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    return 0;
}

int fomoe_b200_table_dequant(fomoe_b200_ctx_t *c, int layer, int expert, int matrix, float *out) {
    const uint8_t *shard;
    fb_shard_geom_t g;
    if (!c || !out || shard_of(c, layer, expert, matrix, &shard, &g)) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    const uint64_t bytes = sizeof(float) * (uint64_t)g.rows_local * g.bpr_local * (g.half >= 0 ? FB_QK / 2 : FB_QK);
    float *tmp = NULL;
    CK(c, cudaMalloc((void **)&tmp, bytes));
    int rc = fb_launch_dequant(tmp, shard, g, c->stream);
    c->launches++;
    cudaError_t e = rc ? (cudaError_t)rc : cudaMemcpyAsync(out, tmp, bytes, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    cudaFree(tmp);
    if (e != cudaSuccess) {
        set_err(c, "table_dequant: %s", cudaGetErrorString(e));
        return -1;
    }
    return 0;
}

int fomoe_b200_router_upload(fomoe_b200_ctx_t *c, int layer, const float *w) {
    if (!c || !w || layer < 0 || layer >= c->cfg.n_layers) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    CK(c, cudaMemcpyAsync(c->layers[layer].router_w, w, sizeof(float) * (uint64_t)c->cfg.n_experts * c->cfg.n_embd,
                          cudaMemcpyHostToDevice, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    return 0;
}

int fomoe_b200_glue_upload(fomoe_b200_ctx_t *c, int layer, const float *resid, const float *normw) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    if (resid)
        CK(c, cudaMemcpyAsync(c->layers[layer].resid, resid, sizeof(float) * c->cfg.n_embd, cudaMemcpyHostToDevice,
                              c->stream));
    if (normw)
        CK(c, cudaMemcpyAsync(c->layers[layer].normw, normw, sizeof(float) * c->cfg.n_embd, cudaMemcpyHostToDevice,
                              c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    return 0;
}

int fomoe_b200_shared_gate_upload(fomoe_b200_ctx_t *c, int layer, const float *w) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers || !c->cfg.has_shared) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    drop_graph(c);
    fb_layer_t *L = &c->layers[layer];
    if (!w) {
        if (L->shared_gate_w) cudaFree(L->shared_gate_w);
        L->shared_gate_w = NULL;
        return 0;
    }
    if (!L->shared_gate_w && dev_alloc(c, (void **)&L->shared_gate_w, sizeof(float) * c->cfg.n_embd)) return -1;
    CK(c, cudaMemcpyAsync(L->shared_gate_w, w, sizeof(float) * c->cfg.n_embd, cudaMemcpyHostToDevice, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    return 0;
}

int fomoe_b200_set_resident_mask(fomoe_b200_ctx_t *c, int layer, const uint32_t *mask) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    drop_graph(c);
    c->layers[layer].mask_set = mask != NULL;
    if (mask) {
        memcpy(c->layers[layer].mask_host, mask, sizeof(uint32_t) * 16);
        CK(c, cudaMemcpyAsync(c->layers[layer].mask, mask, sizeof(uint32_t) * 16, cudaMemcpyHostToDevice, c->stream));
        CK(c, cudaStreamSynchronize(c->stream));
    }
    return 0;
}

int fomoe_b200_set_car(fomoe_b200_ctx_t *c, float threshold, int dampen) {
    if (!c) return -1;
    drop_graph(c);
    c->cfg.car_threshold = threshold;
    c->cfg.car_dampen = dampen ? 1 : 0;
    return 0;
}

/* ------------------------------------------------------------------ launch sequence */
static void fill_args(const fomoe_b200_ctx_t *c, int layer, fb_args_t *a) {
    const fb_layer_t *L = &c->layers[layer];
    memset(a, 0, sizeof(*a));
    a->n_embd = c->cfg.n_embd;
    a->n_inter = c->cfg.n_inter;
    a->inter_local = c->inter_local;
    a->n_experts = c->cfg.n_experts;
    a->top_k = c->cfg.top_k;
    a->has_shared = c->cfg.has_shared ? 1 : 0;
    a->n_slots = c->n_slots;
    a->tp_rank = c->cfg.tp_rank;
    a->tp_size = c->cfg.tp_size;
    a->gate_bpr = c->gate_bpr;
    a->down_bpr = c->down_bpr;
    a->gate_type = c->cfg.gate_type;
    a->gate_groups = c->gate_groups;
    a->down_groups = c->down_groups;
    a->up_off = c->gate_bytes;
    a->down_off = 2 * c->gate_bytes;
    a->rms_eps = c->cfg.rms_eps;
    a->car_threshold = c->cfg.car_threshold;
    a->car_dampen = c->cfg.car_dampen;
    a->table_layer = L->table;
    a->rec_bytes = L->rec_bytes;
    a->down_type = L->down_type;
    a->down_half = c->down_half;
    a->router_w = L->router_w;
    a->resid = L->resid;
    a->normw = L->normw;
    a->resident = L->mask_set ? L->mask : NULL;
    a->shared_gate_w = c->cfg.has_shared ? L->shared_gate_w : NULL;
    a->shared_gate = c->shared_gate;
    a->freq = c->freq ? c->freq + (size_t)layer * c->cfg.n_experts : NULL;
    a->x = c->x;
    a->h = c->h;
    a->moe_out = c->moe_out;
    a->q8h = c->q8h;
    a->logits = c->logits + (size_t)layer * FB_MAX_EXPERTS;
    a->all_scores = c->all_scores + (size_t)layer * FB_MAX_EXPERTS;
    a->ids = c->ids + (size_t)layer * FB_MAX_SLOTS;
    a->ids_orig = c->ids_orig + (size_t)layer * FB_MAX_SLOTS;
    a->scores = c->scores + (size_t)layer * FB_MAX_SLOTS;
    a->slot_rec = c->slot_rec + (size_t)layer * FB_MAX_SLOTS;
    a->act = c->act;
    a->q8a = c->q8a;
    a->dots = c->dots;
    a->counters = c->counters;
    a->status = c->status;
    a->tok_in = c->tok_in;
    a->tok_out = c->tok_out;
    a->tok_ctr = c->tok_ctr;
    a->route_log = c->route_log ? c->route_log + layer : NULL;
    a->route_stride = c->cfg.n_layers;
}

static int grid_router(const fomoe_b200_ctx_t *c) {
    int g = (c->cfg.n_experts + 7) / 8;
    return g < 1 ? 1 : g;
}

static int grid_tasks(const fomoe_b200_ctx_t *c, int tasks) {
    /* 8 warps per block; up to 2 blocks per SM */
    int g = (tasks + 7) / 8, cap = 2 * c->n_sm;
    return g < 1 ? 1 : (g > cap ? cap : g);
}

/* expert phase of one layer: gate/up/SwiGLU then down/combine, on the slots already set */
static int enqueue_experts(fomoe_b200_ctx_t *c, const fb_args_t *a) {
    if (c->act_f32) {
        CKL(c, fb_launch_gate_up_f32(a, grid_tasks(c, a->n_slots * a->gate_groups), c->stream));
        CKL(c, fb_launch_down_f32(a, grid_tasks(c, a->n_slots * a->down_groups), c->stream));
        return 0;
    }
    if (c->variant != 1 || a->n_slots > 15 || a->gate_type != FB_TYPE_Q4_K) {
        CKL(c, fb_launch_gate_up(a, grid_tasks(c, a->n_slots * a->gate_groups), c->stream));
        CKL(c, fb_launch_down(a, grid_tasks(c, a->n_slots * a->down_groups), c->stream));
        return 0;
    }
    /* bulk-copy rings: one block per SM */
    int g1 = (a->n_slots * a->gate_groups + 7) / 8, g2 = a->down_groups;
    CKL(c, fb_launch_gate_up_ring(a, g1 < c->n_sm ? g1 : c->n_sm, c->stream));
    CKL(c, fb_launch_down_ring(a, g2 < c->n_sm ? g2 : c->n_sm, c->stream));
    return 0;
}

/* layers [l0, l1) of one token; flags_first / store select where x comes from and goes to */
static int enqueue_stack(fomoe_b200_ctx_t *c, int l0, int l1, int load_store) {
    fb_args_t a;
    for (int l = l0; l < l1; l++) {
        fill_args(c, l, &a);
        if (!load_store) a.route_log = NULL; /* the log is indexed by the token counter, which only token runs set */
        int flags = FB_PRO_RESID | FB_PRO_NORM | FB_PRO_QUANT;
        if (l > l0) flags |= FB_PRO_ADD_PREV;
        else if (load_store) flags |= FB_PRO_LOAD;
        CKL(c, fb_launch_prologue(&a, flags, c->stream));
        CKL(c, fb_launch_router(&a, grid_router(c), c->stream));
        if (enqueue_experts(c, &a)) return -1;
        if (c->allreduce && c->cfg.tp_size > 1 &&
            c->allreduce(c->allreduce_user, c->moe_out, c->cfg.n_embd, (void *)c->stream)) {
            set_err(c, "the caller's all-reduce reported a failure at layer %d", l);
            return -1;
        }
    }
    fill_args(c, l1 - 1, &a);
    CKL(c, fb_launch_prologue(&a, FB_PRO_ADD_PREV | (load_store ? FB_PRO_STORE : 0), c->stream));
    return 0;
}

/* launches of the per-phase path are replayed from a CUDA graph unless the caller's collective sits between them */
static int graphs_on(const fomoe_b200_ctx_t *c) { return c->use_graphs && !(c->allreduce && c->cfg.tp_size > 1); }

static int stack_kernel_usable(fomoe_b200_ctx_t *c) {
    fb_args_t a;
    if (c->variant != 2 || c->act_f32) return 0;
    if (c->cfg.tp_size > 1 && !c->tp_connected) return 0;
    fill_args(c, 0, &a);
    return fb_stack_supported(&a, c->n_sm);
}

/* layers [l0, l1) of `count` resident tokens starting at index `first`: one launch.  out_host: NULL, or where (mapped
 * host memory) the last token's output goes instead of its slot in tok_out. */
static int launch_stack_kernel(fomoe_b200_ctx_t *c, int l0, int l1, int first, int count, float *out_host) {
    if (!c->layer_args_valid) {
        fb_args_t *tmp = (fb_args_t *)malloc(sizeof(fb_args_t) * (size_t)c->cfg.n_layers);
        if (!tmp) return -1;
        for (int l = 0; l < c->cfg.n_layers; l++) fill_args(c, l, &tmp[l]);
        cudaError_t e = cudaMemcpy(c->d_layer_args, tmp, sizeof(fb_args_t) * (size_t)c->cfg.n_layers, cudaMemcpyHostToDevice);
        free(tmp);
        if (e != cudaSuccess) {
            set_err(c, "uploading layer arguments: %s", cudaGetErrorString(e));
            return -1;
        }
        c->layer_args_valid = 1;
    }
    fb_stack_args_t k;
    k.layers = c->d_layer_args + l0;
    k.n_layers = l1 - l0;
    k.down_mode = c->down_half >= 0 ? 2 : 0;
    for (int l = 0; l < c->cfg.n_layers; l++)
        if (c->down_half < 0 && c->down_types[l] == FB_TYPE_Q5_K) k.down_mode = 1;
    k.tok_count = count;
    k.tok_first = first;
    k.tok_in = c->tok_in;
    k.tok_out = c->tok_out;
    k.out_host = out_host;
    k.tok_ctr = c->tok_ctr;
    k.bar = c->d_bar;
    k.bar_base = c->bar_count;
    k.ll_dots = c->d_ll_dots;
    k.ll_logits = c->d_ll_logits;
    k.gen_base = c->gen_count;
    k.abort_flag = c->d_abort;
    k.spin_limit = c->spin_limit;
    k.status = c->status;
    k.tp_rank = c->cfg.tp_rank;
    k.tp_size = c->cfg.tp_size;
    k.tp_recv = c->tp_recv;
    for (int p = 0; p < FB_MAX_TP; p++) k.tp_peer[p] = c->tp_peer[p];
    k.tp_xsum = c->tp_xsum;
    k.tp_two_stage = c->tp_two_stage;
    k.host_flags = (int *)(c->pin_dev + 3 * (size_t)c->cfg.n_embd);
    k.trace = c->d_trace;
    k.trace_cap = c->d_trace ? c->trace_cap : 0;
    k.trace_cta = c->trace_cta;
    /* the abort flag is zero unless an earlier launch gave up; stack_finish / fomoe_b200_status clear it again */
    CKL(c, fb_launch_stack(&k, c->n_sm, c->stream));
    /* grid barriers per layer-token, every block arriving once at each: one GPU -- activations and block output (the
     * logits cross as self-validating words without a barrier); a tensor-parallel rank -- logits and activations
     * (the block output is exchanged through the ranks' receive buffers) */
    c->bar_count += 2ull * (unsigned long long)((l1 - l0) * count) * (unsigned long long)c->n_sm;
    c->gen_count += (unsigned)((l1 - l0) * count);
    return 0;
}

int fomoe_b200_moe_layer(fomoe_b200_ctx_t *c, int layer, const float *h, float *out, int *ids_out, float *scores_out,
                         int *ids_orig_out, float *all_scores_out) {
    if (!c || !h || !out || layer < 0 || layer >= c->cfg.n_layers) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    const size_t nb = sizeof(float) * c->cfg.n_embd;
    fb_args_t a;
    fill_args(c, layer, &a);
    a.route_log = NULL; /* single-layer calls are not part of a token's trace */
    memcpy(c->pin, h, nb);
    CK(c, cudaMemcpyAsync(c->x, c->pin, nb, cudaMemcpyHostToDevice, c->stream));
    CKL(c, fb_launch_prologue(&a, FB_PRO_QUANT, c->stream));
    CKL(c, fb_launch_router(&a, grid_router(c), c->stream));
    if (enqueue_experts(c, &a)) return -1;
    CK(c, cudaMemcpyAsync(c->pin + c->cfg.n_embd, c->moe_out, nb, cudaMemcpyDeviceToHost, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    memcpy(out, c->pin + c->cfg.n_embd, nb);
    if (ids_out || scores_out || ids_orig_out) {
        if (fomoe_b200_get_routing(c, layer, ids_out, scores_out, ids_orig_out)) return -1;
    }
    if (all_scores_out)
        CK(c, cudaMemcpy(all_scores_out, a.all_scores, sizeof(float) * c->cfg.n_experts, cudaMemcpyDeviceToHost));
    return 0;
}

/* shared by moe_layer_routed and the operator surfaces: n experts given by the caller */
static int run_routed(fomoe_b200_ctx_t *c, int layer, const float *h, const int *ids, const float *scores, int n,
                      int with_shared, int accumulate, float *out, int sync, int down_type) {
    if (n < 1 || n > FB_MAX_TOPK) {
        set_err(c, "n experts %d out of range", n);
        return -1;
    }
    const size_t nb = sizeof(float) * c->cfg.n_embd;
    fb_args_t a;
    if (c->pin_busy) {
        CK(c, cudaStreamSynchronize(c->stream));
        c->pin_busy = 0;
    }
    fill_args(c, layer, &a);
    a.route_log = NULL;
    if (down_type) a.down_type = down_type; /* operator surfaces: the type of this call's records */
    a.top_k = n;
    a.has_shared = with_shared ? 1 : 0;
    a.n_slots = n + a.has_shared;
    a.accumulate = accumulate;
    int *pi = (int *)(c->pin + 2 * c->cfg.n_embd);
    float *ps = (float *)(pi + FB_MAX_SLOTS);
    if (h) {
        memcpy(c->pin, h, nb);
        CK(c, cudaMemcpyAsync(c->x, c->pin, nb, cudaMemcpyHostToDevice, c->stream));
        CKL(c, fb_launch_prologue(&a, FB_PRO_QUANT, c->stream));
    }
    for (int i = 0; i < n; i++) {
        pi[i] = ids[i];
        ps[i] = scores[i];
    }
    CK(c, cudaMemcpyAsync(a.ids, pi, sizeof(int) * n, cudaMemcpyHostToDevice, c->stream));
    CK(c, cudaMemcpyAsync(a.scores, ps, sizeof(float) * n, cudaMemcpyHostToDevice, c->stream));
    CKL(c, fb_launch_set_slots(&a, c->stream));
    if (enqueue_experts(c, &a)) return -1;
    if (out) CK(c, cudaMemcpyAsync(c->pin + c->cfg.n_embd, c->moe_out, nb, cudaMemcpyDeviceToHost, c->stream));
    if (sync) {
        CK(c, cudaStreamSynchronize(c->stream));
        if (out) memcpy(out, c->pin + c->cfg.n_embd, nb);
    } else {
        c->pin_busy = 1;
    }
    return 0;
}

int fomoe_b200_moe_layer_routed(fomoe_b200_ctx_t *c, int layer, const float *h, const int *ids, const float *scores,
                                int n, float *out) {
    if (!c || !h || !ids || !scores || !out || layer < 0 || layer >= c->cfg.n_layers) return -1;
    if (n > c->cfg.top_k) {
        set_err(c, "n %d exceeds top_k %d", n, c->cfg.top_k);
        return -1;
    }
    CK(c, cudaSetDevice(c->cfg.device));
    return run_routed(c, layer, h, ids, scores, n, c->cfg.has_shared, 0, out, 1, 0);
}

int fomoe_b200_stack_run(fomoe_b200_ctx_t *c, const float *x_in, int l0, int l1, float *x_out) {
    if (!c || !x_in || !x_out || l0 < 0 || l1 > c->cfg.n_layers || l0 >= l1) return -1;
    if (c->cfg.tp_size > 1 && !stack_kernel_usable(c) && !c->allreduce) {
        set_err(c, "stack_run on a tensor-parallel rank needs fomoe_b200_tp_connect (or an all-reduce hook) first");
        return -1;
    }
    CK(c, cudaSetDevice(c->cfg.device));
    const size_t nb = sizeof(float) * c->cfg.n_embd;
    memcpy(c->pin, x_in, nb);
    if (stack_kernel_usable(c)) { /* the spare token slot past max_tokens carries host-to-host calls */
        CK(c, cudaMemcpyAsync(c->tok_in + (size_t)c->max_tokens * c->cfg.n_embd, c->pin, nb, cudaMemcpyHostToDevice, c->stream));
        if (launch_stack_kernel(c, l0, l1, c->max_tokens, 1, c->pin_dev + c->cfg.n_embd)) return -1;
        CK(c, cudaStreamSynchronize(c->stream));
        if (stack_finish(c)) return -1; /* x_out is left untouched */
        memcpy(x_out, c->pin + c->cfg.n_embd, nb);
        return trace_append(c, c->max_tokens, 1, l0, l1);
    }
    CK(c, cudaMemcpyAsync(c->x, c->pin, nb, cudaMemcpyHostToDevice, c->stream));
    if (enqueue_stack(c, l0, l1, 0)) return -1;
    CK(c, cudaMemcpyAsync(c->pin + c->cfg.n_embd, c->x, nb, cudaMemcpyDeviceToHost, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    memcpy(x_out, c->pin + c->cfg.n_embd, nb);
    return 0;
}

int fomoe_b200_tokens_upload(fomoe_b200_ctx_t *c, int first, int count, const float *x) {
    if (!c || !x || first < 0 || count < 1 || first + count > c->max_tokens) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    CK(c, cudaMemcpyAsync(c->tok_in + (size_t)first * c->cfg.n_embd, x, sizeof(float) * (size_t)count * c->cfg.n_embd,
                          cudaMemcpyHostToDevice, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    return 0;
}

int fomoe_b200_tokens_download(fomoe_b200_ctx_t *c, int first, int count, float *x_out) {
    if (!c || !x_out || first < 0 || count < 1 || first + count > c->max_tokens) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    CK(c, cudaMemcpyAsync(x_out, c->tok_out + (size_t)first * c->cfg.n_embd,
                          sizeof(float) * (size_t)count * c->cfg.n_embd, cudaMemcpyDeviceToHost, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    return 0;
}

static int build_graph(fomoe_b200_ctx_t *c) {
    cudaGraph_t g = NULL;
    const uint64_t before = c->launches;
    CK(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_stack(c, 0, c->cfg.n_layers, 1);
    cudaError_t e = cudaStreamEndCapture(c->stream, &g);
    c->graph_nodes = (int)(c->launches - before);
    c->launches = before;
    if (rc || e != cudaSuccess || !g) {
        if (g) cudaGraphDestroy(g);
        set_err(c, "graph capture failed: %s", cudaGetErrorString(e));
        return -1;
    }
    e = cudaGraphInstantiate(&c->graph_exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) {
        c->graph_exec = NULL;
        set_err(c, "graph instantiate failed: %s", cudaGetErrorString(e));
        return -1;
    }
    return 0;
}

int fomoe_b200_tokens_run(fomoe_b200_ctx_t *c, int first, int count, float *elapsed_ms) {
    if (!c || first < 0 || count < 1 || first + count > c->max_tokens) return -1;
    if (c->cfg.tp_size > 1 && !stack_kernel_usable(c) && !c->allreduce) {
        set_err(c, "tokens_run on a tensor-parallel rank needs fomoe_b200_tp_connect (or an all-reduce hook) first");
        return -1;
    }
    CK(c, cudaSetDevice(c->cfg.device));
    unsigned f = (unsigned)first;
    if (stack_kernel_usable(c)) {
        CK(c, cudaEventRecord(c->ev0, c->stream));
        if (launch_stack_kernel(c, 0, c->cfg.n_layers, first, count, NULL)) return -1;
        CK(c, cudaEventRecord(c->ev1, c->stream));
        CK(c, cudaStreamSynchronize(c->stream));
        if (elapsed_ms) CK(c, cudaEventElapsedTime(elapsed_ms, c->ev0, c->ev1));
        if (stack_finish(c)) return -1;
        return trace_append(c, first, count, 0, c->cfg.n_layers);
    }
    if (graphs_on(c) && !c->graph_exec && build_graph(c)) return -1;
    CK(c, cudaMemcpyAsync(c->tok_ctr, &f, sizeof(unsigned), cudaMemcpyHostToDevice, c->stream));
    CK(c, cudaEventRecord(c->ev0, c->stream));
    for (int t = 0; t < count; t++) {
        if (graphs_on(c)) {
            CK(c, cudaGraphLaunch(c->graph_exec, c->stream));
            c->launches += (uint64_t)c->graph_nodes;
        } else if (enqueue_stack(c, 0, c->cfg.n_layers, 1))
            return -1;
    }
    CK(c, cudaEventRecord(c->ev1, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    if (elapsed_ms) CK(c, cudaEventElapsedTime(elapsed_ms, c->ev0, c->ev1));
    return trace_append(c, first, count, 0, c->cfg.n_layers);
}

/* records an event before each kernel launch while profiling; the phase is read off the call text */
static void prof_mark(fomoe_b200_ctx_t *c, const char *call) {
    if (c->pev_n >= c->pev_cap) return;
    int ph = strstr(call, "prologue") ? 0 : strstr(call, "router") ? 1 : strstr(call, "gate_up") ? 2
           : strstr(call, "fb_launch_down") ? 3 : 4;
    c->pev_phase[c->pev_n] = ph;
    cudaEventRecord(c->pev[c->pev_n++], c->stream);
}

int fomoe_b200_tokens_profile(fomoe_b200_ctx_t *c, int first, int count, float *phase_ms, int *phase_launches) {
    if (!c || !phase_ms || first < 0 || count < 1 || first + count > c->max_tokens) return -1;
    if (c->cfg.tp_size > 1) {
        set_err(c, "tokens_profile: single-rank only");
        return -1;
    }
    CK(c, cudaSetDevice(c->cfg.device));
    const int per_tok = 4 * c->cfg.n_layers + 1, need = per_tok * count + 1;
    if (c->pev_cap < need) {
        for (int i = 0; i < c->pev_cap; i++) cudaEventDestroy(c->pev[i]);
        free(c->pev);
        free(c->pev_phase);
        c->pev = (cudaEvent_t *)calloc((size_t)need, sizeof(cudaEvent_t));
        c->pev_phase = (int *)calloc((size_t)need, sizeof(int));
        c->pev_cap = 0;
        for (int i = 0; i < need; i++) {
            CK(c, cudaEventCreate(&c->pev[i]));
            c->pev_cap = i + 1;
        }
    }
    unsigned f = (unsigned)first;
    CK(c, cudaMemcpyAsync(c->tok_ctr, &f, sizeof(unsigned), cudaMemcpyHostToDevice, c->stream));
    c->pev_n = 0;
    c->profiling = 1;
    int rc = 0;
    for (int t = 0; t < count && !rc; t++) rc = enqueue_stack(c, 0, c->cfg.n_layers, 1);
    c->profiling = 0;
    if (rc) return -1;
    c->pev_phase[c->pev_n] = -1;
    CK(c, cudaEventRecord(c->pev[c->pev_n], c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    for (int i = 0; i < 5; i++) phase_ms[i] = 0.0f;
    if (phase_launches) for (int i = 0; i < 4; i++) phase_launches[i] = 0;
    for (int i = 0; i < c->pev_n; i++) {
        float ms = 0.0f;
        CK(c, cudaEventElapsedTime(&ms, c->pev[i], c->pev[i + 1]));
        const int ph = c->pev_phase[i];
        if (ph >= 0 && ph < 4) {
            phase_ms[ph] += ms;
            if (phase_launches) phase_launches[ph]++;
        }
    }
    CK(c, cudaEventElapsedTime(&phase_ms[4], c->pev[0], c->pev[c->pev_n]));
    return 0;
}

int fomoe_b200_decode_token(fomoe_b200_ctx_t *c, const float *x_in, float *x_out) {
    if (!c || !x_in || !x_out) return -1;
    if (c->cfg.tp_size > 1 && !stack_kernel_usable(c) && !c->allreduce) {
        set_err(c, "decode_token on a tensor-parallel rank needs fomoe_b200_tp_connect (or an all-reduce hook) first");
        return -1;
    }
    CK(c, cudaSetDevice(c->cfg.device));
    const int use_kernel = stack_kernel_usable(c);
    if (!use_kernel && graphs_on(c) && !c->graph_exec && build_graph(c)) return -1;
    const size_t nb = sizeof(float) * c->cfg.n_embd;
    unsigned *slot = (unsigned *)(c->pin + 2 * c->cfg.n_embd); /* the spare slot past max_tokens */
    *slot = (unsigned)c->max_tokens;
    const size_t spare = (size_t)c->max_tokens * c->cfg.n_embd;
    memcpy(c->pin, x_in, nb);
    CK(c, cudaMemcpyAsync(c->tok_in + spare, c->pin, nb, cudaMemcpyHostToDevice, c->stream));
    if (use_kernel) {
        /* one copy in, one launch, one synchronise: the kernel writes the result into the pinned buffer itself */
        if (launch_stack_kernel(c, 0, c->cfg.n_layers, c->max_tokens, 1, c->pin_dev + c->cfg.n_embd)) return -1;
        CK(c, cudaStreamSynchronize(c->stream));
        if (stack_finish(c)) return -1; /* x_out is left untouched */
        memcpy(x_out, c->pin + c->cfg.n_embd, nb);
        return c->trace_fp ? trace_append(c, c->max_tokens, 1, 0, c->cfg.n_layers) : 0;
    }
    CK(c, cudaMemcpyAsync(c->tok_ctr, slot, sizeof(unsigned), cudaMemcpyHostToDevice, c->stream));
    if (graphs_on(c)) {
        CK(c, cudaGraphLaunch(c->graph_exec, c->stream));
        c->launches += (uint64_t)c->graph_nodes;
    } else if (enqueue_stack(c, 0, c->cfg.n_layers, 1))
        return -1;
    CK(c, cudaMemcpyAsync(c->pin + c->cfg.n_embd, c->tok_out + spare, nb, cudaMemcpyDeviceToHost, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    memcpy(x_out, c->pin + c->cfg.n_embd, nb);
    return trace_append(c, c->max_tokens, 1, 0, c->cfg.n_layers);
}

int fomoe_b200_get_routing(fomoe_b200_ctx_t *c, int layer, int *ids, float *scores, int *ids_orig) {
    if (!c || layer < 0 || layer >= c->cfg.n_layers) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    CK(c, cudaStreamSynchronize(c->stream));
    const int k = c->cfg.top_k;
    if (ids) CK(c, cudaMemcpy(ids, c->ids + (size_t)layer * FB_MAX_SLOTS, sizeof(int) * k, cudaMemcpyDeviceToHost));
    if (scores)
        CK(c, cudaMemcpy(scores, c->scores + (size_t)layer * FB_MAX_SLOTS, sizeof(float) * k, cudaMemcpyDeviceToHost));
    if (ids_orig)
        CK(c, cudaMemcpy(ids_orig, c->ids_orig + (size_t)layer * FB_MAX_SLOTS, sizeof(int) * k, cudaMemcpyDeviceToHost));
    return 0;
}

int fomoe_b200_peek(fomoe_b200_ctx_t *c, int what, void *out, uint64_t bytes) {
    if (!c || !out) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    const void *src = NULL;
    uint64_t cap = 0;
    switch (what) {
        case 0: src = c->act; cap = sizeof(float) * FB_MAX_SLOTS * (uint64_t)c->inter_local; break;
        case 1: src = c->q8a; cap = sizeof(fb_q8_entry_t) * FB_MAX_SLOTS * (uint64_t)(c->inter_local / FB_QK); break;
        case 2: src = c->q8h; cap = sizeof(fb_q8_entry_t) * (uint64_t)(c->cfg.n_embd / FB_QK); break;
        case 3: src = c->dots; cap = sizeof(float) * FB_MAX_SLOTS * (uint64_t)c->cfg.n_embd; break;
        case 4: src = c->h; cap = sizeof(float) * (uint64_t)c->cfg.n_embd; break;
        default: set_err(c, "peek: unknown selector %d", what); return -1;
    }
    if (bytes > cap) {
        set_err(c, "peek: %llu bytes requested, %llu available", (unsigned long long)bytes, (unsigned long long)cap);
        return -1;
    }
    CK(c, cudaStreamSynchronize(c->stream));
    CK(c, cudaMemcpy(out, src, bytes, cudaMemcpyDeviceToHost));
    return 0;
}

/* ------------------------------------------------------------------ micro helpers */
int fomoe_b200_matvec(fomoe_b200_ctx_t *c, int type, const void *w, int rows, int cols, const float *x, float *y) {
    if (!c || !w || !x || !y || rows < 1 || cols % FB_QK || cols < FB_QK) return -1;
    const int bpr = cols / FB_QK;
    if ((type != FB_TYPE_Q4_K && type != FB_TYPE_Q5_K && type != FB_TYPE_Q6_K) || !is_pow2(bpr) || bpr > 32) {
        set_err(c, "matvec: unsupported type %d / cols %d", type, cols);
        return -1;
    }
    CK(c, cudaSetDevice(c->cfg.device));
    fb_shard_geom_t g = {type, rows, bpr, 0, 0, bpr, -1};
    const uint64_t wb = ggml_matrix_bytes(type, rows, cols), sb = fb_shard_bytes(type, (uint64_t)rows * bpr);
    uint8_t *dw = NULL, *ds = NULL;
    float *dx = NULL, *dy = NULL;
    fb_q8_entry_t *dq = NULL;
    int rc = -1;
    if (cudaMalloc((void **)&dw, wb) || cudaMalloc((void **)&ds, sb) || cudaMalloc((void **)&dx, sizeof(float) * cols) ||
        cudaMalloc((void **)&dy, sizeof(float) * rows) || cudaMalloc((void **)&dq, sizeof(fb_q8_entry_t) * bpr)) {
        set_err(c, "matvec: allocation failed");
        goto done;
    }
    if (cudaMemcpyAsync(dw, w, wb, cudaMemcpyHostToDevice, c->stream) ||
        cudaMemcpyAsync(dx, x, sizeof(float) * cols, cudaMemcpyHostToDevice, c->stream))
        goto done;
    c->launches += 3;
    if (fb_launch_repack(ds, dw, g, c->stream) || fb_launch_quantize(dq, dx, bpr, c->stream) ||
        fb_launch_matvec(dy, ds, g, dq, grid_tasks(c, (int)fb_n_groups((uint64_t)rows * bpr)), c->stream))
        goto done;
    if (cudaMemcpyAsync(y, dy, sizeof(float) * rows, cudaMemcpyDeviceToHost, c->stream) ||
        cudaStreamSynchronize(c->stream))
        goto done;
    rc = 0;
done:
    if (rc) set_err(c, "matvec failed: %s", cudaGetErrorString(cudaGetLastError()));
    cudaFree(dw); cudaFree(ds); cudaFree(dx); cudaFree(dy); cudaFree(dq);
    return rc;
}

/* ------------------------------------------------------------------ projections in 32-value blocks */
static uint64_t p32_bytes(int type, int rows, int cols) {
    return (uint64_t)rows * (uint64_t)(cols / 32) * (type == FB_TYPE_Q8_0 ? 34u : 17u);
}
static int p32_type_ok(int type) { return type == FB_TYPE_Q8_0 || type == FB_TYPE_MXFP4; }

/* device view of `bytes` bytes at p: p itself when it is memory of this GPU, else a temporary copy (*tmp, to free) */
static const uint8_t *dev_view(fomoe_b200_ctx_t *c, const void *p, uint64_t bytes, void **tmp) {
    struct cudaPointerAttributes at;
    *tmp = NULL;
    if (cudaPointerGetAttributes(&at, p) == cudaSuccess && at.type == cudaMemoryTypeDevice && at.device == c->cfg.device)
        return (const uint8_t *)p;
    cudaGetLastError();
    if (cudaMalloc(tmp, bytes) != cudaSuccess) {
        *tmp = NULL;
        return NULL;
    }
    if (cudaMemcpyAsync(*tmp, p, bytes, cudaMemcpyDefault, c->stream) != cudaSuccess) return NULL;
    return (const uint8_t *)*tmp;
}

int fomoe_b200_proj_matvec_f32(fomoe_b200_ctx_t *c, int type, const void *w, int rows, int cols, const float *x, float *y) {
    if (!c || !w || !x || !y || rows < 1 || cols < 32 || cols % 32 || !p32_type_ok(type)) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    void *tw = NULL, *tx = NULL, *ty = NULL;
    int rc = -1;
    const uint8_t *dw = dev_view(c, w, p32_bytes(type, rows, cols), &tw);
    const float *dx = (const float *)dev_view(c, x, sizeof(float) * (uint64_t)cols, &tx);
    if (!dw || !dx || cudaMalloc(&ty, sizeof(float) * (size_t)rows) != cudaSuccess) goto done;
    c->launches++;
    if (fb_launch_p32_matvec(type, dw, rows, cols, dx, (float *)ty, c->stream)) goto done;
    if (cudaMemcpyAsync(y, ty, sizeof(float) * (size_t)rows, cudaMemcpyDefault, c->stream) || cudaStreamSynchronize(c->stream))
        goto done;
    rc = 0;
done:
    if (rc) set_err(c, "proj_matvec_f32 failed: %s", cudaGetErrorString(cudaGetLastError()));
    cudaFree(tw); cudaFree(tx); cudaFree(ty);
    return rc;
}

int fomoe_b200_shared_ffn_f32(fomoe_b200_ctx_t *c, const void *gate, int gate_type, const void *up, int up_type,
                              const void *down, int down_type, int n_embd, int n_inter, const float *h, float *out) {
    if (!c || !gate || !up || !down || !h || !out || n_embd < 32 || n_embd % 32 || n_inter < 32 || n_inter % 32 ||
        !p32_type_ok(gate_type) || !p32_type_ok(up_type) || !p32_type_ok(down_type))
        return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    void *tg = NULL, *tu = NULL, *td = NULL, *th = NULL, *ta = NULL, *to = NULL;
    int rc = -1;
    const uint8_t *dg = dev_view(c, gate, p32_bytes(gate_type, n_inter, n_embd), &tg);
    const uint8_t *du = dev_view(c, up, p32_bytes(up_type, n_inter, n_embd), &tu);
    const uint8_t *dd = dev_view(c, down, p32_bytes(down_type, n_embd, n_inter), &td);
    const float *dh = (const float *)dev_view(c, h, sizeof(float) * (uint64_t)n_embd, &th);
    if (!dg || !du || !dd || !dh || cudaMalloc(&ta, sizeof(float) * (size_t)n_inter) != cudaSuccess ||
        cudaMalloc(&to, sizeof(float) * (size_t)n_embd) != cudaSuccess)
        goto done;
    c->launches += 2;
    if (fb_launch_p32_gate_up(gate_type, dg, up_type, du, n_inter, n_embd, dh, (float *)ta, c->stream) ||
        fb_launch_p32_matvec(down_type, dd, n_embd, n_inter, (const float *)ta, (float *)to, c->stream))
        goto done;
    if (cudaMemcpyAsync(out, to, sizeof(float) * (size_t)n_embd, cudaMemcpyDefault, c->stream) || cudaStreamSynchronize(c->stream))
        goto done;
    rc = 0;
done:
    if (rc) set_err(c, "shared_ffn_f32 failed: %s", cudaGetErrorString(cudaGetLastError()));
    cudaFree(tg); cudaFree(tu); cudaFree(td); cudaFree(th); cudaFree(ta); cudaFree(to);
    return rc;
}

int fomoe_b200_quantize_q8k(fomoe_b200_ctx_t *c, const float *x, int n, void *out) {
    if (!c || !x || !out || n % FB_QK || n < FB_QK) return -1;
    CK(c, cudaSetDevice(c->cfg.device));
    const int nb = n / FB_QK;
    float *dx = NULL;
    fb_q8_entry_t *dq = NULL, *hq = (fb_q8_entry_t *)malloc(sizeof(fb_q8_entry_t) * (size_t)nb);
    int rc = -1;
    if (!hq || cudaMalloc((void **)&dx, sizeof(float) * n) || cudaMalloc((void **)&dq, sizeof(fb_q8_entry_t) * nb)) goto done;
    if (cudaMemcpyAsync(dx, x, sizeof(float) * n, cudaMemcpyHostToDevice, c->stream)) goto done;
    c->launches++;
    if (fb_launch_quantize(dq, dx, nb, c->stream)) goto done;
    if (cudaMemcpyAsync(hq, dq, sizeof(fb_q8_entry_t) * nb, cudaMemcpyDeviceToHost, c->stream) ||
        cudaStreamSynchronize(c->stream))
        goto done;
    for (int b = 0; b < nb; b++) { /* back to the reference's block_q8_K order: d, qs, bsums (292 B) */
        uint8_t *o = (uint8_t *)out + (size_t)b * 292;
        memcpy(o, &hq[b].d, 4);
        memcpy(o + 4, hq[b].qs, 256);
        memcpy(o + 260, hq[b].bsums, 32);
    }
    rc = 0;
done:
    if (rc) set_err(c, "quantize failed: %s", cudaGetErrorString(cudaGetLastError()));
    cudaFree(dx); cudaFree(dq); free(hq);
    return rc;
}

/* ------------------------------------------------------------------ host-side generator */
void fomoe_b200_synth_matrix(uint64_t seed, int layer, int expert, int matrix, int type, int rows, int cols,
                             void *out) {
    const uint64_t key = fsyn_key(seed, (uint32_t)layer, (uint32_t)expert, (uint32_t)matrix);
    const uint64_t nblk = (uint64_t)rows * (uint64_t)(cols / FB_QK);
    uint8_t *o = (uint8_t *)out;
    for (uint64_t b = 0; b < nblk; b++) {
        if (type == FB_TYPE_Q4_K) {
            uint32_t w[36];
            fsyn_q4k_block(key, b, w);
            memcpy(o + b * FB_Q4K_BLOCK, w, FB_Q4K_BLOCK);
        } else if (type == FB_TYPE_Q5_K) {
            uint32_t w[44];
            fsyn_q5k_block(key, b, w);
            memcpy(o + b * FB_Q5K_BLOCK, w, FB_Q5K_BLOCK);
        } else {
            uint32_t ql[32], qh[16], sc[4];
            uint16_t d;
            fsyn_q6k_block(key, b, ql, qh, sc, &d);
            uint8_t *p = o + b * FB_Q6K_BLOCK;
            memcpy(p, ql, 128);
            memcpy(p + 128, qh, 64);
            memcpy(p + 192, sc, 16);
            memcpy(p + 208, &d, 2);
        }
    }
}

void fomoe_b200_synth_f32(uint64_t seed, int layer, int stream_id, float mean, float std, uint64_t n, float *out) {
    const uint64_t key = fsyn_key(seed, (uint32_t)layer, 0, (uint32_t)stream_id);
    for (uint64_t i = 0; i < n; i++) out[i] = fsyn_f32(key, i, mean, std);
}

/* ======================================================================================
 * Reference GPU surface (include/gpu.h) and the cpu_expert twin, both on a one-layer
 * engine whose "table" is just the experts of the current call.
 * ====================================================================================== */
#define OP_MAX_EXPERTS 10        /* MAX_EXPERTS,        src/gpu_kernels.hip:438-448 */
#define OP_MAX_EMBD 4096         /* MAX_N_EMBD */
#define OP_MAX_INTER 2048        /* MAX_INTERMEDIATE */
#define OP_MAX_STRIDE (12ull << 20)
#define OP_MAX_WORK 16           /* CPU_EXPERT_MAX_WORK, src/cpu_expert.c:12 */

typedef struct {
    fomoe_b200_ctx_t *eng;
    int n_embd, inter;
} op_engine_t;

/* One engine per shape serves every down type: its record slots are sized for the largest block format (Q6_K) and
 * the type of a call's records travels with the call.  (The 397B model alternates Q6_K and Q4_K down projections
 * from layer to layer; an engine per type, rebuilt on every change, would allocate and free on every layer.) */
static int op_engine_get(op_engine_t *o, int n_embd, int inter, int gate_type) {
    if (o->eng && o->n_embd == n_embd && o->inter == inter && o->eng->cfg.gate_type == gate_type) return 0;
    if (o->eng) fomoe_b200_destroy(o->eng);
    o->eng = NULL;
    fomoe_b200_config_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    int dev = 0, down_type = FB_TYPE_Q6_K;
    cudaGetDevice(&dev);
    cfg.device = dev;
    cfg.n_layers = 1;
    cfg.n_embd = n_embd;
    cfg.n_inter = inter;
    cfg.n_experts = OP_MAX_WORK;
    cfg.top_k = FB_MAX_TOPK;
    cfg.has_shared = 0;
    cfg.gate_type = gate_type; /* one type per model in practice: a change rebuilds the engine */
    cfg.down_types = &down_type;
    cfg.tp_rank = 0;
    cfg.tp_size = 1;
    cfg.rms_eps = 1e-6f;
    cfg.car_threshold = 1.0f;
    o->eng = fomoe_b200_create(&cfg);
    if (!o->eng) return -1;
    const char *act = getenv("FOMOE_B200_ACT"); /* "f32": the reference's fp32-activation definition */
    if (act && (!strcmp(act, "f32") || !strcmp(act, "F32"))) o->eng->act_f32 = 1;
    const char *ser = getenv("FOMOE_B200_SERIAL_UPLOAD"); /* comparison arm: a synchronise after every record */
    if (ser && atoi(ser)) o->eng->serial_upload = 1;
    o->n_embd = n_embd;
    o->inter = inter;
    return 0;
}

struct gpu_ctx {
    op_engine_t op;
    fomoe_b200_ctx_t *dec; /* decoder whose routing the statistics calls report (fomoe_b200_gpu_attach), or NULL */
    uint32_t *freq_host;
    int freq_enabled;
};

gpu_ctx_t *gpu_init(void) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
        fprintf(stderr, "gpu_init: no CUDA device\n");
        return NULL;
    }
    if (cudaSetDevice(0) != cudaSuccess) return NULL;
    return (gpu_ctx_t *)calloc(1, sizeof(gpu_ctx_t));
}

void gpu_free(gpu_ctx_t *ctx) {
    if (!ctx) return;
    if (ctx->op.eng) fomoe_b200_destroy(ctx->op.eng);
    free(ctx->freq_host);
    free(ctx);
}

void gpu_register_buffers(gpu_ctx_t *ctx, void **buffers, int n, uint64_t size) {
    (void)ctx;
    for (int i = 0; i < n; i++)
        if (buffers && buffers[i] && cudaHostRegister(buffers[i], size, cudaHostRegisterDefault) != cudaSuccess) {
            cudaGetLastError();
            fprintf(stderr, "gpu_register_buffers: buffer %d not pinned\n", i);
        }
}

void gpu_unregister_buffers(gpu_ctx_t *ctx, void **buffers, int n) {
    (void)ctx;
    for (int i = 0; i < n; i++)
        if (buffers && buffers[i] && cudaHostUnregister(buffers[i]) != cudaSuccess) cudaGetLastError();
}

int gpu_upload_model(gpu_ctx_t *ctx, const void *model) {
    (void)ctx; (void)model;
    fprintf(stderr, "gpu_upload_model: whole-model engine is not part of this library\n");
    return -1;
}
void gpu_set_ram_cache_mb(gpu_ctx_t *ctx, int mb) { (void)ctx; (void)mb; }
void gpu_set_vram_cache_mb(gpu_ctx_t *ctx, int mb) { (void)ctx; (void)mb; }
float *gpu_forward(gpu_ctx_t *ctx, void *model, int token_id, int pos) {
    (void)ctx; (void)model; (void)token_id; (void)pos;
    return NULL;
}
void gpu_reset_state(gpu_ctx_t *ctx) { (void)ctx; }
int gpu_seed_vram_cache(gpu_ctx_t *ctx, void *model, const char *path) {
    (void)ctx; (void)model; (void)path;
    return 0;
}
/* The reference counts expert selections inside its own forward pass (src/gpu_kernels.hip:7832-7835).  The operator
 * gpu_expert_ffn receives its routing from the caller, so there is nothing to count there; the counters of this
 * surface are those of the decoder context attached to it, which routes on the device. */
int fomoe_b200_gpu_attach(gpu_ctx_t *ctx, fomoe_b200_ctx_t *dec) {
    if (!ctx) return -1;
    ctx->dec = dec;
    if (dec && ctx->freq_enabled) return fomoe_b200_enable_expert_freq(dec);
    return 0;
}
void gpu_enable_expert_freq(gpu_ctx_t *ctx) {
    if (!ctx) return;
    ctx->freq_enabled = 1;
    if (ctx->dec) fomoe_b200_enable_expert_freq(ctx->dec);
}
const uint32_t *gpu_get_expert_freq(gpu_ctx_t *ctx) {
    if (!ctx || !ctx->freq_enabled || !ctx->dec || !ctx->dec->freq) return NULL; /* NULL when not enabled, include/gpu.h:52 */
    const size_t n = (size_t)ctx->dec->cfg.n_layers * ctx->dec->cfg.n_experts;
    uint32_t *p = (uint32_t *)realloc(ctx->freq_host, sizeof(uint32_t) * n);
    if (!p) return NULL;
    ctx->freq_host = p;
    if (fomoe_b200_get_expert_freq(ctx->dec, p)) return NULL;
    return p; /* owned by the context: the caller does not free it */
}
void gpu_get_expert_dims(gpu_ctx_t *ctx, int *n_layers, int *n_experts) {
    if (n_layers) *n_layers = (ctx && ctx->dec) ? ctx->dec->cfg.n_layers : 0;
    if (n_experts) *n_experts = (ctx && ctx->dec) ? ctx->dec->cfg.n_experts : 0;
}
void gpu_get_pingpong_relay_stats(gpu_ctx_t *ctx, uint64_t *handoffs, uint64_t *payload_bytes, uint64_t *d2h_bytes,
                                  uint64_t *h2d_bytes, uint64_t *dma_bytes) {
    (void)ctx;
    if (handoffs) *handoffs = 0;
    if (payload_bytes) *payload_bytes = 0;
    if (d2h_bytes) *d2h_bytes = 0;
    if (h2d_bytes) *h2d_bytes = 0;
    if (dma_bytes) *dma_bytes = 0;
}

static int op_types_ok(int gate_type, int up_type, int down_type) {
    return (gate_type == FB_TYPE_Q4_K || gate_type == FB_TYPE_Q6_K) && up_type == gate_type &&
           (down_type == FB_TYPE_Q4_K || down_type == FB_TYPE_Q5_K || down_type == FB_TYPE_Q6_K);
}

int gpu_expert_ffn(gpu_ctx_t *ctx, const float *h, void **expert_buffers, const float *expert_scores, int n_experts,
                   int n_embd, int expert_intermediate, uint64_t expert_gate_size, uint64_t expert_up_size,
                   uint64_t expert_stride, int gate_type, int up_type, int down_type, float *ffn_out) {
    if (!ctx || !h || !expert_buffers || !expert_scores || !ffn_out) return -1;
    if (n_experts < 1 || n_experts > OP_MAX_EXPERTS || n_embd > OP_MAX_EMBD || expert_intermediate > OP_MAX_INTER ||
        expert_stride > OP_MAX_STRIDE || !op_types_ok(gate_type, up_type, down_type))
        return -1;
    if (n_embd % FB_QK || expert_intermediate % FB_QK) return -1;
    if (expert_gate_size != ggml_matrix_bytes(gate_type, expert_intermediate, n_embd) ||
        expert_up_size != ggml_matrix_bytes(up_type, expert_intermediate, n_embd))
        return -1;
    if (op_engine_get(&ctx->op, n_embd, expert_intermediate, gate_type)) return -1;
    fomoe_b200_ctx_t *c = ctx->op.eng;
    int ids[OP_MAX_EXPERTS];
    for (int e = 0; e < n_experts; e++) ids[e] = e;
    if (upload_records(c, n_experts, expert_buffers, NULL, down_type)) return -1;
    return run_routed(c, 0, h, ids, expert_scores, n_experts, 0, 0, ffn_out, 1, down_type);
}

struct b200_expert_ctx {
    op_engine_t op;
    int n_embd, inter;
    float *partial; /* host copy handed out by b200_expert_result */
    int input_valid; /* the hidden state of this layer is already quantised on the device */
    int dirty;       /* device accumulator holds something */
    double total_us;
    int samples;
    cudaEvent_t e0, e1;
    int timing_pending;
};

b200_expert_ctx_t *b200_expert_create(int n_embd, int expert_intermediate) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) return NULL;
    if (n_embd % FB_QK || expert_intermediate % FB_QK || n_embd < FB_QK || expert_intermediate < FB_QK) return NULL;
    b200_expert_ctx_t *x = (b200_expert_ctx_t *)calloc(1, sizeof(*x));
    if (!x) return NULL;
    x->n_embd = n_embd;
    x->inter = expert_intermediate;
    x->partial = (float *)calloc((size_t)n_embd, sizeof(float));
    if (!x->partial || cudaEventCreate(&x->e0) != cudaSuccess || cudaEventCreate(&x->e1) != cudaSuccess) {
        free(x->partial);
        free(x);
        return NULL;
    }
    return x;
}

void b200_expert_free(b200_expert_ctx_t *x) {
    if (!x) return;
    if (x->op.eng) fomoe_b200_destroy(x->op.eng);
    cudaEventDestroy(x->e0);
    cudaEventDestroy(x->e1);
    free(x->partial);
    free(x);
}

void b200_expert_reset(b200_expert_ctx_t *x) {
    if (!x) return;
    x->input_valid = 0;
    x->dirty = 0;
    if (x->op.eng) {
        cudaSetDevice(x->op.eng->cfg.device);
        cudaMemsetAsync(x->op.eng->moe_out, 0, sizeof(float) * (size_t)x->n_embd, x->op.eng->stream);
    }
}

static int expert_batch(b200_expert_ctx_t *x, const float *input, const b200_expert_work_t *work, int n, int accumulate) {
    for (int i = 0; i < n; i++)
        if (!op_types_ok(work[i].gate_type, work[i].up_type, work[i].down_type) ||
            work[i].down_type != work[0].down_type || work[i].gate_type != work[0].gate_type || !work[i].expert_data)
            return -1;
    int had = x->op.eng != NULL;
    float *carry = NULL;
    if (had && x->op.eng->cfg.gate_type != work[0].gate_type) {
        /* the engine is rebuilt for the other gate/up format: what has been accumulated moves over, the quantised
         * input does not */
        if (x->dirty && accumulate) {
            carry = (float *)malloc(sizeof(float) * (size_t)x->n_embd);
            if (!carry) return -1;
            cudaSetDevice(x->op.eng->cfg.device);
            cudaStreamSynchronize(x->op.eng->stream);
            if (cudaMemcpy(carry, x->op.eng->moe_out, sizeof(float) * (size_t)x->n_embd, cudaMemcpyDeviceToHost) != cudaSuccess) {
                free(carry);
                return -1;
            }
        }
        had = 0;
        x->input_valid = 0;
        if (!input) {
            free(carry);
            return -1;
        }
    }
    if (op_engine_get(&x->op, x->n_embd, x->inter, work[0].gate_type)) {
        free(carry);
        return -1;
    }
    fomoe_b200_ctx_t *c = x->op.eng;
    if (carry) {
        cudaMemcpyAsync(c->moe_out, carry, sizeof(float) * (size_t)x->n_embd, cudaMemcpyHostToDevice, c->stream);
        cudaStreamSynchronize(c->stream);
        free(carry);
        had = 1;
        x->dirty = 1;
    }
    if (!had || !x->dirty) cudaMemsetAsync(c->moe_out, 0, sizeof(float) * (size_t)x->n_embd, c->stream);
    int ids[OP_MAX_WORK];
    float sc[OP_MAX_WORK];
    cudaEventRecord(x->e0, c->stream);
    if (upload_records(c, n, NULL, work, work[0].down_type)) return -1;
    for (int i = 0; i < n; i++) {
        ids[i] = i;
        sc[i] = work[i].score;
    }
    /* at most FB_MAX_TOPK experts per launch */
    int done = 0;
    while (done < n) {
        const int m = n - done > FB_MAX_TOPK ? FB_MAX_TOPK : n - done;
        if (run_routed(c, 0, (done == 0 && !x->input_valid) ? input : NULL, ids + done, sc + done, m, 0,
                       accumulate || done > 0, NULL, 0, work[0].down_type))
            return -1;
        x->input_valid = 1;
        done += m;
    }
    cudaEventRecord(x->e1, c->stream);
    x->timing_pending = 1;
    x->dirty = 1;
    return 0;
}

void b200_expert_ffn(b200_expert_ctx_t *x, const void *expert_data, const float *input, float score, int gate_type,
                     int up_type, int down_type, uint64_t expert_gate_size, uint64_t expert_up_size) {
    if (!x || !expert_data || !input) return;
    b200_expert_work_t w = {expert_data, score, gate_type, up_type, down_type, expert_gate_size, expert_up_size};
    if (expert_batch(x, input, &w, 1, 1)) fprintf(stderr, "b200_expert_ffn: unsupported expert or CUDA failure\n");
    b200_expert_wait(x);
}

void b200_expert_submit_async(b200_expert_ctx_t *x, const float *input, const b200_expert_work_t *work, int n_work) {
    if (!x || !input || !work || n_work <= 0) return;
    if (n_work > OP_MAX_WORK) n_work = OP_MAX_WORK; /* src/cpu_expert.c:246 */
    b200_expert_reset(x);                            /* a batch starts from zero, src/cpu_expert.c:141-142 */
    if (expert_batch(x, input, work, n_work, 0)) fprintf(stderr, "b200_expert_submit_async: unsupported expert or CUDA failure\n");
}

void b200_expert_wait(b200_expert_ctx_t *x) {
    if (!x || !x->op.eng) return;
    cudaSetDevice(x->op.eng->cfg.device);
    cudaStreamSynchronize(x->op.eng->stream);
    if (x->timing_pending) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, x->e0, x->e1) == cudaSuccess) {
            x->total_us += 1e3 * ms;
            x->samples++;
        }
        x->timing_pending = 0;
    }
}

float *b200_expert_result(b200_expert_ctx_t *x) {
    if (!x) return NULL;
    if (x->op.eng && x->dirty) {
        b200_expert_wait(x);
        cudaMemcpy(x->partial, x->op.eng->moe_out, sizeof(float) * (size_t)x->n_embd, cudaMemcpyDeviceToHost);
    } else {
        memset(x->partial, 0, sizeof(float) * (size_t)x->n_embd);
    }
    return x->partial;
}

void b200_expert_get_timing(b200_expert_ctx_t *x, double *avg_wakeup_us, double *avg_compute_us, int *samples) {
    if (samples) *samples = x ? x->samples : 0;
    if (avg_wakeup_us) *avg_wakeup_us = 0.0; /* no worker thread to wake: work is enqueued on a stream */
    if (avg_compute_us) *avg_compute_us = (x && x->samples > 0) ? x->total_us / x->samples : 0.0;
}
