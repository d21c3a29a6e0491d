/*
 * fomoe_b200.h -- C ABI of libfomoe_b200.so: fomoe's routed-expert FFN decode path on B200.
 *
 * Three groups of entry points:
 *   1. the reference's own GPU operator surface, same names and signatures
 *      (reference include/gpu.h:13-83), so a build of the reference can link this
 *      library in place of src/gpu_kernels.hip for the expert FFN;
 *   2. a CUDA-backed twin of the reference's CPU expert engine
 *      (reference include/cpu_expert.h:13-62) under the b200_expert_ prefix;
 *   3. extensions for what the reference has no call for: an HBM-resident expert table
 *      (instead of its VRAM/DRAM/NVMe tiers), the on-device router + cache-aware routing,
 *      and the multi-layer decode stack used by the benchmark.
 *
 * Conventions are the reference's: opaque contexts, constructors return NULL on failure,
 * int functions return 0 on success and -1 on failure, diagnostics go to stderr, nothing
 * aborts.  All pointers are HOST pointers unless a comment says "device".  A context is
 * used from one thread at a time.  There is no CPU fallback inside this library: when
 * CUDA is unavailable every constructor returns NULL.
 */
#ifndef FOMOE_B200_H
#define FOMOE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids, reference include/quant_types.h:56-64 */
#define FOMOE_TYPE_Q4_K 12
#define FOMOE_TYPE_Q5_K 13
#define FOMOE_TYPE_Q6_K 14

/* ======================================================================================
 * 1. Reference GPU surface (include/gpu.h).  gpu_expert_ffn is the operator on the hot
 *    path; the tier-management calls are accepted and do nothing because every expert is
 *    resident; gpu_forward / gpu_upload_model belong to the reference's whole-model engine,
 *    which is outside this library: they report failure so the caller takes its own path
 *    (reference src/inference.c:427-432).
 * ====================================================================================== */
typedef struct gpu_ctx gpu_ctx_t;

gpu_ctx_t *gpu_init(void);                                                         /* gpu.h:13 */
void gpu_free(gpu_ctx_t *ctx);                                                     /* gpu.h:16 */
void gpu_register_buffers(gpu_ctx_t *ctx, void **buffers, int n, uint64_t size);   /* gpu.h:19 */
void gpu_unregister_buffers(gpu_ctx_t *ctx, void **buffers, int n);                /* gpu.h:22 */
int gpu_upload_model(gpu_ctx_t *ctx, const void *model);                           /* gpu.h:26, returns -1 */
void gpu_set_ram_cache_mb(gpu_ctx_t *ctx, int mb);                                 /* gpu.h:30, no-op */
void gpu_set_vram_cache_mb(gpu_ctx_t *ctx, int mb);                                /* gpu.h:34, no-op */
float *gpu_forward(gpu_ctx_t *ctx, void *model, int token_id, int pos);            /* gpu.h:38, returns NULL */
void gpu_reset_state(gpu_ctx_t *ctx);                                              /* gpu.h:41, no-op */
int gpu_seed_vram_cache(gpu_ctx_t *ctx, void *model, const char *freq_profile_path); /* gpu.h:46, returns 0 */
void gpu_enable_expert_freq(gpu_ctx_t *ctx);                                       /* gpu.h:50 */
const uint32_t *gpu_get_expert_freq(gpu_ctx_t *ctx);                               /* gpu.h:54: [n_layers * n_experts]
                                                                                       counters of the attached decoder
                                                                                       (fomoe_b200_gpu_attach), NULL when
                                                                                       not enabled; not to be freed */
void gpu_get_expert_dims(gpu_ctx_t *ctx, int *n_layers, int *n_experts);           /* gpu.h:57: of the attached decoder */
void gpu_get_pingpong_relay_stats(gpu_ctx_t *ctx, uint64_t *handoffs, uint64_t *payload_bytes,
                                  uint64_t *d2h_bytes, uint64_t *h2d_bytes, uint64_t *dma_bytes); /* gpu.h:61, zeros */

/* Batched expert FFN: ffn_out[n_embd] = sum_e expert_scores[e] * FFN_e(h).
 * Same arguments as reference gpu.h:70-83.  expert_buffers[e] points at one expert record
 * in ggml byte order (gate | up | down back to back).  Returns 0, or -1 for shapes/types
 * outside the supported set (the reference's limits, src/gpu_kernels.hip:8393-8403, plus:
 * gate and up must share one type, Q4_K or Q6_K; down Q4_K, Q5_K or Q6_K), in which case the caller falls back
 * (src/inference.c:551).  Activations are quantised to Q8_K as in src/cpu_expert.c.
 * expert_buffers[e] may be host memory (staged: two staging buffers filled on a copy stream, the host does not
 * wait between records) or memory of the current GPU (regrouped where it lies, no staging). */
int gpu_expert_ffn(gpu_ctx_t *ctx, const float *h, void **expert_buffers, const float *expert_scores,
                   int n_experts, int n_embd, int expert_intermediate, uint64_t expert_gate_size,
                   uint64_t expert_up_size, uint64_t expert_stride, int gate_type, int up_type, int down_type,
                   float *ffn_out);

/* ======================================================================================
 * 2. CUDA twin of the reference CPU expert engine (include/cpu_expert.h).
 * ====================================================================================== */
typedef struct b200_expert_ctx b200_expert_ctx_t;

typedef struct { /* cpu_expert.h:13-18 */
    const void *expert_data;
    float score;
    int gate_type, up_type, down_type;
    uint64_t expert_gate_size, expert_up_size;
} b200_expert_work_t;

b200_expert_ctx_t *b200_expert_create(int n_embd, int expert_intermediate);        /* cpu_expert.h:23 */
void b200_expert_free(b200_expert_ctx_t *ctx);                                     /* cpu_expert.h:26 */
void b200_expert_reset(b200_expert_ctx_t *ctx);                                    /* cpu_expert.h:29 */
void b200_expert_ffn(b200_expert_ctx_t *ctx, const void *expert_data, const float *input, float score,
                     int gate_type, int up_type, int down_type, uint64_t expert_gate_size,
                     uint64_t expert_up_size);                                      /* cpu_expert.h:39 */
void b200_expert_submit_async(b200_expert_ctx_t *ctx, const float *input, const b200_expert_work_t *work,
                              int n_work);                                          /* cpu_expert.h:50 */
void b200_expert_wait(b200_expert_ctx_t *ctx);                                     /* cpu_expert.h:55 */
float *b200_expert_result(b200_expert_ctx_t *ctx);                                 /* cpu_expert.h:59 */
void b200_expert_get_timing(b200_expert_ctx_t *ctx, double *avg_wakeup_us, double *avg_compute_us,
                            int *samples);                                          /* cpu_expert.h:62 */

/* ======================================================================================
 * 3. Extensions: resident expert table, on-device routing, decode stack.
 * ====================================================================================== */
typedef struct fomoe_b200_ctx fomoe_b200_ctx_t;

typedef struct {
    int device;              /* CUDA device ordinal */
    int n_layers;
    int n_embd;              /* hidden size, multiple of 256, <= 8192 */
    int n_inter;             /* expert intermediate size, multiple of 256; tp_size divides n_inter/256, or is twice it */
    int n_experts;           /* routed experts per layer, <= 512 */
    int top_k;               /* experts used per token, <= 15 */
    int has_shared;          /* 1: one shared expert per layer (record index n_experts) */
    int gate_type;           /* gate and up type: FOMOE_TYPE_Q4_K, or FOMOE_TYPE_Q6_K (served by the per-phase kernels;
                                the persistent stack kernel and the bulk-copy variants take Q4_K) */
    const int *down_types;   /* [n_layers] FOMOE_TYPE_Q4_K / FOMOE_TYPE_Q5_K / FOMOE_TYPE_Q6_K; NULL = all Q6_K */
    int tp_rank, tp_size;    /* tensor parallelism over the intermediate dimension, tp_size <= 8.  With W = n_inter/256
                                windows: tp_size dividing W gives every rank W/tp_size whole windows; tp_size == 2 W
                                (8 ranks at n_inter 1024) gives ranks 2p and 2p+1 window p together: both compute its
                                gate/up rows, each owns one 128-column half of the down projection */
    float rms_eps;
    float car_threshold;     /* CAR runs when 0 < threshold < 1 (reference src/car.c:68, gpu_kernels.hip:7170) */
    int car_dampen;          /* 1: substitute weight = original weight * ratio, no renormalise */
    int max_tokens;          /* capacity of the device-resident token buffers (0 = 1) */
} fomoe_b200_config_t;

fomoe_b200_ctx_t *fomoe_b200_create(const fomoe_b200_config_t *cfg);
void fomoe_b200_destroy(fomoe_b200_ctx_t *ctx);
const char *fomoe_b200_last_error(fomoe_b200_ctx_t *ctx);
/* What went wrong on the device since the last call of this function: 0 nothing, 1 a kernel met an expert id
 * outside the table, 2 the stack kernel gave a bounded wait up (the run that met it has already returned -1 and left
 * its output buffer untouched).  Reading clears it: after a failure, a later successful run reports 0 again. */
int fomoe_b200_status(fomoe_b200_ctx_t *ctx);
/* bytes of one expert record in the reference's ggml order (gate | up | down), full (unsharded) */
uint64_t fomoe_b200_record_bytes(fomoe_b200_ctx_t *ctx, int layer);
/* bytes this rank holds in HBM for the table */
uint64_t fomoe_b200_table_bytes(fomoe_b200_ctx_t *ctx);

/* Fill table, routers, residuals and norm weights of every layer on the device from `seed`
 * (generator: fomoe_b200_synth_* below produce the same bytes on the host). */
int fomoe_b200_table_generate(fomoe_b200_ctx_t *ctx, uint64_t seed);
/* Upload one expert record in ggml order (expert == n_experts addresses the shared expert). */
int fomoe_b200_table_upload(fomoe_b200_ctx_t *ctx, int layer, int expert, const void *record);
/* Which of the reference's two definitions of the expert FFN the context computes.  FOMOE_B200_ACT_Q8K (default):
 * activations quantised to Q8_K int8 blocks, integer dots -- src/cpu_expert.c, the reference's CPU expert engine.
 * FOMOE_B200_ACT_F32: fp32 activations against dequantised weights -- the reference's CPU forward pass without
 * cpu_expert (src/inference.c:556-575, dots src/quant.c:109-143, 177-212, 249-262) and, up to summation order, its
 * GPU kernels.  The two differ by a few percent of the layer output on the same inputs.  The fp32 mode runs on
 * the per-phase kernels (it is the parity path for that definition, not a tuned one); the environment variable
 * FOMOE_B200_ACT=f32 selects it for the gpu_expert_ffn / b200_expert_* surfaces. */
#define FOMOE_B200_ACT_Q8K 0
#define FOMOE_B200_ACT_F32 1
int fomoe_b200_set_act_mode(fomoe_b200_ctx_t *ctx, int mode);
/* Optional scalar gate of the shared expert (src/inference.c:586-592, include/model.h shared_expert_gate): with a
 * vector w[n_embd] uploaded, the shared expert's output is multiplied by sigmoid(h . w) before it is added to the
 * routed sum; NULL removes the gate again (the default: weight 1). */
int fomoe_b200_shared_gate_upload(fomoe_b200_ctx_t *ctx, int layer, const float *w);
/* Fill the routed experts of the table from an expert store file of the reference (".qmoe",
 * include/expert_store.h:9-40, written by tools/prepare_experts.c): store layers first_store_layer ..
 * first_store_layer + n_layers - 1.  Header and per-layer down types must match the configuration; the shared
 * expert (not part of such files) is left alone.  Returns the number of experts loaded or -1. */
int fomoe_b200_table_load_qmoe(fomoe_b200_ctx_t *ctx, const char *path, int first_store_layer);
/* The configuration a context was created with (down_types points at the context's own copy). */
const fomoe_b200_config_t *fomoe_b200_get_config(fomoe_b200_ctx_t *ctx);
/* Fill a context from a GGUF model file (the container the reference reads its model from, include/gguf.h:6-145),
 * blocks first_block .. first_block + n_layers - 1: the router (blk.N.ffn_gate_inp.weight, F32/F16/BF16), the routed
 * experts cut out of the stacked tensors blk.N.ffn_{gate,up,down}_exps.weight (as tools/prepare_experts.c:262-291
 * cuts them into .qmoe records; types and shapes must be the context's), the shared expert
 * (blk.N.ffn_{gate,up,down}_shexp.weight, when it is stored in the experts' formats) with its optional scalar gate
 * (blk.N.ffn_gate_inp_shexp.weight), and the RMSNorm weight in front of the block (blk.N.post_attention_norm.weight
 * or blk.N.ffn_norm.weight, src/model.c:277-283).  One file (no -0000i-of-N splits).  Returns the number of layers
 * loaded or -1 (reason on stderr). */
int fomoe_b200_load_gguf(fomoe_b200_ctx_t *ctx, const char *path, int first_block);
/* Host-only look-up in a GGUF file (no GPU involved): type (ggml id), dims[4] (fastest first, unused = 1) and byte
 * size of tensor `name`; with buf != NULL its bytes as well.  0, or -1 when the file or the tensor is not there, the
 * type is one this library has no use for, or buf is too small. */
int fomoe_b200_gguf_tensor(const char *path, const char *name, int *type, int64_t *dims, uint64_t *nbytes, void *buf,
                           uint64_t buf_bytes);
/* Read this rank's shard of one matrix (0 gate, 1 up, 2 down) back in ggml order / as fp32. */
int fomoe_b200_table_export(fomoe_b200_ctx_t *ctx, int layer, int expert, int matrix, void *ggml_out);
int fomoe_b200_table_dequant(fomoe_b200_ctx_t *ctx, int layer, int expert, int matrix, float *out);
int fomoe_b200_router_upload(fomoe_b200_ctx_t *ctx, int layer, const float *w);
int fomoe_b200_glue_upload(fomoe_b200_ctx_t *ctx, int layer, const float *resid, const float *normw);
int fomoe_b200_set_resident_mask(fomoe_b200_ctx_t *ctx, int layer, const uint32_t *mask /* [16] or NULL */);
int fomoe_b200_set_car(fomoe_b200_ctx_t *ctx, float threshold, int dampen);

/* One MoE block on an already normalised hidden state: route on the device, run the selected
 * experts and the shared expert, return out[n_embd] (this rank's partial when tp_size > 1).
 * ids_out / scores_out ([top_k], optional) receive the routing after CAR, ids_orig_out the
 * top-k before CAR, all_scores_out [n_experts] the softmax. */
int fomoe_b200_moe_layer(fomoe_b200_ctx_t *ctx, int layer, const float *h, float *out, int *ids_out,
                         float *scores_out, int *ids_orig_out, float *all_scores_out);
/* Same with routing supplied by the caller (n <= top_k experts of `layer`). */
int fomoe_b200_moe_layer_routed(fomoe_b200_ctx_t *ctx, int layer, const float *h, const int *ids,
                                const float *scores, int n, float *out);
/* Decode stack, layers [l0, l1): x += resid_l; h = rmsnorm(x) * normw_l; x += moe_l(h).
 * Host in, host out; copies are part of the call. */
int fomoe_b200_stack_run(fomoe_b200_ctx_t *ctx, const float *x_in, int l0, int l1, float *x_out);
/* Device-resident variant for throughput: tokens are uploaded once, then `count` tokens run
 * back to back through all layers without touching the host; elapsed_ms (optional) is the
 * CUDA-event time of the run on the library's stream. */
int fomoe_b200_tokens_upload(fomoe_b200_ctx_t *ctx, int first, int count, const float *x);
int fomoe_b200_tokens_run(fomoe_b200_ctx_t *ctx, int first, int count, float *elapsed_ms);
int fomoe_b200_tokens_download(fomoe_b200_ctx_t *ctx, int first, int count, float *x_out);
/* One token, host to host, through every layer as one graph launch: pinned H2D of x_in, the stack,
 * pinned D2H of the result, one synchronise.  This is the end-to-end call. */
int fomoe_b200_decode_token(fomoe_b200_ctx_t *ctx, const float *x_in, float *x_out);
/* Like tokens_run but with plain launches bracketed by CUDA events per kernel; phase_ms[5] receives
 * the summed device time of prologue, router, gate/up, down kernels and the whole run;
 * phase_launches[4] the number of launches of each. */
int fomoe_b200_tokens_profile(fomoe_b200_ctx_t *ctx, int first, int count, float *phase_ms, int *phase_launches);
/* Routing of the most recent token at `layer`. */
int fomoe_b200_get_routing(fomoe_b200_ctx_t *ctx, int layer, int *ids, float *scores, int *ids_orig);
/* Routing trace in the reference's file format (32-byte header, one packed record per layer and token: the top-k
 * before and after cache-aware routing with their weights and a source code per slot; src/gpu_kernels.hip:451-484,
 * read by tools/read_trace.py).  While a trace is open every token that stack_run (whole stack), tokens_run or
 * decode_token runs is appended.  Source codes: 0 expert marked resident (or no mask set), 2 not resident (what the
 * reference would fetch from NVMe; here it is in HBM like every other expert), 3 substituted by CAR, 4 weight zero. */
int fomoe_b200_routing_trace_open(fomoe_b200_ctx_t *ctx, const char *path);
int fomoe_b200_routing_trace_close(fomoe_b200_ctx_t *ctx);
/* Histogram of routed expert ids before substitution (the reference: include/gpu.h:50-57): enable, then read
 * out[n_layers * n_experts].  fomoe_b200_gpu_attach makes gpu_enable_expert_freq / gpu_get_expert_freq /
 * gpu_get_expert_dims of a gpu_ctx_t report this decoder. */
int fomoe_b200_enable_expert_freq(fomoe_b200_ctx_t *ctx);
int fomoe_b200_get_expert_freq(fomoe_b200_ctx_t *ctx, uint32_t *out);
int fomoe_b200_gpu_attach(gpu_ctx_t *gpu, fomoe_b200_ctx_t *decoder);
/* Counters since creation: CAR substitutions, kernels launched by this library. */
uint64_t fomoe_b200_substitutions(fomoe_b200_ctx_t *ctx);
uint64_t fomoe_b200_kernel_launches(fomoe_b200_ctx_t *ctx);
/* The same for ranks that live in ONE process (one context per GPU, as the reference drives its two GPUs from one
 * process, src/tp.hip): the receive buffers are exchanged as plain device pointers; the caller enables peer access
 * between the devices (cudaDeviceEnablePeerAccess). */
void *fomoe_b200_tp_recv_ptr(fomoe_b200_ctx_t *ctx);
int fomoe_b200_tp_connect_ptrs(fomoe_b200_ctx_t *ctx, void *const *recv_ptrs /* tp_size pointers, rank order */);
/* cudaDeviceEnablePeerAccess from this context's device to peer_device (already enabled is fine). */
int fomoe_b200_tp_enable_peer(fomoe_b200_ctx_t *ctx, int peer_device);
/* Host-side stand-in for a rank (diagnostics, tests, a supervisor that lost a rank): writes partial[n_embd]
 * (NULL = zeros) into this context's receive buffer as rank src_rank's contribution to the layer-token `ahead`
 * (>= 1) layer-tokens after the last one launched. */
int fomoe_b200_tp_inject(fomoe_b200_ctx_t *ctx, int src_rank, const float *partial, unsigned ahead);
/* Every wait of the stack kernel on another block or rank gives up after `polls` polls (0 = the default, about
 * four million: seconds), sets status 2 ("bounded wait ran out") and lets the kernel return; a rank whose peer
 * has gone away therefore reports instead of hanging: the call returns -1, fomoe_b200_status says 2, the kernel's
 * flags are re-armed, and the context stays usable.  Every rank must have made the same calls (a launch advances the
 * generation numbers of the exchange on the rank that made it, finished or not). */
int fomoe_b200_set_wait_limit(fomoe_b200_ctx_t *ctx, unsigned polls);
/* Tensor parallelism with the CALLER's collective instead of the fused exchange (the reference's arrangement:
 * kernels per phase and tp_allreduce_sum between them, include/tp.h:53-79).  With a hook installed and the per-phase
 * kernels selected (fomoe_b200_set_variant 0 or 1), the hook is called once per layer, after the down projection
 * has been enqueued, with this rank's partial block output (device memory, n floats) and the CUDA stream the
 * library works on; it must enqueue an in-place sum over all ranks on that stream (e.g. ncclAllReduce) and return 0.
 * CUDA-graph replay is off while a hook is installed.  The benchmark uses it for its NCCL comparison arm. */
typedef int (*fomoe_b200_allreduce_fn)(void *user, float *partial_dev, int n, void *cuda_stream);
int fomoe_b200_set_allreduce(fomoe_b200_ctx_t *ctx, fomoe_b200_allreduce_fn fn, void *user);
/* The cudaStream_t every call of this context enqueues on. */
void *fomoe_b200_stream(fomoe_b200_ctx_t *ctx);
/* Tensor parallelism over the expert intermediate dimension, one process per GPU (tp_rank / tp_size of the
 * configuration).  Each rank exports a 64-byte handle of its receive buffer, the caller gathers the handles of all
 * ranks (rank order) and gives them to every rank; after that stack_run / tokens_run / decode_token run on all ranks
 * together, each call made by every rank with the same arguments, and return the full (summed) result on every
 * rank.  Replaces the reference's host-staged tp_allreduce_sum (include/tp.h:53-79) by stores into the peers'
 * memory from inside the kernel. */
int fomoe_b200_tp_export(fomoe_b200_ctx_t *ctx, void *handle64);
int fomoe_b200_tp_connect(fomoe_b200_ctx_t *ctx, const void *handles /* tp_size x 64 bytes */);
/* Profiling aid for the persistent stack kernel: record up to `cap` %globaltimer stamps of block `cta` at its
 * phase boundaries during the following runs (cap 0 = off; cta < 0 = every block, `cap` stamps each, block-major);
 * trace_read copies the first n out.  Each word is
 * (index << 56) | nanoseconds; index 0 layer top, 1 previous barrier joined, 2 RMSNorm/Q8_K done, 3 router rows
 * done, 4 logits received, 5 expert ids known (first gate/up weights requested), 6 gate/up done, 7 activation barrier
 * passed, 8 down done. */
int fomoe_b200_trace_enable(fomoe_b200_ctx_t *ctx, int cap, int cta);
int fomoe_b200_trace_read(fomoe_b200_ctx_t *ctx, unsigned long long *out, int n);
/* Execution variant: 2 (default) the persistent stack kernel runs whole tokens (stack_run, tokens_run,
 * decode_token) and per-phase kernels serve the single-layer calls; 0 per-phase kernels with plain
 * coalesced loads everywhere; 1 per-phase kernels with bulk-copy shared-memory rings. */
int fomoe_b200_set_variant(fomoe_b200_ctx_t *ctx, int variant);
/* For the per-phase variants: 1 replays each token as one CUDA graph (default), 0 plain stream launches. */
int fomoe_b200_set_graphs(fomoe_b200_ctx_t *ctx, int enable);

/* Copy an intermediate of the most recent layer call to the host (parity tests look inside the
 * block): what = 0 act float[n_slots][inter_local]; 1 quantised act, 304-byte entries
 * {int8 qs[256]; int16 bsums[16]; float d; pad[12]} [n_slots][inter_local/256]; 2 quantised hidden
 * state, same entries [n_embd/256]; 3 per-expert down outputs float[n_slots][n_embd];
 * 4 normalised hidden state float[n_embd]. */
int fomoe_b200_peek(fomoe_b200_ctx_t *ctx, int what, void *out, uint64_t bytes);

/* Microbenchmark / parity helpers: y[rows] = W[rows x cols] . Q8_K(x), W given in ggml order. */
int fomoe_b200_matvec(fomoe_b200_ctx_t *ctx, int type, const void *w_ggml, int rows, int cols, const float *x,
                      float *y);
/* Projections stored in 32-value blocks -- Q8_0 (type 8) and MXFP4 (type 39), the types some models keep their
 * shared expert in -- on fp32 activations, the only form the reference has for them (src/quant.c:266-337 through
 * mat_vec_mul, src/tensor.c:158-171; its GPU kernel: src/gpu_kernels.hip:2070-2103).  Weights in ggml order; a
 * weight or activation pointer may be host memory (copied for the call) or memory of the context's GPU (used where
 * it lies); results go to the host.
 *   proj_matvec_f32: y[rows] = W[rows x cols] x.
 *   shared_ffn_f32:  out[n_embd] = down (silu(gate h) * (up h)), the reference's shared_expert_ffn
 *                    (src/inference.c:361-374); each matrix with its own type.
 * Return 0, or -1 for other types / shapes that are not multiples of 32. */
#define FOMOE_TYPE_Q8_0 8
#define FOMOE_TYPE_MXFP4 39
int fomoe_b200_proj_matvec_f32(fomoe_b200_ctx_t *ctx, int type, const void *w_ggml, int rows, int cols, const float *x,
                               float *y);
int fomoe_b200_shared_ffn_f32(fomoe_b200_ctx_t *ctx, const void *gate, int gate_type, const void *up, int up_type,
                              const void *down, int down_type, int n_embd, int n_inter, const float *h, float *out);
/* y[rows] = W[rows x cols] . Q8_K(x) with NO allocation of any kind.  (No counterpart in the reference: added for
 * callers that cannot call cudaMalloc while they run, such as a serving loop whose device memory was all handed out
 * at start-up or a latency-critical path that must not take cudaMalloc's device synchronisation.)
 * w_ggml_dev (ggml-ordered blocks, type Q4_K, Q5_K or Q6_K), x_dev and y_dev are DEVICE pointers supplied by the caller;
 * the kernels are enqueued on `stream` (a cudaStream_t, NULL = default stream) of the current device and the call
 * does not synchronise.  The two temporaries fomoe_b200_matvec allocates per call live in a fixed array inside the
 * library instead, which limits the matrix to 4 MiB of quantised weights (e.g. 1024 x 4096 Q4_K, 4096 x 1024 Q6_K)
 * and 8192 columns; larger requests return -1 with a message.  Every call on a device shares that array: calls
 * that may overlap on the GPU race, calls on one stream do not.  The first call on a device looks the array's
 * address up; make that call before starting any stream capture.  Returns 0 or -1. */
int fomoe_b200_matvec_noalloc(int type, const void *w_ggml_dev, int rows, int cols, const float *x_dev, float *y_dev,
                              void *stream);
int fomoe_b200_quantize_q8k(fomoe_b200_ctx_t *ctx, const float *x, int n, void *q8k_out /* n/256 * 292 B, reference block_q8_K */);

/* ======================================================================================
 * 4. Batched routed-expert FFN: many tokens per call (prefill, or decode of many sequences) on the tensor cores.
 *    No counterpart in the reference, whose expert kernels are batch-1 only (src/gpu_kernels.hip:1320-1384) and whose
 *    operator takes one hidden state (include/gpu.h:70-83); the definition computed is src/cpu_expert.c applied to
 *    every token.  Q4_K gate, up and down.  Tokens are bucketed by expert on the device; each (expert, 128-row tile)
 *    is one tcgen05 tile with the weights dequantised to fp16 on their way from HBM.
 * ====================================================================================== */
typedef struct fomoe_b200_batch fomoe_b200_batch_t;

typedef struct {
    int device;
    int n_layers;
    int n_embd;      /* multiple of 256 (and so of 128), <= 8192 */
    int n_inter;     /* multiple of 256, <= 8192 */
    int n_experts;   /* <= 512 */
    int top_k;       /* <= 16 */
    int has_shared;
    int max_tokens;  /* tokens per call, at most */
    float rms_eps;
    int tp_rank;     /* tensor parallel over the intermediate dimension, as the decode path shards it: rank r of */
    int tp_size;     /* tp_size (0 = 1; n_inter a multiple of 256 tp_size) holds rows [r I/N, (r+1) I/N) of gate and up
                        and the same columns of down */
} fomoe_b200_batch_config_t;

fomoe_b200_batch_t *fomoe_b200_batch_create(const fomoe_b200_batch_config_t *cfg);
void fomoe_b200_batch_destroy(fomoe_b200_batch_t *b);
const char *fomoe_b200_batch_last_error(fomoe_b200_batch_t *b);
int fomoe_b200_batch_status(fomoe_b200_batch_t *b);             /* 0 ok, 1 bad expert id, 2 bounded wait ran out; reading clears */
uint64_t fomoe_b200_batch_table_bytes(fomoe_b200_batch_t *b);
uint64_t fomoe_b200_batch_kernel_launches(fomoe_b200_batch_t *b);
/* Experts, residuals and norm weights of every layer from `seed` (the same bytes as fomoe_b200_synth_matrix makes on
 * the host); with_logits: also seeded router logits N(0,1) for max_tokens tokens per layer, as the batched
 * benchmark configuration draws them (fomoe_b200_batch_synth_logits gives the host copy). */
int fomoe_b200_batch_generate(fomoe_b200_batch_t *b, uint64_t seed, int with_logits);
/* One expert record in ggml order (gate | up | down, all Q4_K); expert == n_experts is the shared expert. */
int fomoe_b200_batch_upload(fomoe_b200_batch_t *b, int layer, int expert, const void *record);
int fomoe_b200_batch_export(fomoe_b200_batch_t *b, int layer, int expert, void *record_out);
/* One MoE block on n_tokens normalised hidden states h[n_tokens][n_embd] with router logits[n_tokens][n_experts]
 * given by the caller: softmax, ordered top-k, renormalise, experts + shared expert; out[n_tokens][n_embd];
 * ids_out / scores_out [n_tokens][top_k] optional. */
int fomoe_b200_batch_moe_layer(fomoe_b200_batch_t *b, int layer, int n_tokens, const float *h, const float *logits,
                               float *out, int *ids_out, float *scores_out);
/* Stack on device-resident tokens: upload x[n_tokens][n_embd]; layers [l0, l1): x += resid_l; h = rmsnorm(x) normw_l;
 * x += moe_l(h, generated logits of layer l); download.  elapsed_ms: CUDA-event time on the library's stream. */
int fomoe_b200_batch_tokens_upload(fomoe_b200_batch_t *b, int n_tokens, const float *x);
int fomoe_b200_batch_stack_run(fomoe_b200_batch_t *b, int n_tokens, int l0, int l1, float *elapsed_ms);
int fomoe_b200_batch_tokens_download(fomoe_b200_batch_t *b, int n_tokens, float *x_out);
/* Routing of the most recent layer call, and how many pairs every expert received (n_experts + has_shared counts). */
int fomoe_b200_batch_get_routing(fomoe_b200_batch_t *b, int n_tokens, int *ids, float *scores, int *counts);
/* Profiling aid: on = 1 starts counting the clock cycles block 0 of the two grouped-GEMM kernels spends waiting, per
 * role; on = 0 copies the 16 counters out (0..7 down pass, 8..15 gate/up pass: copy thread, producers x3, MMA thread
 * x2, epilogue, the block's whole run time) and stops. */
/* Tensor parallel: every layer ends with the sum of the ranks' partial block outputs, [n_tokens][n_embd] floats
 * (the reference's tp_allreduce_sum, include/tp.h:53-79, for a whole batch).  The caller supplies the collective
 * (NCCL, MPI, ...): it is called once per layer with the partial output on the device and the library's stream, must
 * enqueue an in-place sum over the ranks on that stream and return 0.  Without one installed a tensor-parallel rank
 * returns its partial output (tests sum them on the host).  upload takes whole ggml records on every rank and keeps
 * this rank's part; export returns this rank's shard (gate rows | up rows | down columns, ggml block order). */
int fomoe_b200_batch_set_allreduce(fomoe_b200_batch_t *b, fomoe_b200_allreduce_fn fn, void *user);
int fomoe_b200_batch_wait_profile(fomoe_b200_batch_t *b, int on, unsigned long long *out);
void fomoe_b200_batch_synth_logits(uint64_t seed, int layer, int max_tokens, int n_experts, int n_tokens, float *out);

/* Host-side synthetic generator (same bytes as fomoe_b200_table_generate puts on the device). */
void fomoe_b200_synth_matrix(uint64_t seed, int layer, int expert, int matrix, int type, int rows, int cols,
                             void *ggml_out);
void fomoe_b200_synth_f32(uint64_t seed, int layer, int stream_id, float mean, float std, uint64_t n, float *out);
#define FOMOE_STREAM_ROUTER 3
#define FOMOE_STREAM_RESID 4
#define FOMOE_STREAM_NORMW 5
#define FOMOE_STREAM_HIDDEN 6
/* distribution parameters table_generate uses */
#define FOMOE_ROUTER_STD 0.02f
#define FOMOE_RESID_STD 1.0f
#define FOMOE_NORMW_MEAN 1.0f
#define FOMOE_NORMW_STD 0.1f

#ifdef __cplusplus
}
#endif
#endif
