/*
 * ref_driver.c -- glue over the REFERENCE's own API (TEST INFRASTRUCTURE ONLY).
 *
 * Compiled together with the reference's unmodified C files (found at build
 * time, never copied) into oracle/_ref/libfomoe_ref.so.  Nothing here does
 * arithmetic of its own: it only composes reference calls the way the
 * reference's callers do, so the result can be used as ground truth:
 *   router+softmax+top-k+renorm   src/inference.c:486-502
 *   residency classify + CAR      src/gpu_kernels.hip:7097-7187
 *   routed experts                src/cpu_expert.c:226-240 (reset + ffn per expert)
 *   shared expert, added after    src/inference.c:582-596 (through cpu_expert_ffn, weight 1)
 */
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "car.h"
#include "cpu_expert.h"
#include "expert_cache.h"
#include "quant.h"
#include "tensor.h"

int refdrv_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void refdrv_set_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* all_scores[n_experts] <- softmax(W h); ids/scores <- renormalised top-k; then CAR
 * against a one-tier residency mask (NULL = everything resident). Returns substitutions. */
int refdrv_route(const float *router_w, const float *h, int n_experts, int n_embd, int k,
                 const uint32_t *mask, float threshold, int dampen, float *all_scores, int *ids,
                 float *scores) {
    mat_vec_mul(all_scores, router_w, GGML_TYPE_F32, h, n_experts, n_embd);
    softmax(all_scores, n_experts);
    top_k(all_scores, n_experts, k, ids, scores);
    float sum = 0.0f;
    for (int i = 0; i < k; i++) sum += scores[i];
    if (sum > 0.0f) {
        float inv = 1.0f / sum;
        for (int i = 0; i < k; i++) scores[i] *= inv;
    }
    if (!mask || !(threshold > 0.0f)) return 0;

    vram_cache_t vc;
    if (vram_cache_init(&vc, 1, n_experts, n_experts, 1024) != 0) return -1;
    int slot = 0;
    for (int e = 0; e < n_experts; e++)
        if ((mask[e >> 5] >> (e & 31)) & 1u) vc.map[e] = slot++;
    int unc[16], n_unc = 0;
    for (int i = 0; i < k; i++)
        if (vc.map[ids[i]] < 0) unc[n_unc++] = i;
    int subs = 0;
    if (n_unc > 0) {
        car_state_t car;
        car_init(&car, threshold);
        car.skip_renorm = dampen ? true : false;
        int vsi[16], vss[16], nv = 0, rsi[16], rss[16], nr = 0;
        subs = car_evaluate(&car, 0, -1, ids, scores, k, all_scores, n_experts, &vc, NULL, NULL, unc,
                            &n_unc, vsi, vss, &nv, NULL, NULL, NULL, rsi, rss, &nr);
    }
    vram_cache_free(&vc);
    return subs;
}

/* Raw car_evaluate on caller-provided selections (for the reference's own CAR scenarios,
 * src/test_v2.c:201-291): vram_ids / ram_ids list the experts cached in each tier. */
int refdrv_car_case(float threshold, int dampen, int *ids, float *scores, int k, const float *all_scores,
                    int n_experts, const int *vram_ids, int n_vram, const int *ram_ids, int n_ram,
                    int *n_uncached_out, int *vram_sub_idx_out, int *n_vram_subs_out) {
    vram_cache_t vc;
    ram_cache_t rc;
    vram_cache_init(&vc, 1, n_experts, n_vram > 0 ? n_vram : 1, 1024);
    ram_cache_init(&rc, 1, n_experts, n_ram > 0 ? n_ram : 1, 1024);
    for (int i = 0; i < n_vram; i++) vram_cache_alloc_slot(&vc, 0, vram_ids[i]);
    for (int i = 0; i < n_ram; i++) ram_cache_alloc_slot(&rc, 0, ram_ids[i]);
    int unc[16], n_unc = 0;
    for (int i = 0; i < k; i++)
        if (vc.map[ids[i]] < 0 && rc.map[ids[i]] < 0) unc[n_unc++] = i;
    car_state_t car;
    car_init(&car, threshold);
    car.skip_renorm = dampen ? true : false;
    int vsi[16], vss[16], nv = 0, rsi[16], rss[16], nr = 0;
    int subs = car_evaluate(&car, 0, -1, ids, scores, k, all_scores, n_experts, &vc, NULL,
                            n_ram > 0 ? &rc : NULL, unc, &n_unc, vsi, vss, &nv, NULL, NULL, NULL, rsi,
                            rss, &nr);
    *n_uncached_out = n_unc;
    *n_vram_subs_out = nv;
    for (int i = 0; i < nv; i++) vram_sub_idx_out[i] = vsi[i];
    vram_cache_free(&vc);
    ram_cache_free(&rc);
    return subs;
}

/* out[n_embd] = sum_e score_e * ffn_e(h) (+ shared expert, weight 1, added after). */
void refdrv_moe_block(float *out, const float *h, const void *const *experts, const float *scores, int k,
                      const void *shared_data, int gate_type, int up_type, int down_type,
                      uint64_t gate_size, uint64_t up_size, int n_embd, int inter) {
    static cpu_expert_ctx_t *ctx = NULL, *sctx = NULL;
    static int c_embd = 0, c_inter = 0;
    if (!ctx || c_embd != n_embd || c_inter != inter) {
        if (ctx) cpu_expert_free(ctx);
        if (sctx) cpu_expert_free(sctx);
        ctx = cpu_expert_create(n_embd, inter);
        sctx = cpu_expert_create(n_embd, inter);
        c_embd = n_embd;
        c_inter = inter;
    }
    cpu_expert_reset(ctx);
    for (int i = 0; i < k; i++)
        cpu_expert_ffn(ctx, experts[i], h, scores[i], gate_type, up_type, down_type, gate_size, up_size);
    memcpy(out, cpu_expert_result(ctx), sizeof(float) * (size_t)n_embd);
    if (shared_data) {
        cpu_expert_reset(sctx);
        cpu_expert_ffn(sctx, shared_data, h, 1.0f, gate_type, up_type, down_type, gate_size, up_size);
        vec_add(out, out, cpu_expert_result(sctx), n_embd);
    }
}

/* ---- the same block with fp32 activations: the reference's CPU forward pass without cpu_expert
 * (src/inference.c:556-575 for the routed experts, 361-374 and 582-596 for the shared one), composed from its own
 * mat_vec_mul / silu / vec_mul / vec_scaled_add / vec_add (src/tensor.c). ---- */
void refdrv_moe_block_f32(float *out, const float *h, const void *const *experts, const float *scores, int k,
                          const void *shared_data, int gate_type, int up_type, int down_type,
                          uint64_t gate_size, uint64_t up_size, int n_embd, int inter) {
    float *g = (float *)malloc(sizeof(float) * (size_t)inter);
    float *u = (float *)malloc(sizeof(float) * (size_t)inter);
    float *dn = (float *)malloc(sizeof(float) * (size_t)n_embd);
    memset(out, 0, sizeof(float) * (size_t)n_embd);
    for (int i = 0; i <= k; i++) {
        const uint8_t *e = (const uint8_t *)(i < k ? experts[i] : shared_data);
        if (!e) break;
        mat_vec_mul(g, e, (enum ggml_dtype)gate_type, h, inter, n_embd);
        silu(g, inter);
        mat_vec_mul(u, e + gate_size, (enum ggml_dtype)up_type, h, inter, n_embd);
        vec_mul(g, g, u, inter);
        mat_vec_mul(dn, e + gate_size + up_size, (enum ggml_dtype)down_type, g, n_embd, inter);
        if (i < k) vec_scaled_add(out, dn, scores[i], n_embd);
        else vec_add(out, out, dn, n_embd);
    }
    free(g);
    free(u);
    free(dn);
}

/* ---- expert store files: written with the reference's own writer (src/expert_store.c:128-172) so that the
 * loader under test reads exactly what tools/prepare_experts.c produces.  records[l][e] = gate | up | down bytes of
 * expert e of layer l; every expert is padded to a 4096-aligned stride as prepare_experts.c does. ---- */
#include <unistd.h>

#include "expert_store.h"

int refdrv_write_store(const char *path, int n_layers, int n_experts, uint64_t gate_size, uint64_t up_size,
                       const uint64_t *down_sizes, const uint32_t *down_types, const void *const *records) {
    uint64_t max_down = 0;
    for (int l = 0; l < n_layers; l++)
        if (down_sizes[l] > max_down) max_down = down_sizes[l];
    const uint64_t stride = ALIGN_UP(gate_size + up_size + max_down, (uint64_t)QMOE_ALIGNMENT);
    qmoe_header_t hd;
    memset(&hd, 0, sizeof(hd));
    hd.magic = QMOE_MAGIC;
    hd.version = QMOE_VERSION;
    hd.n_moe_layers = (uint32_t)n_layers;
    hd.n_experts = (uint32_t)n_experts;
    hd.quant_type = 12;
    hd.alignment = QMOE_ALIGNMENT;
    hd.expert_gate_size = gate_size;
    hd.expert_up_size = up_size;
    hd.expert_down_size = max_down;
    hd.expert_stride = stride;
    qmoe_layer_entry_t *layers = (qmoe_layer_entry_t *)calloc((size_t)n_layers, sizeof(qmoe_layer_entry_t));
    uint64_t off = ALIGN_UP((uint64_t)64 + (uint64_t)n_layers * sizeof(qmoe_layer_entry_t), (uint64_t)QMOE_ALIGNMENT);
    for (int l = 0; l < n_layers; l++) {
        layers[l].data_offset = off;
        layers[l].expert_stride = stride;
        layers[l].down_size = down_sizes[l];
        layers[l].down_type = down_types[l];
        off += stride * (uint64_t)n_experts;
    }
    int fd = expert_store_create(path, &hd, layers);
    if (fd < 0) {
        free(layers);
        return -1;
    }
    void *buf = NULL;
    if (posix_memalign(&buf, QMOE_ALIGNMENT, stride)) {
        close(fd);
        free(layers);
        return -1;
    }
    int rc = 0;
    for (int l = 0; l < n_layers && !rc; l++)
        for (int e = 0; e < n_experts && !rc; e++) {
            memset(buf, 0, stride);
            memcpy(buf, records[(size_t)l * n_experts + e], gate_size + up_size + down_sizes[l]);
            if (!expert_store_write_expert(fd, &layers[l], e, stride, buf, stride)) rc = -1;
        }
    free(buf);
    free(layers);
    close(fd);
    return rc;
}
