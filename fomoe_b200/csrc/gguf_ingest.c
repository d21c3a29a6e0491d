/*
 * gguf_ingest.c -- the MoE tensors of a GGUF model file into the resident table.
 *
 * The reference reads its model from GGUF (src/gguf.c, include/gguf.h:6-145; the tensor names it asks for:
 * src/model.c:277-283, 351-371, 391-395; tools/prepare_experts.c:262-291 cuts the stacked expert tensors into the
 * records of a .qmoe store).  This file reads the same container with a reader of its own -- header, key/value
 * section (skipped, except general.alignment), tensor directory -- and feeds the upload calls of the library:
 *
 *   blk.N.ffn_gate_inp.weight          router           [n_embd, n_experts]          F32 / F16 / BF16
 *   blk.N.ffn_gate_exps.weight         experts' gate    [n_embd, n_inter, n_experts] the context's gate type
 *   blk.N.ffn_up_exps.weight           experts' up      the same
 *   blk.N.ffn_down_exps.weight         experts' down    [n_inter, n_embd, n_experts] the layer's down type
 *   blk.N.ffn_{gate,up,down}_shexp.weight  shared expert, same types (skipped with a note otherwise)
 *   blk.N.ffn_gate_inp_shexp.weight    shared expert's scalar gate [n_embd]           optional
 *   blk.N.post_attention_norm.weight | blk.N.ffn_norm.weight   RMSNorm weight in front of the block, optional
 *
 * GGUF lists dimensions fastest first; an expert's matrix is one contiguous slice of its stacked tensor.
 * Single-file models only (the reference also follows -00001-of-N splits).
 */
#define _FILE_OFFSET_BITS 64
#define _POSIX_C_SOURCE 200809L
#include <sys/types.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/fomoe_b200.h"
#include "layout.h"

#define GG_MAGIC 0x46554747u /* "GGUF" */
#define GG_MAX_DIMS 4

typedef struct {
    char *name;
    uint32_t n_dims;
    uint64_t dims[GG_MAX_DIMS];
    uint32_t type;
    uint64_t offset; /* within the data section */
    uint64_t nbytes;
} gg_tensor_t;

typedef struct {
    FILE *f;
    uint64_t n_tensors, data_offset, alignment, file_size;
    gg_tensor_t *t;
} gg_file_t;

static int gg_rd(gg_file_t *g, void *dst, size_t n) { return fread(dst, 1, n, g->f) == n ? 0 : -1; }

static int gg_skip(gg_file_t *g, uint64_t n) { return fseeko(g->f, (off_t)n, SEEK_CUR); }

/* length-prefixed string: returned as a new C string when out != NULL, skipped otherwise */
static int gg_string(gg_file_t *g, char **out) {
    uint64_t len;
    if (gg_rd(g, &len, 8) || len > (1u << 20)) return -1;
    if (!out) return gg_skip(g, len);
    char *s = (char *)malloc(len + 1);
    if (!s || gg_rd(g, s, len)) {
        free(s);
        return -1;
    }
    s[len] = 0;
    *out = s;
    return 0;
}

static int gg_scalar_size(uint32_t type) {
    switch (type) {
        case 0: case 1: case 7: return 1;   /* u8, i8, bool */
        case 2: case 3: return 2;           /* u16, i16 */
        case 4: case 5: case 6: return 4;   /* u32, i32, f32 */
        case 10: case 11: case 12: return 8; /* u64, i64, f64 */
        default: return 0;
    }
}

/* skips one value of the key/value section; *u32_out receives it when it is a u32 */
static int gg_skip_value(gg_file_t *g, uint32_t type, uint32_t *u32_out) {
    if (type == 8) return gg_string(g, NULL);
    if (type == 9) {
        uint32_t et;
        uint64_t n;
        if (gg_rd(g, &et, 4) || gg_rd(g, &n, 8)) return -1;
        if (et == 8) {
            for (uint64_t i = 0; i < n; i++)
                if (gg_string(g, NULL)) return -1;
            return 0;
        }
        const int sz = gg_scalar_size(et);
        return sz ? gg_skip(g, n * (uint64_t)sz) : -1;
    }
    const int sz = gg_scalar_size(type);
    if (!sz) return -1;
    if (type == 4 && u32_out) return gg_rd(g, u32_out, 4);
    return gg_skip(g, (uint64_t)sz);
}

/* bytes of n elements of a ggml type (the types an expert model's MoE tensors come in) */
static uint64_t gg_nbytes(uint32_t type, uint64_t n) {
    switch (type) {
        case 0: return 4 * n;                    /* F32 */
        case 1: case 30: return 2 * n;           /* F16, BF16 */
        case 8: return n / 32 * 34;              /* Q8_0 */
        case 39: return n / 32 * 17;             /* MXFP4 */
        case FB_TYPE_Q4_K: return n / 256 * FB_Q4K_BLOCK;
        case FB_TYPE_Q5_K: return n / 256 * FB_Q5K_BLOCK;
        case FB_TYPE_Q6_K: return n / 256 * FB_Q6K_BLOCK;
        default: return 0;
    }
}

static void gg_close(gg_file_t *g) {
    if (!g) return;
    if (g->t)
        for (uint64_t i = 0; i < g->n_tensors; i++) free(g->t[i].name);
    free(g->t);
    if (g->f) fclose(g->f);
    free(g);
}

static gg_file_t *gg_open(const char *path, char *err, size_t err_len) {
    gg_file_t *g = (gg_file_t *)calloc(1, sizeof(*g));
    if (!g) return NULL;
    const char *why = "cannot open";
    g->f = fopen(path, "rb");
    if (!g->f) goto fail;
    fseeko(g->f, 0, SEEK_END);
    g->file_size = (uint64_t)ftello(g->f);
    fseeko(g->f, 0, SEEK_SET);
    uint32_t magic, version;
    uint64_t n_kv;
    why = "not a GGUF file (magic / version 2 or 3 expected)";
    if (gg_rd(g, &magic, 4) || gg_rd(g, &version, 4) || magic != GG_MAGIC || (version != 2 && version != 3)) goto fail;
    why = "truncated header";
    if (gg_rd(g, &g->n_tensors, 8) || gg_rd(g, &n_kv, 8) || g->n_tensors > (1u << 20) || n_kv > (1u << 20)) goto fail;
    g->alignment = 32; /* include/gguf.h:55 */
    why = "malformed key/value section";
    for (uint64_t i = 0; i < n_kv; i++) {
        char *key = NULL;
        uint32_t type, u32 = 0;
        if (gg_string(g, &key) || gg_rd(g, &type, 4) || gg_skip_value(g, type, &u32)) {
            free(key);
            goto fail;
        }
        if (type == 4 && !strcmp(key, "general.alignment") && u32) g->alignment = u32;
        free(key);
    }
    why = "malformed tensor directory";
    g->t = (gg_tensor_t *)calloc(g->n_tensors ? g->n_tensors : 1, sizeof(gg_tensor_t));
    if (!g->t) goto fail;
    for (uint64_t i = 0; i < g->n_tensors; i++) {
        gg_tensor_t *t = &g->t[i];
        if (gg_string(g, &t->name) || gg_rd(g, &t->n_dims, 4) || t->n_dims < 1 || t->n_dims > GG_MAX_DIMS) goto fail;
        uint64_t n = 1;
        for (uint32_t d = 0; d < GG_MAX_DIMS; d++) t->dims[d] = 1;
        for (uint32_t d = 0; d < t->n_dims; d++) {
            if (gg_rd(g, &t->dims[d], 8) || t->dims[d] == 0 || t->dims[d] > (1ull << 40) / n) goto fail;
            n *= t->dims[d];
        }
        if (gg_rd(g, &t->type, 4) || gg_rd(g, &t->offset, 8)) goto fail;
        t->nbytes = gg_nbytes(t->type, n); /* 0: a type this library has no use for */
    }
    {
        const uint64_t here = (uint64_t)ftello(g->f);
        g->data_offset = (here + g->alignment - 1) / g->alignment * g->alignment;
    }
    return g;
fail:
    if (err) snprintf(err, err_len, "%s: %s", path, why);
    gg_close(g);
    return NULL;
}

static const gg_tensor_t *gg_find(const gg_file_t *g, const char *name) {
    for (uint64_t i = 0; i < g->n_tensors; i++)
        if (!strcmp(g->t[i].name, name)) return &g->t[i];
    return NULL;
}

static int gg_read(gg_file_t *g, const gg_tensor_t *t, uint64_t at, void *dst, uint64_t n) {
    /* every term is checked by itself: a malformed directory must not wrap the sum */
    if (at > t->nbytes || n > t->nbytes - at || g->data_offset > g->file_size || t->offset > g->file_size - g->data_offset ||
        t->nbytes > g->file_size - g->data_offset - t->offset)
        return -1;
    if (fseeko(g->f, (off_t)(g->data_offset + t->offset + at), SEEK_SET)) return -1;
    return gg_rd(g, dst, n);
}

/* ------------------------------------------------------------------ host-only look-up (no GPU involved) */
int fomoe_b200_gguf_tensor(const char *path, const char *name, int *type, int64_t *dims, uint64_t *nbytes, void *buf,
                           uint64_t buf_bytes) {
    if (!path || !name) return -1;
    gg_file_t *g = gg_open(path, NULL, 0);
    if (!g) return -1;
    const gg_tensor_t *t = gg_find(g, name);
    int rc = -1;
    if (t) {
        if (type) *type = (int)t->type;
        if (dims)
            for (int d = 0; d < GG_MAX_DIMS; d++) dims[d] = (int64_t)t->dims[d];
        if (nbytes) *nbytes = t->nbytes;
        rc = 0;
        if (buf && (t->nbytes == 0 || t->nbytes > buf_bytes || gg_read(g, t, 0, buf, t->nbytes))) rc = -1;
    }
    gg_close(g);
    return rc;
}

/* ------------------------------------------------------------------ into the table */
static float gg_f16(uint16_t h) { /* IEEE half to float, subnormals included (as src/quant.c:30-47) */
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 31u, man = h & 1023u;
    uint32_t bits;
    if (exp == 0) {
        if (!man) bits = sign;
        else {
            uint32_t m = man, e = 113;
            while (!(m & 1024u)) {
                m <<= 1;
                e--;
            }
            bits = sign | (e << 23) | ((m & 1023u) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* a whole tensor as fp32 (F32 / F16 / BF16 sources), n elements expected; NULL when absent or of another shape */
static float *gg_read_f32(gg_file_t *g, const char *name, uint64_t n) {
    const gg_tensor_t *t = gg_find(g, name);
    if (!t || (t->type != 0 && t->type != 1 && t->type != 30) || t->nbytes != gg_nbytes(t->type, n)) return NULL;
    float *out = (float *)malloc(sizeof(float) * n);
    if (!out) return NULL;
    if (t->type == 0) {
        if (gg_read(g, t, 0, out, 4 * n)) goto bad;
        return out;
    }
    uint16_t *tmp = (uint16_t *)malloc(2 * n);
    if (!tmp || gg_read(g, t, 0, tmp, 2 * n)) {
        free(tmp);
        goto bad;
    }
    for (uint64_t i = 0; i < n; i++) {
        if (t->type == 1) out[i] = gg_f16(tmp[i]);
        else {
            const uint32_t b = (uint32_t)tmp[i] << 16;
            memcpy(&out[i], &b, 4);
        }
    }
    free(tmp);
    return out;
bad:
    free(out);
    return NULL;
}

static uint64_t mat_bytes(int type, int rows, int cols) { return (uint64_t)rows * (uint64_t)(cols / FB_QK) * fb_block_bytes(type); }

int fomoe_b200_load_gguf(fomoe_b200_ctx_t *ctx, const char *path, int first_block) {
    const fomoe_b200_config_t *cfg = fomoe_b200_get_config(ctx);
    if (!ctx || !path || !cfg || first_block < 0) return -1;
    char err[160];
    gg_file_t *g = gg_open(path, err, sizeof(err));
    if (!g) {
        fprintf(stderr, "fomoe_b200_load_gguf: %s\n", err);
        return -1;
    }
    const int nE = cfg->n_experts, ne = cfg->n_embd, ni = cfg->n_inter;
    const uint64_t gb = mat_bytes(cfg->gate_type, ni, ne);
    int loaded = 0, rc = -1;
    uint8_t *rec = NULL;
    char name[96];
    for (int l = 0; l < cfg->n_layers; l++) {
        const int blk = first_block + l;
        const int dt = cfg->down_types ? cfg->down_types[l] : FB_TYPE_Q6_K;
        const uint64_t db = mat_bytes(dt, ne, ni), rb = 2 * gb + db;
        uint8_t *nrec = (uint8_t *)realloc(rec, rb);
        if (!nrec) goto done;
        rec = nrec;
        /* router */
        snprintf(name, sizeof(name), "blk.%d.ffn_gate_inp.weight", blk);
        float *w = gg_read_f32(g, name, (uint64_t)nE * ne);
        if (!w) {
            fprintf(stderr, "fomoe_b200_load_gguf: %s missing or not [%d x %d] F32/F16/BF16\n", name, ne, nE);
            goto done;
        }
        const int e1 = fomoe_b200_router_upload(ctx, l, w);
        free(w);
        if (e1) goto done;
        /* routed experts: one contiguous slice of each stacked tensor per expert */
        const gg_tensor_t *tg, *tu, *td;
        snprintf(name, sizeof(name), "blk.%d.ffn_gate_exps.weight", blk);
        tg = gg_find(g, name);
        snprintf(name, sizeof(name), "blk.%d.ffn_up_exps.weight", blk);
        tu = gg_find(g, name);
        snprintf(name, sizeof(name), "blk.%d.ffn_down_exps.weight", blk);
        td = gg_find(g, name);
        if (!tg || !tu || !td || (int)tg->type != cfg->gate_type || (int)tu->type != cfg->gate_type || (int)td->type != dt ||
            tg->nbytes != gb * (uint64_t)nE || tu->nbytes != gb * (uint64_t)nE || td->nbytes != db * (uint64_t)nE ||
            tg->dims[0] != (uint64_t)ne || tg->dims[1] != (uint64_t)ni || td->dims[0] != (uint64_t)ni || td->dims[1] != (uint64_t)ne) {
            fprintf(stderr, "fomoe_b200_load_gguf: block %d: stacked expert tensors missing, or of another type or shape than "
                            "the context's\n", blk);
            goto done;
        }
        for (int e = 0; e < nE; e++) {
            if (gg_read(g, tg, gb * (uint64_t)e, rec, gb) || gg_read(g, tu, gb * (uint64_t)e, rec + gb, gb) ||
                gg_read(g, td, db * (uint64_t)e, rec + 2 * gb, db) || fomoe_b200_table_upload(ctx, l, e, rec))
                goto done;
        }
        /* shared expert, when the context has one and the file stores it in the experts' formats */
        if (cfg->has_shared) {
            snprintf(name, sizeof(name), "blk.%d.ffn_gate_shexp.weight", blk);
            tg = gg_find(g, name);
            snprintf(name, sizeof(name), "blk.%d.ffn_up_shexp.weight", blk);
            tu = gg_find(g, name);
            snprintf(name, sizeof(name), "blk.%d.ffn_down_shexp.weight", blk);
            td = gg_find(g, name);
            if (tg && tu && td && (int)tg->type == cfg->gate_type && (int)tu->type == cfg->gate_type && (int)td->type == dt &&
                tg->nbytes == gb && tu->nbytes == gb && td->nbytes == db) {
                if (gg_read(g, tg, 0, rec, gb) || gg_read(g, tu, 0, rec + gb, gb) || gg_read(g, td, 0, rec + 2 * gb, db) ||
                    fomoe_b200_table_upload(ctx, l, nE, rec))
                    goto done;
            } else {
                fprintf(stderr, "fomoe_b200_load_gguf: block %d: shared expert absent or not in the experts' formats and "
                                "shape: left as it is (Q8_0 / MXFP4 ones run through fomoe_b200_shared_ffn_f32)\n", blk);
            }
            snprintf(name, sizeof(name), "blk.%d.ffn_gate_inp_shexp.weight", blk);
            float *sg = gg_read_f32(g, name, (uint64_t)ne);
            if (sg) {
                const int e2 = fomoe_b200_shared_gate_upload(ctx, l, sg);
                free(sg);
                if (e2) goto done;
            }
        }
        /* the RMSNorm weight in front of the block (src/model.c:277-283) */
        snprintf(name, sizeof(name), "blk.%d.post_attention_norm.weight", blk);
        float *nw = gg_read_f32(g, name, (uint64_t)ne);
        if (!nw) {
            snprintf(name, sizeof(name), "blk.%d.ffn_norm.weight", blk);
            nw = gg_read_f32(g, name, (uint64_t)ne);
        }
        if (nw) {
            const int e3 = fomoe_b200_glue_upload(ctx, l, NULL, nw);
            free(nw);
            if (e3) goto done;
        }
        loaded++;
    }
    rc = loaded;
done:
    free(rec);
    gg_close(g);
    return rc;
}
