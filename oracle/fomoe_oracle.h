/*
 * fomoe_oracle.h -- CPU restatement of fomoe's routed-expert FFN decode path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product library links, loads or
 * calls this code; it exists so the CUDA path can be checked against the
 * reference's arithmetic.  Every function cites the reference file:line it
 * restates.  Parity is PINNED: tests/test_oracle_pin.py checks each function
 * bit-for-bit against the reference's own C files compiled unmodified
 * (oracle/_ref/libfomoe_ref.so) and against golden vectors those files
 * produced (tests/golden/).
 */
#ifndef FOMOE_ORACLE_H
#define FOMOE_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORC_QK_K 256
#define ORC_TYPE_Q4_K 12 /* include/quant_types.h:56-64 */
#define ORC_TYPE_Q5_K 13
#define ORC_TYPE_Q6_K 14
#define ORC_TYPE_Q8_0 8
#define ORC_TYPE_MXFP4 39

/* Block layouts, include/quant_types.h:17-41 and include/quant.h:94-98. */
typedef struct {
    uint16_t d, dmin;
    uint8_t scales[12];
    uint8_t qs[128];
} orc_block_q4_K; /* 144 B */

typedef struct {
    uint16_t d, dmin;
    uint8_t scales[12];
    uint8_t qh[32];
    uint8_t qs[128];
} orc_block_q5_K; /* 176 B */

#pragma pack(push, 1)
typedef struct {
    uint8_t ql[128];
    uint8_t qh[64];
    int8_t scales[16];
    uint16_t d;
} orc_block_q6_K; /* 210 B */
#pragma pack(pop)

typedef struct {
    float d;
    int8_t qs[256];
    int16_t bsums[16];
} orc_block_q8_K; /* 292 B */

float orc_fp16_to_fp32(uint16_t h);                                        /* src/quant.c:30-47 */
void orc_dequantize_row_q4_K(const void *x, float *y, int64_t k);          /* src/quant.c:82-105 */
void orc_dequantize_row_q5_K(const void *x, float *y, int64_t k);          /* src/quant.c:216-247 */
void orc_dequantize_row_q6_K(const void *x, float *y, int64_t k);          /* src/quant.c:147-175 */
void orc_quantize_row_q8_K(const float *x, void *y, int64_t k);            /* src/quant.c:343-375 */
float orc_vec_dot_q4_K_q8_K(const void *x, const void *y, int nb);         /* src/quant.c:405-476 */
float orc_vec_dot_q5_K_q8_K(const void *x, const void *y, int nb);         /* src/quant.c:609-621 */
float orc_vec_dot_q6_K_q8_K(const void *x, const void *y, int nb);         /* src/quant.c:478-607 */
/* fp32-activation dots, the reference's second definition of the same products (its CPU forward pass without
 * cpu_expert and, up to summation order, its GPU kernels) */
float orc_vec_dot_q4_K_f32(const void *x, const float *y, int64_t n);      /* src/quant.c:109-143 */
void orc_dequantize_row_q8_0(const void *x, float *y, int64_t k);           /* src/quant.c:266-274 */
void orc_dequantize_row_mxfp4(const void *x, float *y, int64_t k);          /* src/quant.c:299-318 */
float orc_vec_dot_q8_0_f32(const void *x, const float *y, int64_t n);       /* src/quant.c:276-288 */
float orc_vec_dot_mxfp4_f32(const void *x, const float *y, int64_t n);      /* src/quant.c:320-337 */
void orc_mat_vec_mul_f32act(float *out, const void *mat, int type, const float *x, int M, int K); /* src/tensor.c:102-171 */
void orc_shared_ffn_f32(float *out, const float *h, const void *gate, int gate_type, const void *up, int up_type,
                        const void *down, int down_type, int n_embd, int inter); /* src/inference.c:361-374 */
float orc_vec_dot_q5_K_f32(const void *x, const float *y, int64_t n);      /* src/quant.c:249-262 */
float orc_vec_dot_q6_K_f32(const void *x, const float *y, int64_t n);      /* src/quant.c:177-212 */
void orc_moe_block_f32(float *out, const float *h, const void *const *experts, const float *scores, int k,
                       const void *shared_data, int gate_type, int up_type, int down_type, uint64_t gate_size,
                       uint64_t up_size, int n_embd, int inter);            /* src/inference.c:556-596 */
uint64_t orc_row_bytes(int type, int k);                                   /* include/quant_types.h:93-97 */

/* out[i] = vec_dot(row_i, q8); src/cpu_expert.c:52-72 */
void orc_matvec_q8(float *out, const void *mat, int type, const void *q8, int M, int K);

/* One expert's SwiGLU FFN accumulated into partial[n_embd]; src/cpu_expert.c:75-116.
 * q8_input is the already-quantised hidden state (n_embd/256 blocks).
 * act_out (optional, may be NULL) receives silu(gate)*up, [inter]. */
void orc_expert_ffn(float *partial, const void *expert_data, const void *q8_input, float score,
                    int gate_type, int up_type, int down_type, uint64_t gate_size, uint64_t up_size,
                    int n_embd, int inter, float *act_out);

/* Router: logits = W[n_experts x n_embd] . h (sequential fp32 multiply-then-add per row,
 * src/tensor.c:104-113), then softmax in place (src/tensor.c:186-200). */
void orc_router_logits(float *logits, const float *w, const float *h, int n_experts, int n_embd);
void orc_softmax(float *x, int64_t n);
void orc_top_k(const float *x, int64_t n, int k, int *indices, float *values); /* src/tensor.c:226-252 */
void orc_renorm(float *scores, int k);                                        /* src/inference.c:496-502 */
float orc_shared_gate(const float *h, const float *w, int n_embd);               /* src/inference.c:586-590 */
void orc_rms_norm(float *out, const float *x, const float *w, int64_t n, float eps); /* src/tensor.c:175-184 */

/* Cache-aware routing over a single residency tier given as a bit mask
 * (bit e of mask[e/32] set = expert e resident).  Restates the classify loop
 * src/gpu_kernels.hip:7097-7149 (single tier), the guard at 7168-7171 and
 * src/car.c:36-264 with budgets off.  Returns the number of substitutions;
 * ids/scores are updated in place. */
int orc_car(int *ids, float *scores, int k, const float *all_scores, int n_experts,
            const uint32_t *resident_mask, float threshold, int dampen);

/* router -> softmax -> top-k -> renorm -> CAR; returns substitutions. */
int orc_route(const float *router_w, const float *h, int n_experts, int n_embd, int k,
              const uint32_t *resident_mask, float threshold, int dampen, float *all_scores,
              int *ids, float *scores);

/* Full MoE block on a given normalised hidden state h:
 *   out = sum_e score_e * ffn_e(h)  (+ shared expert with weight 1 when shared_data != NULL).
 * experts[i] points at expert ids[i]'s record (gate|up|down back to back). */
void orc_moe_block(float *out, const float *h, const void *const *experts, const float *scores, int k,
                   const void *shared_data, int gate_type, int up_type, int down_type,
                   uint64_t gate_size, uint64_t up_size, int n_embd, int inter);

#ifdef __cplusplus
}
#endif
#endif
