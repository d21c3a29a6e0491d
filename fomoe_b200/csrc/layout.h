/*
 * layout.h -- how expert weights lie in HBM ("lane-striped groups").
 *
 * The ggml block formats (Q4_K 144 B, Q5_K 176 B, Q6_K 210 B; the reference's include/quant_types.h:17-41)
 * are kept bit for bit, but the bytes of every 32 consecutive blocks of a matrix shard are
 * regrouped so that lane L of a warp owns block L of the group and every 16-byte piece a
 * lane needs sits next to the same piece of its 31 neighbours:
 *
 *   Q4_K group (4608 B):  uint4 hdr[32]      hdr[L] = {d | dmin<<16, scales[0..11]}
 *                         uint4 qs[8][32]    qs[k][L] = bytes 16k..16k+15 of block L's qs
 *   Q5_K group (5632 B):  uint4 hdr[32]      as Q4_K
 *                         uint4 qh[2][32]    qh[k][L] = bytes 16k..16k+15 of block L's qh (the fifth bits)
 *                         uint4 qs[8][32]    as Q4_K
 *   Q6_K group (6720 B):  uint4 ql[8][32]    ql[k][L] = bytes 16k..16k+15 of block L's ql
 *                         uint4 qh[4][32]    qh[k][L] = bytes 16k..16k+15 of block L's qh
 *                         uint4 sc[32]       sc[L]    = the 16 int8 scales
 *                         uint16 d[32]
 *
 * A warp therefore fetches a whole group with 9 (Q4_K), 11 (Q5_K) or 14 (Q6_K) fully coalesced
 * 512-byte requests, all independent, and no byte is padded: a shard occupies exactly
 * its ggml size.  Blocks of a shard are numbered row-major over the rows and the
 * 256-column blocks this rank owns (tensor parallelism splits gate/up by rows and down
 * by column blocks), so with bpr blocks per row a group covers 32/bpr consecutive rows.
 * Shards whose block count is not a multiple of 32 are padded with zero blocks at the end
 * (never the case at the 397B shape).
 *
 * HALF super-blocks (down shards when twice as many tensor-parallel ranks as 256-column windows share an expert:
 * each rank then owns 128 columns of every row).  Both halves of a Q6_K block are self-contained apart from the
 * fp16 d (src/quant.c:157-173); the halves of a Q4_K block share the 12 scale bytes (src/quant.c:72-80), so the
 * 16-byte header is stored with both halves.  Half h of block L:
 *
 *   Q4_K half group (2560 B):  uint4 hdr[32]      the full header {d | dmin<<16, scales[0..11]}
 *                              uint4 qs[4][32]    bytes 64h+16k .. 64h+16k+15 of block L's qs
 *   Q6_K half group (3392 B):  uint4 ql[4][32]    bytes 64h+16k .. of block L's ql
 *                              uint4 qh[2][32]    bytes 32h+16k .. of block L's qh
 *                              uint2 sc[32]       scales 8h .. 8h+7
 *                              uint16 d[32]
 */
#ifndef FOMOE_B200_LAYOUT_H
#define FOMOE_B200_LAYOUT_H

#include <stdint.h>

#define FB_TYPE_Q4_K 12
#define FB_TYPE_Q5_K 13
#define FB_TYPE_Q6_K 14
#define FB_TYPE_Q8_0 8    /* 32-value blocks, fp32 activations only: proj32.cu */
#define FB_TYPE_MXFP4 39
#define FB_QK 256
#define FB_Q4K_BLOCK 144u
#define FB_Q5K_BLOCK 176u
#define FB_Q6K_BLOCK 210u
#define FB_GROUP 32u
#define FB_Q4K_GROUP (FB_Q4K_BLOCK * FB_GROUP) /* 4608 */
#define FB_Q5K_GROUP (FB_Q5K_BLOCK * FB_GROUP) /* 5632 */
#define FB_Q6K_GROUP (FB_Q6K_BLOCK * FB_GROUP) /* 6720 */
#define FB_Q6K_OFF_QH 4096u
#define FB_Q6K_OFF_SC 6144u
#define FB_Q6K_OFF_D 6656u
#define FB_Q4K_HALF 80u
#define FB_Q5K_HALF 112u /* header 16, fifth-bit field 32 (kept whole: a half uses four bits of every byte), quants 64 */
#define FB_Q6K_HALF 106u
#define FB_Q4K_HGROUP (FB_Q4K_HALF * FB_GROUP) /* 2560 */
#define FB_Q5K_HGROUP (FB_Q5K_HALF * FB_GROUP) /* 3584 */
#define FB_Q6K_HGROUP (FB_Q6K_HALF * FB_GROUP) /* 3392 */
#define FB_Q6K_HOFF_QH 2048u
#define FB_Q6K_HOFF_SC 3072u
#define FB_Q6K_HOFF_D 3328u

#define FB_MAX_SLOTS 16   /* routed experts per token + shared expert */
#define FB_MAX_TOPK 15
#define FB_MAX_EXPERTS 512 /* the reference's MAX_N_EXPERTS_TOTAL, src/gpu_kernels.hip:438-448 */

#if defined(__CUDACC__)
#define FB_HD __host__ __device__ static inline
#else
#define FB_HD static inline
#endif

FB_HD uint64_t fb_block_bytes(int type) {
    return type == FB_TYPE_Q4_K ? FB_Q4K_BLOCK : type == FB_TYPE_Q5_K ? FB_Q5K_BLOCK : type == FB_TYPE_Q6_K ? FB_Q6K_BLOCK : 0;
}
FB_HD uint64_t fb_group_bytes(int type) { return fb_block_bytes(type) * FB_GROUP; }
/* the same for a shard of half super-blocks (half = 0 or 1; half < 0: whole blocks) */
FB_HD uint64_t fb_block_bytes_h(int type, int half) {
    if (half < 0) return fb_block_bytes(type);
    return type == FB_TYPE_Q4_K ? FB_Q4K_HALF : type == FB_TYPE_Q5_K ? FB_Q5K_HALF : type == FB_TYPE_Q6_K ? FB_Q6K_HALF : 0;
}
FB_HD uint64_t fb_group_bytes_h(int type, int half) { return fb_block_bytes_h(type, half) * FB_GROUP; }
FB_HD uint64_t fb_n_groups(uint64_t n_blocks) { return (n_blocks + FB_GROUP - 1) / FB_GROUP; }
/* bytes of a shard of n_blocks blocks in the device layout */
FB_HD uint64_t fb_shard_bytes(int type, uint64_t n_blocks) {
    return fb_n_groups(n_blocks) * fb_group_bytes(type);
}
FB_HD uint64_t fb_shard_bytes_h(int type, int half, uint64_t n_blocks) {
    return fb_n_groups(n_blocks) * fb_group_bytes_h(type, half);
}

#endif
