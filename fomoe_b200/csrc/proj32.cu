/*
 * proj32.cu -- projections whose weights come in 32-value blocks: Q8_0 (34 bytes: fp16 scale, 32 int8) and MXFP4
 * (17 bytes: E8M0 shared exponent, 32 E2M1 nibbles).  Some models store the shared expert's gate/up/down projections
 * in these types; the reference multiplies them with fp32 activations only (src/quant.c:266-337 through
 * mat_vec_mul, src/tensor.c:158-171; on its GPU: src/gpu_kernels.hip:2070-2103), so there is no Q8_K form of them.
 *
 * The matrices stay in ggml byte order (a row is cols/32 consecutive blocks; rows are only 2-byte / 1-byte aligned,
 * so nothing wider than the natural element is loaded).  One warp per row; lane j owns element j of every block, so
 * a block's quant bytes and the 32 activations it meets are each one contiguous run per warp instruction.  Every
 * product d * q is exact in fp32 (11 significant bits x 7, or a power of two x a 2-bit significand); the sum over a
 * row is formed per lane and then across lanes, i.e. it differs from the reference's block-by-block order by fp32
 * reassociation only.
 */
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "launch.h"

#define FULL 0xffffffffu

/* E2M1: sign, two exponent bits, one mantissa bit -- the table of src/quant.c:294-297 */
__device__ __forceinline__ float p32_e2m1(uint32_t n) {
    const uint32_t m = n & 7u;
    /* 0, 0.5, 1, 1.5, 2, 3, 4, 6 */
    const float v = m < 2 ? 0.5f * (float)m : (m & 1u ? 1.5f : 1.0f) * (float)(1u << ((m >> 1) - 1));
    return (n & 8u) ? -v : v;
}

/* 2^(s - 127); s == 255 encodes NaN and is read as zero (src/quant.c:303-309) */
__device__ __forceinline__ float p32_e8m0(uint32_t s) {
    if (s == 0xffu) return 0.0f;
    if (s == 0u) return __uint_as_float(0x00400000u); /* 2^-127, a subnormal */
    return __uint_as_float(s << 23);
}

template <int TYPE>
__device__ __forceinline__ float p32_row_dot(const uint8_t *row, const float *x, int nb, int lane) {
    float acc0 = 0.0f, acc1 = 0.0f;
    if (TYPE == FB_TYPE_Q8_0) {
        int b = 0;
        for (; b + 1 < nb; b += 2) { /* two blocks in flight */
            const uint8_t *p0 = row + (size_t)b * 34, *p1 = p0 + 34;
            const float d0 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(p0)));
            const float d1 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(p1)));
            const float q0 = (float)(int)(signed char)p0[2 + lane], q1 = (float)(int)(signed char)p1[2 + lane];
            acc0 = __fmaf_rn(__fmul_rn(d0, q0), __ldg(x + b * 32 + lane), acc0);
            acc1 = __fmaf_rn(__fmul_rn(d1, q1), __ldg(x + b * 32 + 32 + lane), acc1);
        }
        if (b < nb) {
            const uint8_t *p0 = row + (size_t)b * 34;
            const float d0 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(p0)));
            acc0 = __fmaf_rn(__fmul_rn(d0, (float)(int)(signed char)p0[2 + lane]), __ldg(x + b * 32 + lane), acc0);
        }
    } else {
        /* ggml order inside a block: low nibbles are elements 0..15, high nibbles 16..31 */
        const int byte = 1 + (lane & 15), sh = (lane >> 4) * 4;
        int b = 0;
        for (; b + 1 < nb; b += 2) {
            const uint8_t *p0 = row + (size_t)b * 17, *p1 = p0 + 17;
            const float w0 = __fmul_rn(p32_e2m1((p0[byte] >> sh) & 15u), p32_e8m0(p0[0]));
            const float w1 = __fmul_rn(p32_e2m1((p1[byte] >> sh) & 15u), p32_e8m0(p1[0]));
            acc0 = __fmaf_rn(w0, __ldg(x + b * 32 + lane), acc0);
            acc1 = __fmaf_rn(w1, __ldg(x + b * 32 + 32 + lane), acc1);
        }
        if (b < nb) {
            const uint8_t *p0 = row + (size_t)b * 17;
            acc0 = __fmaf_rn(__fmul_rn(p32_e2m1((p0[byte] >> sh) & 15u), p32_e8m0(p0[0])), __ldg(x + b * 32 + lane), acc0);
        }
    }
    float acc = __fadd_rn(acc0, acc1);
#pragma unroll
    for (int o = 16; o; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(FULL, acc, o));
    return acc;
}

__device__ __forceinline__ float p32_dot_any(int type, const uint8_t *w, int row, const float *x, int cols, int lane) {
    const int nb = cols / 32;
    return type == FB_TYPE_Q8_0 ? p32_row_dot<FB_TYPE_Q8_0>(w + (size_t)row * nb * 34, x, nb, lane)
                                : p32_row_dot<FB_TYPE_MXFP4>(w + (size_t)row * nb * 17, x, nb, lane);
}

/* y[rows] = W x */
__global__ void __launch_bounds__(256) k_p32_matvec(int type, const uint8_t *w, int rows, int cols, const float *x, float *y) {
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
        const float f = p32_dot_any(type, w, r, x, cols, lane);
        if (lane == 0) y[r] = f;
    }
}

/* act[inter] = silu(gate h) * (up h), src/inference.c:365-370 with silu of src/tensor.c:202-206 */
__global__ void __launch_bounds__(256) k_p32_gate_up(int gate_type, const uint8_t *gate, int up_type, const uint8_t *up,
                                                     int inter, int n_embd, const float *h, float *act) {
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < inter; r += gridDim.x * wpb) {
        const float g = p32_dot_any(gate_type, gate, r, h, n_embd, lane);
        const float u = p32_dot_any(up_type, up, r, h, n_embd, lane);
        if (lane == 0) act[r] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
    }
}

static int p32_grid(int rows) {
    const int g = (rows + 7) / 8;
    return g < 1 ? 1 : (g > 148 * 8 ? 148 * 8 : g);
}

extern "C" int fb_launch_p32_matvec(int type, const uint8_t *w, int rows, int cols, const float *x, float *y, void *stream) {
    k_p32_matvec<<<p32_grid(rows), 256, 0, (cudaStream_t)stream>>>(type, w, rows, cols, x, y);
    return (int)cudaGetLastError();
}

extern "C" int fb_launch_p32_gate_up(int gate_type, const uint8_t *gate, int up_type, const uint8_t *up, int inter,
                                     int n_embd, const float *h, float *act, void *stream) {
    k_p32_gate_up<<<p32_grid(inter), 256, 0, (cudaStream_t)stream>>>(gate_type, gate, up_type, up, inter, n_embd, h, act);
    return (int)cudaGetLastError();
}
