/*
 * stream.cuh -- bulk-copy (TMA) streaming of weight groups into shared memory.
 *
 * A lane-striped group (layout.h) is one contiguous, 16-byte aligned run of 4608 or 6720
 * bytes, so a whole group is fetched by ONE untiled bulk copy (cp.async.bulk, global ->
 * shared, completion counted in bytes on an mbarrier).  Each warp owns a private ring of
 * stages: lane 0 issues the copies, all lanes wait on the stage's mbarrier, read their
 * 16-byte pieces conflict-free, and the stage is refilled as soon as the warp has read it.
 * With two or three stages per warp an SM keeps 100-200 KB of weight bytes in flight with
 * almost no registers or instructions spent on addressing.
 *
 * Every wait is bounded: when the limit runs out the kernel records FB_ST_WAIT_TIMEOUT
 * in the status word and stops consuming (it never spins forever).
 */
#pragma once
#include <stdint.h>

#include "launch.h"

#define FB_WAIT_LIMIT (1u << 20) /* polls of a time-limited try_wait */

__device__ __forceinline__ uint32_t fb_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void fb_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fb_mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fb_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void fb_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t fb_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

/* Bounded wait; returns false when the limit ran out (status word is set by the caller). */
__device__ __forceinline__ bool fb_mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < FB_WAIT_LIMIT; i++)
        if (fb_mbar_try_wait(bar, parity)) return true;
    return false;
}

/* global -> shared bulk copy; src, dst 16-byte aligned, bytes a multiple of 16 */
__device__ __forceinline__ void fb_bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

/* Ask for `bytes` (a multiple of 16, source 16-byte aligned) to be brought into L2; nothing waits for it. */
__device__ __forceinline__ void fb_prefetch_l2(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ uint4 fb_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
