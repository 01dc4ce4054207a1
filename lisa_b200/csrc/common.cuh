// Shared device helpers: bf16 bit casts, mbarrier / bulk-copy / programmatic-launch
// PTX wrappers and the host-side error plumbing used by every translation unit.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "lisa_cuda.h"

namespace lisa {

// ---------------------------------------------------------------- host side
void set_error(const std::string &msg);
int fail(int code, const std::string &msg);
int cuda_fail(cudaError_t err, const char *what);
void count_launch(unsigned n = 1);
int sm_count();           // SMs of the current device (cached per device)
int max_smem_optin();     // opt-in shared memory per block of the current device

#define LISA_CUDA_TRY(expr)                                         \
    do {                                                            \
        cudaError_t _e = (expr);                                    \
        if (_e != cudaSuccess) return ::lisa::cuda_fail(_e, #expr); \
    } while (0)

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------- device side
#ifdef __CUDACC__

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

// Round-to-nearest-even f32 -> bf16 bits (NaN stays NaN).
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float v) {
    uint32_t out;
    asm("{ .reg .b16 t; cvt.rn.bf16.f32 t, %1; mov.b32 %0, {t, t}; }" : "=r"(out) : "f"(v));
    return out & 0xffffu;
}
// Packs {lo, hi} into one 32-bit word of two bf16 (lo in the low half).
__device__ __forceinline__ uint32_t f32x2_to_bf16x2(float lo, float hi) {
    uint32_t out;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
    return out;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// d = a * b + c on two packed f32 lanes (sm_100 fma.rn.f32x2).
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    unsigned long long ra, rb, rc, rd;
    ra = (static_cast<unsigned long long>(__float_as_uint(a.y)) << 32) | __float_as_uint(a.x);
    rb = (static_cast<unsigned long long>(__float_as_uint(b.y)) << 32) | __float_as_uint(b.x);
    rc = (static_cast<unsigned long long>(__float_as_uint(c.y)) << 32) | __float_as_uint(c.x);
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    d.x = __uint_as_float(static_cast<uint32_t>(rd));
    d.y = __uint_as_float(static_cast<uint32_t>(rd >> 32));
    return d;
}

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking poll (try_wait may suspend the thread for a while when the phase is not complete).
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls and returns false, so a lost
// arrival ends in an error status instead of a hung GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity,
                                          uint32_t limit = 4000000u) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// The same for many waiting warps that are not on the critical path: sleep between polls, so that
// their polling does not fill the shared-memory pipeline that the few latency-critical threads
// (TMA producer, MMA issuer) of the CTA also go through.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t *bar, uint32_t parity, uint32_t sleep_ns = 64,
                                                  uint32_t limit = 4000000u) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(sleep_ns);
    }
    return false;
}

// One lane of a converged warp (elect.sync).  The single-thread roles (TMA producer, MMA issuer) run
// their loops with the whole warp -- waits, counters and addresses stay warp-uniform -- and only the
// instruction that must be issued once sits behind this predicate.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
    return pred != 0;
}

// ---- bulk async copy global -> shared (TMA, untiled), completes on an mbarrier ----
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---- programmatic dependent launch ----
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

#endif  // __CUDACC__

}  // namespace lisa
