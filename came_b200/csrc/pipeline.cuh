// Shared-memory staging primitives for sm_100a: mbarrier + bulk asynchronous copies (TMA, untiled
// cp.async.bulk) and packed fp32x2 arithmetic.  Every wait is bounded: when a barrier does not complete
// within the limit the kernel records a code in the plan's status word and leaves.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace came {

constexpr uint32_t MBAR_SPIN_LIMIT = 1u << 22;   // try_wait suspends for a hardware time slice per call
constexpr int STATUS_MBAR_TIMEOUT = 1;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// make the initialised barriers visible to the async proxy before any copy names them
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// barrier among the first `nthreads` threads of the CTA (a multiple of 32), leaving the other warps out
__device__ __forceinline__ void named_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// bounded wait; false on timeout
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < MBAR_SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned), completing on `bar`
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// L2 eviction-priority policies for streams (read once: evict first) and for data another pass reads back soon
// (evict last), and the copy / store forms that carry them
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void st_global_v2_hint(void* dst, uint2 v, uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.v2.b32 [%0], {%1, %2}, %3;" ::"l"(dst), "r"(v.x), "r"(v.y), "l"(policy) : "memory");
}

// ---- packed fp32x2 (two independent IEEE fp32 operations per instruction, sm_100 FFMA2 / FADD2 / FMUL2) ----
typedef float2 u64;   // a pair of fp32 values living in an aligned register pair
#define F2ZERO make_float2(0.0f, 0.0f)
__device__ __forceinline__ u64 pk(float lo, float hi) { return make_float2(lo, hi); }
__device__ __forceinline__ u64 pk_u32(uint32_t lo, uint32_t hi) { return make_float2(__uint_as_float(lo), __uint_as_float(hi)); }
__device__ __forceinline__ void upk(u64 v, float& lo, float& hi) { lo = v.x; hi = v.y; }
__device__ __forceinline__ void upk_u32(u64 v, uint32_t& lo, uint32_t& hi) { lo = __float_as_uint(v.x); hi = __float_as_uint(v.y); }
#ifdef CAME_SCALAR_FP32   // build-time experiment: the same arithmetic with scalar instructions
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) { return make_float2(__fmaf_rn(a.x, b.x, c.x), __fmaf_rn(a.y, b.y, c.y)); }
__device__ __forceinline__ u64 mul2(u64 a, u64 b) { return make_float2(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y)); }
__device__ __forceinline__ u64 add2(u64 a, u64 b) { return make_float2(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y)); }
__device__ __forceinline__ u64 sub2(u64 a, u64 b) { return make_float2(__fsub_rn(a.x, b.x), __fsub_rn(a.y, b.y)); }
#else
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ u64 mul2(u64 a, u64 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ u64 add2(u64 a, u64 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ u64 sub2(u64 a, u64 b) { return __fadd2_rn(a, make_float2(-b.x, -b.y)); }
#endif
__device__ __forceinline__ u64 splat(float x) { return make_float2(x, x); }

// two int8 codes (bytes `b`, `b+1` of the word `x`, already biased by ^0x80) -> packed exact floats:
// the byte is dropped into the mantissa of 2^23, then 2^23 + 128 is subtracted
__device__ __forceinline__ u64 codes_to_f2(uint32_t x, int b) {
    const uint32_t lo = __byte_perm(x, 0x4B000000u, 0x7540u + b);
    const uint32_t hi = __byte_perm(x, 0x4B000000u, 0x7541u + b);
    return add2(pk_u32(lo, hi), splat(-8388736.0f));
}
// packed floats holding integers in [-127, 127] plus 1.5 * 2^23: the low byte of each is the int8 code
__device__ __forceinline__ uint32_t pack_codes4(u64 y01, u64 y23) {
    uint32_t a, b, c, d;
    upk_u32(y01, a, b);
    upk_u32(y23, c, d);
    return __byte_perm(__byte_perm(a, b, 0x0040u), __byte_perm(c, d, 0x0040u), 0x5410u);
}
constexpr float ROUND_MAGIC = 12582912.0f;   // 1.5 * 2^23: adding it rounds to the nearest integer, ties to even

}  // namespace came
