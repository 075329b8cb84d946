// Building blocks shared by the shared-memory staged ("wide") momentum / apply kernels: stage geometry, staged-run
// conversions, the bounded abort-aware waits, and the copy stream of a persistent CTA.
#pragma once

#include "common.cuh"
#include "launch.h"
#include "pipeline.cuh"

#include <type_traits>

namespace came {

constexpr int W_WARPS = W_THREADS / 32;          // 16
constexpr int W_BAND = 16;
constexpr int W_BANDS = W_TR / W_BAND;           // 8
constexpr int W_MROW = W_TC + 64;                // staged row of int8 codes (+64: rows r, r+1 fall in different banks)

template <typename T> struct WideCfg {
    static constexpr int ROW = W_TC * (int)sizeof(T);                  // staged row of T
    static constexpr int AMAX_OFF = W_BAND * (ROW + W_MROW);           // the band's W_TC / 16 tile absmax values
    static constexpr int STAGE = AMAX_OFF + (W_TC / TILE) * (int)sizeof(float);
    static constexpr int STAGES = sizeof(T) == 2 ? 4 : 2;
};

// 8 consecutive staged elements -> 4 packed fp32 pairs
__device__ __forceinline__ void wide_run8(const __nv_bfloat16* p, u64* out) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j] = pk_u32(w[j] << 16, w[j] & 0xffff0000u);
}
__device__ __forceinline__ void wide_run8(const __half* p, u64* out) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        out[j] = pk(f.x, f.y);
    }
}
__device__ __forceinline__ void wide_run8(const float* p, u64* out) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    out[0] = pk(a.x, a.y); out[1] = pk(a.z, a.w); out[2] = pk(b.x, b.y); out[3] = pk(b.z, b.w);
}
// 8 values -> T, one or two 16-byte stores
__device__ __forceinline__ void wide_store8(__nv_bfloat16* dst, const u64* v) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float lo, hi;
        upk(v[j], lo, hi);
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void wide_store8(__half* dst, const u64* v) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float lo, hi;
        upk(v[j], lo, hi);
        const __half2 h = __floats2half2_rn(lo, hi);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void wide_store8(float* dst, const u64* v) {
    float a, b, c, d;
    upk(v[0], a, b); upk(v[1], c, d);
    reinterpret_cast<float4*>(dst)[0] = make_float4(a, b, c, d);
    upk(v[2], a, b); upk(v[3], c, d);
    reinterpret_cast<float4*>(dst)[1] = make_float4(a, b, c, d);
}
// the same, also at the same offset of every peer buffer of the push mode (plain stores over NVLink; n_push is 0
// unless the plan was given peers)
template <typename T>
__device__ __forceinline__ void wide_store8_push(T* dst, const u64* v, const StepArgs& a) {
    wide_store8(dst, v);
    for (int k = 0; k < a.n_push; ++k)
        wide_store8(reinterpret_cast<T*>(reinterpret_cast<unsigned char*>(dst) + a.push_delta[k]), v);
}
// the value a T-typed parameter holds after a store, for a packed pair
template <typename T> __device__ __forceinline__ u64 round_pair(u64 v);
template <> __device__ __forceinline__ u64 round_pair<float>(u64 v) { return v; }
template <> __device__ __forceinline__ u64 round_pair<__nv_bfloat16>(u64 v) {
    float lo, hi;
    upk(v, lo, hi);
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
    return pk_u32(w << 16, w & 0xffff0000u);
}
template <> __device__ __forceinline__ u64 round_pair<__half>(u64 v) {
    float lo, hi;
    upk(v, lo, hi);
    const float2 f = __half22float2(__floats2half2_rn(lo, hi));
    return pk(f.x, f.y);
}

// geometry of one work item, as the producer and the consumers need it
struct WideItem {
    const unsigned char* a_src;   // operand A (gradient or parameter), first byte of the tile
    const unsigned char* m_src;   // int8 codes, first byte of the tile
    const unsigned char* x_src;   // apply pass, tile layout: absmax of the first band's tiles (else null)
    int64_t a_pitch, m_pitch, x_pitch;
    int tensor, R, C, row0, col0, wcols, nbands, tr, tc;
};

template <typename TA>
__device__ __forceinline__ WideItem wide_item(const StepArgs& a, const Work& w, bool a_is_grad) {
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    WideItem it;
    it.tensor = w.tensor;
    it.R = (int)d.rows;
    it.C = (int)d.cols;
    it.tr = w.tile / s.ptiles_c;
    it.tc = w.tile - it.tr * s.ptiles_c;
    it.row0 = it.tr * W_TR;
    it.col0 = it.tc * W_TC;
    it.wcols = min(W_TC, it.C - it.col0);
    it.nbands = min(W_BANDS, (it.R - it.row0 + W_BAND - 1) / W_BAND);
    it.a_pitch = (int64_t)it.C * sizeof(TA);
    it.m_pitch = it.C;
    it.a_src = reinterpret_cast<const unsigned char*>(a_is_grad ? d.g : d.p) + (int64_t)it.row0 * it.a_pitch +
               (int64_t)it.col0 * sizeof(TA);
    it.m_src = reinterpret_cast<const unsigned char*>(d.m) + (int64_t)it.row0 * it.m_pitch + it.col0;
    it.x_pitch = (int64_t)(it.C >> 4) * sizeof(float);
    it.x_src = (d.mode == CAME_MODE_TILE8 && !a_is_grad)      // the apply pass only: the momentum pass loads it ahead itself
        ? reinterpret_cast<const unsigned char*>(d.m_absmax) + (int64_t)(it.row0 >> 4) * it.x_pitch + (it.col0 >> 4) * sizeof(float)
        : nullptr;
    return it;
}

// Warps 0..15 consume (compute); the warps after them produce: they only issue the copies, because a bulk-copy
// instruction blocks while the copy engine's queue is full and a band's 32 copies keep a warp busy for about as long
// as the consumers need for a band.  Per ring slot there is a "full" barrier (the producer's expect_tx + the copies'
// bytes) and an "empty" barrier (one arrival per consumer warp).  Nobody synchronises CTA-wide inside the band
// loop; consumer warps may drift apart by up to STAGES-1 bands.  A waiter that times out raises `abort` in
// shared memory; everybody polls it.
constexpr int W_CONSUMERS = W_THREADS;            // 512 consumer threads
constexpr int W_ALL_THREADS = W_THREADS + 32;     // + the producer warp

struct WideShared {
    uint64_t full[4];
    uint64_t empty[4];
    uint64_t ready[2];      // momentum pass: the helper warp has prepared the item of this buffer
    uint64_t done[2];       // momentum pass: every computing warp has finished the item of this buffer
    int abort;
    int pad[3];             // 112 bytes: what follows in shared memory stays 16-byte aligned (bulk-copy destinations)
};
static_assert(sizeof(WideShared) % 16 == 0, "the factor slices behind it are bulk-copy destinations");

// Bounded wait that also gives up when another warp raised `abort`.  On its own timeout it records the failure
// in the plan's status word and raises `abort`, so that every other waiter of the CTA leaves too.
__device__ __forceinline__ bool wide_wait(uint64_t* bar, uint32_t parity, WideShared* sh, const StepArgs& a, int lane,
                                          uint32_t limit = MBAR_SPIN_LIMIT) {
    volatile int* abort = &sh->abort;
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return *abort == 0;
        if ((i & 15u) == 15u && *abort) return false;
    }
    if (lane == 0) { atomicExch(a.status, STATUS_MBAR_TIMEOUT); atomicExch(&sh->abort, 1); }
    return false;
}
// after a failed wait: give the copies in flight one more bounded chance to land before the CTA's shared
// memory is released
__device__ __forceinline__ void wide_drain(WideShared* sh, int stages) {
    for (int i = 0; i < stages; ++i)
        for (uint32_t t = 0; t < (1u << 16); ++t)
            if (mbar_try_wait(&sh->full[i], 0) || mbar_try_wait(&sh->full[i], 1)) break;
}

// The copy stream of one CTA: every band of every work item of the CTA, in consumption order.
template <typename TA>
struct WideProducer {
    static constexpr int STAGES = WideCfg<TA>::STAGES;
    int item, band, q;
    bool live;
    WideItem it;
    uint64_t stream_policy;      // every operand of these passes is read once: first in line for eviction from L2
    __device__ __forceinline__ void init(const StepArgs& a, const Work* work, int n_items, bool a_is_grad) {
        stream_policy = l2_policy_evict_first();
        item = blockIdx.x; band = 0; q = 0;
        live = item < n_items;
        if (live) it = wide_item<TA>(a, work[item], a_is_grad);
    }
    // Issue the next band of the stream (all 32 lanes of a producer warp call this); false on a timed-out wait.
    // With `nprod` producer warps, warp `which` copies the bands whose stream position is `which` modulo nprod and
    // only steps over the others (one warp alone tops out near 5.7 TB/s of copies per GPU, two reach 6.5: measured
    // on the bare ring).
    __device__ __forceinline__ bool issue(const StepArgs& a, const Work* work, int n_items, bool a_is_grad,
                                          unsigned char* smem, WideShared* sh, int lane, int which = 0, int nprod = 1) {
        if (!live) return true;
        constexpr int STAGE = WideCfg<TA>::STAGE, ROW = WideCfg<TA>::ROW;
        if (nprod == 1 || q % nprod == which) {
            const int slot = q % STAGES;
            if (q >= STAGES) {   // every consumer warp must have released the slot's previous band
                if (!wide_wait(&sh->empty[slot], ((q / STAGES) - 1) & 1, sh, a, lane)) return false;
            }
            const int rows = min(W_BAND, it.R - it.row0 - band * W_BAND);
            const uint32_t a_bytes = (uint32_t)it.wcols * sizeof(TA), m_bytes = (uint32_t)it.wcols;
            const uint32_t x_bytes = it.x_src ? (uint32_t)(it.wcols >> 4) * sizeof(float) : 0u;   // a multiple of 16: wcols % 64 == 0
            if (lane == 0) {
                mbar_arrive_expect_tx(&sh->full[slot], (uint32_t)rows * (a_bytes + m_bytes) + x_bytes);
                if (x_bytes) bulk_g2s_hint(smem + slot * STAGE + WideCfg<TA>::AMAX_OFF, it.x_src + band * it.x_pitch, x_bytes, &sh->full[slot], stream_policy);
            }
            __syncwarp();
            const int r = lane & 15;
            if (r < rows) {
                const int64_t row = band * W_BAND + r;
                if (lane < 16) bulk_g2s_hint(smem + slot * STAGE + r * ROW, it.a_src + row * it.a_pitch, a_bytes, &sh->full[slot], stream_policy);
                else bulk_g2s_hint(smem + slot * STAGE + W_BAND * ROW + r * W_MROW, it.m_src + row * it.m_pitch, m_bytes, &sh->full[slot], stream_policy);
            }
        }
        ++q;
        if (++band == it.nbands) {
            band = 0;
            item += gridDim.x;
            live = item < n_items;
            if (live) it = wide_item<TA>(a, work[item], a_is_grad);
        }
        return true;
    }
};

// consumer side of one band: wait for the data
__device__ __forceinline__ bool wide_wait_full(const StepArgs& a, WideShared* sh, int slot, int parity, int lane) {
    return wide_wait(&sh->full[slot], (uint32_t)parity, sh, a, lane);
}
__device__ __forceinline__ void wide_release(WideShared* sh, int slot, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(&sh->empty[slot]);
}

// sum of x[0..n) computed by one warp (same order in every warp that calls it)
__device__ __forceinline__ float warp_vector_sum(const float* x, int n, int lane) {
    float t = 0.0f;
    for (int i = lane; i < n; i += 32) t += x[i];
    return warp_sum(t);
}

}  // namespace came
