// Fused first pass over the gradient: ONE read of g yields the row sums and column sums of g^2 (for the
// factored second moment) AND the column sums of g^2 / v_row (from which S = sum (g r c)^2, the quantity the
// RMS clip needs, follows without a second read of g):
//
//     S = sum_ij g_ij^2 r_i^2 c_j^2 = mean(v_row) * sum_j (1 / v_col_j) * T_j,   T_j = sum_i g_ij^2 / v_row_i
//
// which holds because r_i^2 = mean(v_row) / v_row_i and c_j^2 = 1 / v_col_j when no 1e-30 clamp is active
// (tensors carrying CAME_F_SQ_CLAMP take the two-pass kernels instead).  v_row_i needs the complete row,
// so a CTA owns whole rows: a strip of 128 rows, staged through shared memory in batches of `rb` rows by
// bulk asynchronous copies (three slots: two batches in flight while one is computed on), swept twice from
// shared memory.
//
// Replaces kUpdateSqRowQuantized, the column walk of kUpdateSqColQuantizedFinalize and kSumUpdateSq
// (came_kernels.cu:61-96, 198-243, 596-619), which read g three times.
#include "common.cuh"
#include "launch.h"
#include "pipeline.cuh"

#include <cstdio>

namespace came {

constexpr int FA_THREADS = 512;
constexpr int FA_WARPS = FA_THREADS / 32;
constexpr int FA_STAGES = 3;
constexpr int FA_RB_MAX = 16;

// 8 consecutive staged elements -> 4 packed fp32 pairs
__device__ __forceinline__ void smem_run8(const __nv_bfloat16* p, u64* out) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j] = pk_u32(w[j] << 16, w[j] & 0xffff0000u);
}
__device__ __forceinline__ void smem_run8(const __half* p, u64* out) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        out[j] = pk(f.x, f.y);
    }
}
__device__ __forceinline__ void smem_run8(const float* p, u64* out) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    out[0] = pk(a.x, a.y); out[1] = pk(a.z, a.w); out[2] = pk(b.x, b.y); out[3] = pk(b.z, b.w);
}

// Sum N per-lane values v[0..N) over the 32 lanes of a warp with a halving butterfly: after log2(N) exchange
// steps every lane holds one row's partial, the remaining steps finish it.  Lane L ends with the total of row
// (L >> (5 - log2 N)) & (N - 1)   (N = 16: (L >> 1) & 15, N = 8: (L >> 2) & 7, N = 4: (L >> 3) & 3).
template <int N>
__device__ __forceinline__ float warp_reduce_rows(float* v, int lane) {
    int mask = 16;
#pragma unroll
    for (int n = N; n > 1; n >>= 1, mask >>= 1) {
        const bool upper = (lane & mask) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float send = upper ? v[i] : v[i + n / 2];
            const float keep = upper ? v[i + n / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
        }
    }
    float t = v[0];
#pragma unroll
    for (; mask > 0; mask >>= 1) t += __shfl_xor_sync(0xffffffffu, t, mask);
    return t;
}

// Shared bookkeeping of one CTA: ring barriers and the abort flag every waiter polls (same protocol as the momentum / apply passes).
struct FaShared {
    uint64_t full[FA_STAGES];
    uint64_t empty[FA_STAGES];
    int abort;
    int pad;
};

__device__ __forceinline__ bool fa_wait(uint64_t* bar, uint32_t parity, FaShared* sh, const StepArgs& a, int lane) {
    volatile int* abort = &sh->abort;
    for (uint32_t i = 0; i < MBAR_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return *abort == 0;
        if ((i & 15u) == 15u && *abort) return false;
    }
    if (lane == 0) { atomicExch(a.status, STATUS_MBAR_TIMEOUT); atomicExch(&sh->abort, 1); }
    return false;
}

// Warps 0..15 compute; warp 16 only issues the bulk copies (a bulk-copy instruction blocks while the copy
// engine's queue is full, which would otherwise stall a computing warp for about as long as a batch takes).
template <typename TG, int NG>
__global__ void __launch_bounds__(FA_THREADS + 32, 1) k_sqstat_fused(StepArgs a, const Work* __restrict__ work) {
    // most rows a batch can hold for this column count.  One column group per thread (cols <= 4096): batches are
    // capped at 4 rows and the squares stay in registers between the two sweeps instead of being re-read.
    constexpr bool KEEP = NG == 1;
    constexpr int RBM = NG == 1 ? 4 : (NG == 2 ? 8 : 4);
    extern __shared__ __align__(128) unsigned char smem[];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const int R = (int)d.rows, C = (int)d.cols;
    const int rb = s.fa_rb;
    const int row_bytes = C * (int)sizeof(TG);
    const int stage_bytes = rb * row_bytes;
    FaShared* sh = reinterpret_cast<FaShared*>(smem + FA_STAGES * stage_bytes);
    float* s_part = reinterpret_cast<float*>(sh + 1);                // [2][FA_WARPS][FA_RB_MAX], double-buffered by batch
    float* s_old = s_part + 2 * FA_WARPS * FA_RB_MAX;                // [K_TR] dequantised old v_row of the strip's rows

    const int strip = w.tile;
    const int row0 = strip * K_TR;
    const int nrows = min(K_TR, R - row0);
    const int nbatch = (nrows + rb - 1) / rb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned char* g_src = reinterpret_cast<const unsigned char*>(d.g);

    if (threadIdx.x == 0) {
        for (int i = 0; i < FA_STAGES; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], FA_WARPS); }
        sh->abort = 0;
        mbar_init_fence();
    }
    // old second-moment state of the strip's rows, fetched once (a dependent global load per batch would sit on
    // every warp's critical path)
    if (threadIdx.x < nrows) {
        const int row = row0 + threadIdx.x;
        s_old[threadIdx.x] = d.mode != CAME_MODE_FP32
            ? (float)reinterpret_cast<const uint8_t*>(d.sq_row)[row] * (d.sq_row_absmax[row >> 8] / QMAX_U8)
            : reinterpret_cast<const float*>(d.sq_row)[row];
    }
    __syncthreads();

    if (warp == FA_WARPS) {      // producer: lane r copies row r of batch b
        for (int b = 0; b < nbatch; ++b) {
            const int slot = b % FA_STAGES;
            if (b >= FA_STAGES && !fa_wait(&sh->empty[slot], ((b / FA_STAGES) - 1) & 1, sh, a, lane)) return;
            const int rows = min(rb, nrows - b * rb);
            if (lane == 0) mbar_arrive_expect_tx(&sh->full[slot], (uint32_t)rows * (uint32_t)row_bytes);
            __syncwarp();
            if (lane < rows)
                bulk_g2s(smem + slot * stage_bytes + lane * row_bytes, g_src + (int64_t)(row0 + b * rb + lane) * row_bytes,
                         (uint32_t)row_bytes, &sh->full[slot]);
        }
        return;
    }

    // this thread's column groups: 8 consecutive columns starting at 8 * (threadIdx.x + FA_THREADS * j)
    bool gvalid[NG];
    u64 colb[NG][4], colT[NG][4];
#pragma unroll
    for (int j = 0; j < NG; ++j) {
        gvalid[j] = (threadIdx.x + FA_THREADS * j) * 8 < C;
#pragma unroll
        for (int e = 0; e < 4; ++e) { colb[j][e] = F2ZERO; colT[j][e] = F2ZERO; }
    }
    bool ok = true;
#ifdef CAME_WIDE_PROFILE
    long long pf_wait = 0, pf_s1 = 0, pf_bar = 0, pf_fin = 0, pf_s2 = 0;
    const long long pf_start = clock64();
#endif

    for (int b = 0; b < nbatch; ++b) {
        const int slot = b % FA_STAGES;
        // After a failed wait a warp keeps walking the batches without touching data, so that it still meets
        // the other consumer warps at the hardware barrier below once per batch (nobody is left waiting).
#ifdef CAME_WIDE_PROFILE
        const long long c0 = clock64();
#endif
        if (ok && !fa_wait(&sh->full[slot], (b / FA_STAGES) & 1, sh, a, lane)) ok = false;
#ifdef CAME_WIDE_PROFILE
        const long long c1 = clock64();
#endif
        if (!ok) { named_sync(1, FA_THREADS); continue; }
        const int rows = min(rb, nrows - b * rb);
        const unsigned char* st = smem + slot * stage_bytes;
        float* part = s_part + (b & 1) * (FA_WARPS * FA_RB_MAX);

        // sweep 1: row sums and column sums of g^2.  Row partials stay in registers (static indices: the loops
        // are fully unrolled and guarded) and are reduced across the warp together.
        float rp[RBM];
        u64 sqk[KEEP ? RBM : 1][4];      // KEEP: g^2 of this thread's elements, reused by sweep 2
#pragma unroll
        for (int r = 0; r < RBM; ++r) {
            rp[r] = 0.0f;
            if (KEEP) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sqk[KEEP ? r : 0][e] = F2ZERO;
            }
            if (r < rows) {
                u64 racc = F2ZERO;
#pragma unroll
                for (int j = 0; j < NG; ++j) {
                    if (gvalid[j]) {
                        u64 g2[4];
                        smem_run8(reinterpret_cast<const TG*>(st + r * row_bytes) + (threadIdx.x + FA_THREADS * j) * 8, g2);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (KEEP) {
                                const u64 sq = mul2(g2[e], g2[e]);
                                sqk[KEEP ? r : 0][e] = sq;
                                colb[j][e] = add2(colb[j][e], sq);
                                racc = add2(racc, sq);
                            } else {
                                colb[j][e] = fma2(g2[e], g2[e], colb[j][e]);
                                racc = fma2(g2[e], g2[e], racc);
                            }
                        }
                    }
                }
                rp[r] = racc.x + racc.y;
            }
        }
        if (KEEP) {      // the slot's bytes are in registers: hand it back before the barrier
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->empty[slot]);
        }
        if (RBM > 8 && rows > 8) {
            float v16[16];
#pragma unroll
            for (int r = 0; r < 16; ++r) v16[r] = r < RBM ? rp[r] : 0.0f;
            const float t = warp_reduce_rows<16>(v16, lane);
            if ((lane & 1) == 0) part[warp * FA_RB_MAX + ((lane >> 1) & 15)] = t;
        } else if (RBM > 4 && rows > 4) {
            float v8[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) v8[r] = r < RBM ? rp[r] : 0.0f;
            const float t = warp_reduce_rows<8>(v8, lane);
            if ((lane & 3) == 0) part[warp * FA_RB_MAX + ((lane >> 2) & 7)] = t;
        } else {
            float v4[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) v4[r] = rp[r];
            const float t = warp_reduce_rows<4>(v4, lane);
            if ((lane & 7) == 0) part[warp * FA_RB_MAX + ((lane >> 3) & 3)] = t;
        }
        // barrier among the 16 consumer warps: the per-warp row partials of this batch are complete
#ifdef CAME_WIDE_PROFILE
        const long long c2 = clock64();
#endif
        named_sync(1, FA_THREADS);
#ifdef CAME_WIDE_PROFILE
        const long long c3 = clock64();
#endif

        // every warp finishes the row sums itself (lane r: row r), so no second barrier is needed; warp 0
        // publishes v_row.  Mean of g^2 + eps0 over the row (came_kernels.cu:77-88), EMA with the dequantised state.
        float wrow = 0.0f;
        if (lane < rows) {
            float sum = 0.0f;
#pragma unroll
            for (int ww = 0; ww < FA_WARPS; ++ww) sum += part[ww * FA_RB_MAX + lane];
            const int row = row0 + b * rb + lane;
            const float mean = (sum + (float)C * h.eps0) / (float)C;
            const float v = s_old[b * rb + lane] * h.beta2 + h.om_beta2 * mean;
            if (warp == 0) s.vr[row] = v;
            wrow = v > 0.0f ? 1.0f / v : 0.0f;
        }
#ifdef CAME_WIDE_PROFILE
        const long long c4 = clock64();
#endif
        // sweep 2: column sums of g^2 / v_row
#pragma unroll
        for (int r = 0; r < RBM; ++r) {
            if (r < rows) {
                const u64 w2 = splat(__shfl_sync(0xffffffffu, wrow, r));
                if (KEEP) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) colT[0][e] = fma2(sqk[KEEP ? r : 0][e], w2, colT[0][e]);
                } else {
#pragma unroll
                    for (int j = 0; j < NG; ++j) {
                        if (gvalid[j]) {
                            u64 g2[4];
                            smem_run8(reinterpret_cast<const TG*>(st + r * row_bytes) + (threadIdx.x + FA_THREADS * j) * 8, g2);
#pragma unroll
                            for (int e = 0; e < 4; ++e) colT[j][e] = fma2(mul2(g2[e], g2[e]), w2, colT[j][e]);
                        }
                    }
                }
            }
        }
        if (!KEEP) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->empty[slot]);
        }
#ifdef CAME_WIDE_PROFILE
        const long long c5 = clock64();
        pf_wait += c1 - c0; pf_s1 += c2 - c1; pf_bar += c3 - c2; pf_fin += c4 - c3; pf_s2 += c5 - c4;
#endif
    }
#ifdef CAME_WIDE_PROFILE
    if ((blockIdx.x == 0 || blockIdx.x == 200) && lane == 0 && (warp == 0 || warp == 9))
        printf("sqstat NG %d cta %d warp %d rb %d: total %lld wait %lld sweep1 %lld barrier %lld finalize %lld sweep2 %lld batches %d\n", NG,
               blockIdx.x, warp, rb, clock64() - pf_start, pf_wait, pf_s1, pf_bar, pf_fin, pf_s2, nbatch);
#endif
    if (!ok) return;      // the status word is set; the partial sums of this strip stay unwritten
#pragma unroll
    for (int j = 0; j < NG; ++j) {
        if (gvalid[j]) {
            const int64_t off = (int64_t)strip * C + (threadIdx.x + FA_THREADS * j) * 8;
            reinterpret_cast<float4*>(s.colpart + off)[0] = make_float4(colb[j][0].x, colb[j][0].y, colb[j][1].x, colb[j][1].y);
            reinterpret_cast<float4*>(s.colpart + off)[1] = make_float4(colb[j][2].x, colb[j][2].y, colb[j][3].x, colb[j][3].y);
            reinterpret_cast<float4*>(s.tpart + off)[0] = make_float4(colT[j][0].x, colT[j][0].y, colT[j][1].x, colT[j][1].y);
            reinterpret_cast<float4*>(s.tpart + off)[1] = make_float4(colT[j][2].x, colT[j][2].y, colT[j][3].x, colT[j][3].y);
        }
    }
}

// rows per staged batch for a row of `row_bytes`: as many as fit 64 KB per slot; at most 4 when a thread owns a
// single column group (cols <= 4096), else at most 8
int fused_sq_rows_per_batch(int64_t row_bytes, int64_t cols) {
    int64_t rb = (64 * 1024) / row_bytes;
    const int64_t cap = cols <= (int64_t)FA_THREADS * 8 ? 4 : 8;
    if (rb > cap) rb = cap;
    if (rb < 1) rb = 1;
    return (int)rb;
}

bool fused_sq_eligible(int64_t cols, int elem_bytes) {
    return cols % 8 == 0 && cols <= (int64_t)FA_THREADS * 8 * 4 && cols * elem_bytes <= 64 * 1024;
}

template <typename TG, int NG>
static cudaError_t launch_one(const StepArgs& a, const Work* work, int n, size_t smem, cudaStream_t st) {
    cudaError_t e = cudaFuncSetAttribute(k_sqstat_fused<TG, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    k_sqstat_fused<TG, NG><<<n, FA_THREADS + 32, smem, st>>>(a, work);
    return cudaGetLastError();
}

template <typename TG>
static cudaError_t launch_ng(int ng, const StepArgs& a, const Work* work, int n, size_t smem, cudaStream_t st) {
    switch (ng) {
        case 1: return launch_one<TG, 1>(a, work, n, smem, st);
        case 2: return launch_one<TG, 2>(a, work, n, smem, st);
        case 3: return launch_one<TG, 3>(a, work, n, smem, st);
        default: return launch_one<TG, 4>(a, work, n, smem, st);
    }
}

// key.mode carries the number of column groups per thread (1..4); all tensors of one launch share it and
// `max_stage_bytes` is the largest slot (rows per batch x row bytes) among them
cudaError_t launch_fused_sq(const KernelKey& key, const StepArgs& a, const Work* work, int n, size_t max_stage_bytes,
                            cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    const size_t smem = FA_STAGES * max_stage_bytes + sizeof(FaShared) + (2 * FA_WARPS * FA_RB_MAX + K_TR) * sizeof(float);
    switch (key.g_dtype) {
        case CAME_DT_F32: return launch_ng<float>(key.mode, a, work, n, smem, st);
        case CAME_DT_F16: return launch_ng<__half>(key.mode, a, work, n, smem, st);
        default: return launch_ng<__nv_bfloat16>(key.mode, a, work, n, smem, st);
    }
}

}  // namespace came
