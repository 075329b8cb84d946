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

constexpr int FA_MAX_STAGES = 8;

// Shared bookkeeping of one CTA: ring barriers and the abort flag every waiter polls (same protocol as the
// momentum / apply passes).
struct FaShared {
    uint64_t full[FA_MAX_STAGES];
    uint64_t empty[FA_MAX_STAGES];
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
//
// GROUPS = 2 (matrices of at most 2048 columns): the computing warps form two groups of 8 that take alternate
// batches, each with its own barrier, so that one group sweeps while the other sits in the latency of its
// row-sum exchange; each group spans a whole row with 256 threads, which also keeps every thread busy down to
// 2048 columns.  NG = column groups (of 8 columns) per thread within its group.
// KEEP (NG <= 2): batches are small enough for the squares to stay in registers between the two sweeps.
template <typename TG, int NG, int GROUPS>
__global__ void __launch_bounds__(FA_THREADS + 32, 1) k_sqstat_fused(StepArgs a, const Work* __restrict__ work) {
    constexpr bool KEEP = NG <= 2;
    constexpr int RBM = KEEP ? 4 / NG : 4;                 // most rows of a batch (the plan sizes batches accordingly)
    constexpr int GT = FA_THREADS / GROUPS;                // threads of a group
    constexpr int WPG = FA_WARPS / GROUPS;                 // warps of a group
    extern __shared__ __align__(128) unsigned char smem[];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const int R = (int)d.rows, C = (int)d.cols;
    const int rb = s.fa_rb, nstages = s.fa_stages;
    const int row_bytes = C * (int)sizeof(TG);
    const int stage_bytes = rb * row_bytes;
    FaShared* sh = reinterpret_cast<FaShared*>(smem + nstages * stage_bytes);
    float* s_part = reinterpret_cast<float*>(sh + 1);                // [2][FA_WARPS][4], double-buffered by batch
    float* s_old = s_part + 2 * FA_WARPS * 4;                        // [K_TR] dequantised old v_row of the strip's rows

    const int strip = w.tile;
    const int row0 = strip * K_TR;
    const int nrows = min(K_TR, R - row0);
    const int nbatch = (nrows + rb - 1) / rb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned char* g_src = reinterpret_cast<const unsigned char*>(d.g);

    if (threadIdx.x == 0) {
        for (int i = 0; i < nstages; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], WPG); }
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
        int slot = 0;
        uint32_t phase = 1;      // parity of the slot's previous use (meaningless during the first lap)
        for (int b = 0; b < nbatch; ++b, ++slot) {
            if (slot == nstages) { slot = 0; phase ^= 1u; }
            if (b >= nstages && !fa_wait(&sh->empty[slot], phase, sh, a, lane)) return;
            const int rows = min(rb, nrows - b * rb);
            if (lane == 0) mbar_arrive_expect_tx(&sh->full[slot], (uint32_t)rows * (uint32_t)row_bytes);
            __syncwarp();
            if (lane < rows)
                bulk_g2s(smem + slot * stage_bytes + lane * row_bytes, g_src + (int64_t)(row0 + b * rb + lane) * row_bytes,
                         (uint32_t)row_bytes, &sh->full[slot]);
        }
        return;
    }

    const int group = threadIdx.x / GT, tig = threadIdx.x - group * GT, wig = warp - group * WPG;
    // this thread's column groups: 8 consecutive columns starting at 8 * (tig + GT * j)
    bool gvalid[NG];
    u64 colb[NG][4], colT[NG][4];
#pragma unroll
    for (int j = 0; j < NG; ++j) {
        gvalid[j] = (tig + GT * j) * 8 < C;
#pragma unroll
        for (int e = 0; e < 4; ++e) { colb[j][e] = F2ZERO; colT[j][e] = F2ZERO; }
    }
    bool ok = true;
    int nb_done = 0;       // batches this group has gone through (selects the s_part buffer)

    int slot = group;      // ring position of batch b, advanced without a division (GROUPS <= slots)
    uint32_t phase = 0;
    for (int b = group; b < nbatch; b += GROUPS, ++nb_done, slot += GROUPS) {
        if (slot >= nstages) { slot -= nstages; phase ^= 1u; }
        // After a failed wait a warp keeps walking its batches without touching data, so that it still meets
        // the other warps of its group at the hardware barrier below once per batch (nobody is left waiting).
        if (ok && !fa_wait(&sh->full[slot], phase, sh, a, lane)) ok = false;
        if (!ok) { named_sync(1 + group, GT); continue; }
        const int rows = min(rb, nrows - b * rb);
        const unsigned char* st = smem + slot * stage_bytes;
        float* part = s_part + (nb_done & 1) * (FA_WARPS * 4) + group * (WPG * 4);

        // sweep 1: row sums and column sums of g^2.  Row partials stay in registers (static indices: the loops
        // are fully unrolled and guarded) and are reduced across the warp together.
        float rp[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        u64 sqk[KEEP ? RBM : 1][KEEP ? NG : 1][4];      // KEEP: g^2 of this thread's elements, reused by sweep 2
#pragma unroll
        for (int r = 0; r < RBM; ++r) {
            if (KEEP) {
#pragma unroll
                for (int j = 0; j < NG; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) sqk[KEEP ? r : 0][KEEP ? j : 0][e] = F2ZERO;
            }
            if (r < rows) {
                u64 racc = F2ZERO;
#pragma unroll
                for (int j = 0; j < NG; ++j) {
                    if (gvalid[j]) {
                        u64 g2[4];
                        smem_run8(reinterpret_cast<const TG*>(st + r * row_bytes) + (tig + GT * j) * 8, g2);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (KEEP) {
                                const u64 sq = mul2(g2[e], g2[e]);
                                sqk[KEEP ? r : 0][KEEP ? j : 0][e] = sq;
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
        {
            const float t = warp_reduce_rows<4>(rp, lane);
            if ((lane & 7) == 0) part[wig * 4 + ((lane >> 3) & 3)] = t;
        }
        // barrier among the warps of this group: the per-warp row partials of the batch are complete
        named_sync(1 + group, GT);

        // every warp finishes the row sums itself (lane r: row r), so no second barrier is needed; the group's first
        // warp publishes v_row.  Mean of g^2 + eps0 over the row (came_kernels.cu:77-88), EMA with the old state.
        float wrow = 0.0f;
        if (lane < rows) {
            float sum = 0.0f;
#pragma unroll
            for (int ww = 0; ww < WPG; ++ww) sum += part[ww * 4 + lane];
            const int row = row0 + b * rb + lane;
            const float mean = (sum + (float)C * h.eps0) / (float)C;
            const float v = s_old[b * rb + lane] * h.beta2 + h.om_beta2 * mean;
            if (wig == 0) s.vr[row] = v;
            wrow = v > 0.0f ? 1.0f / v : 0.0f;
        }
        // sweep 2: column sums of g^2 / v_row
#pragma unroll
        for (int r = 0; r < RBM; ++r) {
            if (r < rows) {
                const u64 w2 = splat(__shfl_sync(0xffffffffu, wrow, r));
#pragma unroll
                for (int j = 0; j < NG; ++j) {
                    if (KEEP) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) colT[j][e] = fma2(sqk[KEEP ? r : 0][KEEP ? j : 0][e], w2, colT[j][e]);
                    } else if (gvalid[j]) {
                        u64 g2[4];
                        smem_run8(reinterpret_cast<const TG*>(st + r * row_bytes) + (tig + GT * j) * 8, g2);
#pragma unroll
                        for (int e = 0; e < 4; ++e) colT[j][e] = fma2(mul2(g2[e], g2[e]), w2, colT[j][e]);
                    }
                }
            }
        }
        if (!KEEP) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->empty[slot]);
        }
    }
    if (!ok) return;      // the status word is set; the partial sums of this strip stay unwritten
    // one set of column partials per (strip, group)
#pragma unroll
    for (int j = 0; j < NG; ++j) {
        if (gvalid[j]) {
            const int64_t off = (int64_t)(strip * GROUPS + group) * C + (tig + GT * j) * 8;
            reinterpret_cast<float4*>(s.colpart + off)[0] = make_float4(colb[j][0].x, colb[j][0].y, colb[j][1].x, colb[j][1].y);
            reinterpret_cast<float4*>(s.colpart + off)[1] = make_float4(colb[j][2].x, colb[j][2].y, colb[j][3].x, colb[j][3].y);
            reinterpret_cast<float4*>(s.tpart + off)[0] = make_float4(colT[j][0].x, colT[j][0].y, colT[j][1].x, colT[j][1].y);
            reinterpret_cast<float4*>(s.tpart + off)[1] = make_float4(colT[j][2].x, colT[j][2].y, colT[j][3].x, colT[j][3].y);
        }
    }
}

// Geometry of the fused first pass for a matrix of `cols` columns of `elem_bytes` each:
//   groups   2 up to 2048 columns (two 8-warp groups on alternate batches), else 1
//   ng       column groups of 8 per thread within its group (1..4)
//   rb       rows per staged batch: at most 4/ng while the squares are kept in registers (ng <= 2), at most 4
//            otherwise, and never more than fit 64 KB
//   stages   ring slots: as many as fit ~160 KB, between 3 and 8
void fused_sq_geometry(int64_t cols, int elem_bytes, int* groups, int* ng, int* rb, int* stages) {
    const int g = cols <= (int64_t)FA_THREADS * 4 ? 2 : 1;
    const int gt = FA_THREADS / g;
    const int n = (int)((cols / 8 + gt - 1) / gt);
    const int64_t row_bytes = cols * elem_bytes;
    int64_t r = (64 * 1024) / row_bytes;
    const int64_t cap = n <= 2 ? 4 / n : 4;
    if (r > cap) r = cap;
    if (r < 1) r = 1;
    int64_t st = (160 * 1024) / (r * row_bytes);
    if (st > FA_MAX_STAGES) st = FA_MAX_STAGES;
    if (st < 3) st = 3;
    *groups = g; *ng = n < 1 ? 1 : n; *rb = (int)r; *stages = (int)st;
}

bool fused_sq_eligible(int64_t cols, int elem_bytes) {
    return cols % 8 == 0 && cols <= (int64_t)FA_THREADS * 8 * 4 && cols * elem_bytes <= 64 * 1024;
}

template <typename TG, int NG, int GROUPS>
static cudaError_t launch_one(const StepArgs& a, const Work* work, int n, size_t smem, cudaStream_t st) {
    cudaError_t e = cudaFuncSetAttribute(k_sqstat_fused<TG, NG, GROUPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    k_sqstat_fused<TG, NG, GROUPS><<<n, FA_THREADS + 32, smem, st>>>(a, work);
    return cudaGetLastError();
}

template <typename TG>
static cudaError_t launch_ng(int ng, int groups, const StepArgs& a, const Work* work, int n, size_t smem, cudaStream_t st) {
    if (groups == 2) return launch_one<TG, 1, 2>(a, work, n, smem, st);      // at most 2048 columns: one column group per thread
    switch (ng) {
        case 1: return launch_one<TG, 1, 1>(a, work, n, smem, st);
        case 2: return launch_one<TG, 2, 1>(a, work, n, smem, st);
        case 3: return launch_one<TG, 3, 1>(a, work, n, smem, st);
        default: return launch_one<TG, 4, 1>(a, work, n, smem, st);
    }
}

// key.mode carries ng | (groups << 4); all tensors of one launch share it and `max_ring_bytes` is the largest
// ring (slots x rows per batch x row bytes) among them
cudaError_t launch_fused_sq(const KernelKey& key, const StepArgs& a, const Work* work, int n, size_t max_ring_bytes,
                            cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    const size_t smem = max_ring_bytes + sizeof(FaShared) + (2 * FA_WARPS * 4 + K_TR) * sizeof(float);
    const int ng = key.mode & 15, groups = key.mode >> 4;
    switch (key.g_dtype) {
        case CAME_DT_F32: return launch_ng<float>(ng, groups, a, work, n, smem, st);
        case CAME_DT_F16: return launch_ng<__half>(ng, groups, a, work, n, smem, st);
        default: return launch_ng<__nv_bfloat16>(ng, groups, a, work, n, smem, st);
    }
}

}  // namespace came
