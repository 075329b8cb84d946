// Fused first pass over the gradient: ONE read of g yields the row sums and column sums of g^2 (for the
// factored second moment) AND the column sums of g^2 / v_row (from which S = sum (g r c)^2, the quantity the
// RMS clip needs, follows without a second read of g):
//
//     S = sum_ij g_ij^2 r_i^2 c_j^2 = mean(v_row) * sum_j (1 / v_col_j) * T_j,   T_j = sum_i g_ij^2 / v_row_i
//
// which holds because r_i^2 = mean(v_row) / v_row_i and c_j^2 = 1 / v_col_j when no 1e-30 clamp is active
// (tensors carrying CAME_F_SQ_CLAMP take the two-pass kernels instead).  v_row_i needs the complete row,
// so a CTA owns whole rows: a strip of 128 rows, staged through shared memory in batches of `rb` rows by
// bulk asynchronous copies into a ring of three to eight slots, swept twice from
// shared memory.
//
// Replaces kUpdateSqRowQuantized, the column walk of kUpdateSqColQuantizedFinalize and kSumUpdateSq
// (came_kernels.cu:61-96, 198-243, 596-619), which read g three times.
#include "common.cuh"
#include "launch.h"
#include "pipeline.cuh"

#include <cstdio>
#include <algorithm>
#include <cstdlib>

namespace came {

constexpr int FA_THREADS = 512;
constexpr int FA_WARPS = FA_THREADS / 32;
constexpr int FA_RB = 16;          // most rows of a staged batch (one per computing warp)

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
// A batch of rb rows (a power of two, at most 16) is swept twice from shared memory with two different
// thread mappings:
//   row sweep     the 16 warps split the batch into 16 row pieces (16 / rb pieces per row); a warp sums the
//                 squares of its piece, so a row sum costs one warp reduction and 16 / rb partials in shared
//                 memory -- no cross-warp tree, and the row's new v_row is completed once per warp;
//   column sweep  a thread owns the same 8 consecutive columns (NG such groups) for every row and accumulates
//                 g^2 and g^2 / v_row down the columns.  RS = 2 (matrices of at most 2048 columns): the
//                 threads form two sets that take the even and the odd rows of a batch, which keeps every
//                 thread busy; each set leaves its own column partials.
// Software pipeline: the row sweep of batch i+1 is issued before the column sweep of batch i, with one hardware
// barrier per batch, so the exchange of row partials never stalls the warps.  A warp holds two ring slots.
template <typename TG, int NG, int RS>
__global__ void __launch_bounds__(FA_THREADS + 32, 1) k_sqstat_fused(StepArgs a, const Work* __restrict__ work) {
    extern __shared__ __align__(128) unsigned char smem[];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const int R = (int)d.rows, C = (int)d.cols;
    const int rb = s.fa_rb, nstages = s.fa_stages;
    // everything the batch loop needs from the tables in global memory, read once: the barriers in the loop are
    // memory fences for the compiler, which would otherwise reload these on every batch
    const float eps0C = (float)C * h.eps0, fC = (float)C, beta2 = h.beta2, om_beta2 = h.om_beta2;
    float* const vr = s.vr;
    float* const colpart = s.colpart;
    float* const tpart = s.tpart;
    const int row_bytes = C * (int)sizeof(TG);
    const int stage_bytes = rb * row_bytes;
    FaShared* sh = reinterpret_cast<FaShared*>(smem + nstages * stage_bytes);
    float* s_part = reinterpret_cast<float*>(sh + 1);                // [2][FA_WARPS] row-piece sums, double-buffered by batch
    float* s_old = s_part + 2 * FA_WARPS;                            // [K_TR] dequantised old v_row of the strip's rows

    const int strip = w.tile;
    const int row0 = strip * K_TR;
    const int nrows = min(K_TR, R - row0);
    const int nbatch = (nrows + rb - 1) / rb;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned char* g_src = reinterpret_cast<const unsigned char*>(d.g);

    if (threadIdx.x == 0) {
        for (int i = 0; i < nstages; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], FA_WARPS); }
        sh->abort = 0;
        mbar_init_fence();
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

    // old second-moment state of the strip's rows, fetched once while the first copies are in flight (a dependent
    // global load per batch would sit on every warp's critical path)
    if (threadIdx.x < nrows) {
        const int row = row0 + threadIdx.x;
        s_old[threadIdx.x] = d.mode != CAME_MODE_FP32
            ? (float)reinterpret_cast<const uint8_t*>(d.sq_row)[row] * (d.sq_row_absmax[row >> 8] / QMAX_U8)
            : reinterpret_cast<const float*>(d.sq_row)[row];
    }
    named_sync(1, FA_THREADS);

    // row sweep: this warp's row of a batch and its span of 8-column groups within the row
    const int ncg = C >> 3;                      // 8-column groups per row
    const int ppr = FA_WARPS / rb;               // pieces per row (rb is a power of two <= 16)
    const int my_row = warp / ppr, my_piece = warp - my_row * ppr;
    const int cg_lo = (int)((int64_t)my_piece * ncg / ppr), cg_hi = (int)((int64_t)(my_piece + 1) * ncg / ppr);
    const int piece_chunks = (cg_hi - cg_lo) >> 5, piece_rem = (cg_hi - cg_lo) & 31;
    // column sweep: row set (RS = 2: even / odd rows) and 8-column groups of this thread
    constexpr int ST = FA_THREADS / RS;          // threads of a row set
    const int rset = threadIdx.x / ST, tis = threadIdx.x - rset * ST;
    // a thread whose group lies beyond the last column sweeps group 0 instead and drops the result: the sweep
    // itself then needs no per-group test
    bool gvalid[NG];
    int coff[NG];
    u64 colb[NG][4], colT[NG][4];
#pragma unroll
    for (int j = 0; j < NG; ++j) {
        gvalid[j] = tis + ST * j < ncg;
        coff[j] = (gvalid[j] || NG > 2) ? (tis + ST * j) * 8 : 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) { colb[j][e] = F2ZERO; colT[j][e] = F2ZERO; }
    }

    auto row_sweep = [&](int b, int slot, float* part) {
        const int rows = min(rb, nrows - b * rb);
        float t = 0.0f;
        if (my_row < rows) {
            const TG* src = reinterpret_cast<const TG*>(smem + slot * stage_bytes + my_row * row_bytes);
            u64 acc[4] = {F2ZERO, F2ZERO, F2ZERO, F2ZERO};
            // whole 32-group chunks without a per-lane test, then the ragged end of the piece
            const TG* p = src + (cg_lo + lane) * 8;
#pragma unroll 4
            for (int i = 0; i < piece_chunks; ++i, p += 256) {
                u64 g2[4];
                smem_run8(p, g2);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] = fma2(g2[e], g2[e], acc[e]);
            }
            if (lane < piece_rem) {
                u64 g2[4];
                smem_run8(p, g2);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] = fma2(g2[e], g2[e], acc[e]);
            }
            const u64 q = add2(add2(acc[0], acc[1]), add2(acc[2], acc[3]));
            t = q.x + q.y;
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) t += __shfl_xor_sync(0xffffffffu, t, m);
        if (lane == 0) part[warp] = t;
    };
    // completes the row sums of batch b (each warp for itself, lane r: row r, so no second barrier is needed; warp 0
    // publishes v_row), then the column sweep.  Mean of g^2 + eps0 over the row (came_kernels.cu:77-88), EMA with
    // the old state.
    auto col_sweep = [&](int b, int slot, const float* part) {
        const int rows = min(rb, nrows - b * rb);
        const unsigned char* st = smem + slot * stage_bytes;
        float wrow = 0.0f;
        if (lane < rows) {
            float sum = 0.0f;
            for (int q = 0; q < ppr; ++q) sum += part[lane * ppr + q];
            const int row = row0 + b * rb + lane;
            const float mean = (sum + eps0C) / fC;
            const float v = s_old[b * rb + lane] * beta2 + om_beta2 * mean;
            if (warp == 0) vr[row] = v;
            wrow = v > 0.0f ? 1.0f / v : 0.0f;
        }
        // rows of this thread's set; the trip count is uniform across the warp, so the shuffle is converged
        const TG* src = reinterpret_cast<const TG*>(st + rset * row_bytes);
#pragma unroll 2
        for (int r = rset; r < rows; r += RS, src += RS * C) {
            const u64 w2 = splat(__shfl_sync(0xffffffffu, wrow, r));
#pragma unroll
            for (int j = 0; j < NG; ++j) {
                if (NG <= 2 || gvalid[j]) {      // wide rows keep the test: without it the offsets cost registers they lack
                    u64 g2[4];
                    smem_run8(src + coff[j], g2);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const u64 sq = mul2(g2[e], g2[e]);
                        colb[j][e] = add2(colb[j][e], sq);
                        colT[j][e] = fma2(sq, w2, colT[j][e]);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->empty[slot]);
    };

    // After a failed wait a warp keeps walking its batches without touching data, so that it still meets the
    // other warps at the hardware barrier once per batch (nobody is left waiting).
    bool ok = true;
    int slot = 0;      // ring position advanced without a division
    uint32_t phase = 0;
    float* part_cur = s_part;
    float* part_nxt = s_part + FA_WARPS;
    if (fa_wait(&sh->full[0], 0, sh, a, lane)) row_sweep(0, 0, part_cur);
    else ok = false;
    named_sync(1, FA_THREADS);
    for (int b = 0; b < nbatch; ++b) {
        int nslot = slot + 1;
        uint32_t nphase = phase;
        if (nslot == nstages) { nslot = 0; nphase ^= 1u; }
        if (ok && b + 1 < nbatch) {
            if (fa_wait(&sh->full[nslot], nphase, sh, a, lane)) row_sweep(b + 1, nslot, part_nxt);
            else ok = false;
        }
        if (ok) col_sweep(b, slot, part_cur);
        named_sync(1, FA_THREADS);
        slot = nslot; phase = nphase;
        float* t = part_cur; part_cur = part_nxt; part_nxt = t;
    }
    if (!ok) return;      // the status word is set; the partial sums of this strip stay unwritten
    // one set of column partials per (strip, row set)
#pragma unroll
    for (int j = 0; j < NG; ++j) {
        if (gvalid[j]) {
            const int64_t off = (int64_t)(strip * RS + rset) * C + coff[j];
            reinterpret_cast<float4*>(colpart + off)[0] = make_float4(colb[j][0].x, colb[j][0].y, colb[j][1].x, colb[j][1].y);
            reinterpret_cast<float4*>(colpart + off)[1] = make_float4(colb[j][2].x, colb[j][2].y, colb[j][3].x, colb[j][3].y);
            reinterpret_cast<float4*>(tpart + off)[0] = make_float4(colT[j][0].x, colT[j][0].y, colT[j][1].x, colT[j][1].y);
            reinterpret_cast<float4*>(tpart + off)[1] = make_float4(colT[j][2].x, colT[j][2].y, colT[j][3].x, colT[j][3].y);
        }
    }
}

// Geometry of the fused first pass for a matrix of `cols` columns of `elem_bytes` each:
//   groups   row sets of the column sweep: 2 up to 2048 columns, else 1
//   ng       8-column groups per thread in the column sweep (1..4)
//   rb       rows per staged batch: the largest power of two that fits 64 KB, between 1 and 16 (the cost of a
//            batch is mostly fixed, so large batches pay)
//   stages   ring slots: as many as fit 192 KB, between 3 and 8 (a computing warp holds two at a time)
void fused_sq_geometry(int64_t cols, int elem_bytes, int* groups, int* ng, int* rb, int* stages) {
    const int64_t ncg = cols / 8;
    const int g = ncg <= FA_THREADS / 2 ? 2 : 1;
    const int n = g == 2 ? 1 : (int)((ncg + FA_THREADS - 1) / FA_THREADS);
    const int64_t row_bytes = cols * elem_bytes;
    int64_t r = 1;
    while (r < FA_RB && 2 * r * row_bytes <= 64 * 1024) r *= 2;
    int64_t st = (192 * 1024) / (r * row_bytes);
#ifdef CAME_TUNE      // build-time experiment switch: geometry overrides from the environment
    if (const char* e = getenv("CAME_FA_RB")) { r = atoi(e); while (r > 1 && r * row_bytes > 64 * 1024) r /= 2; st = (192 * 1024) / (r * row_bytes); }
    if (const char* e = getenv("CAME_FA_STAGES")) st = std::min<int64_t>(st, atoi(e));
#endif
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
    const size_t smem = max_ring_bytes + sizeof(FaShared) + (2 * FA_WARPS + K_TR) * sizeof(float);
    const int ng = key.mode & 15, groups = key.mode >> 4;
    switch (key.g_dtype) {
        case CAME_DT_F32: return launch_ng<float>(ng, groups, a, work, n, smem, st);
        case CAME_DT_F16: return launch_ng<__half>(ng, groups, a, work, n, smem, st);
        default: return launch_ng<__nv_bfloat16>(ng, groups, a, work, n, smem, st);
    }
}

}  // namespace came
