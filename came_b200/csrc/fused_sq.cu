// Fused first pass over the gradient: ONE read of g yields the row sums and column sums of g^2 (for the
// factored second moment) AND the column sums of g^2 / v_row (from which S = sum (g r c)^2, the quantity the
// RMS clip needs, follows without a second read of g):
//
//     S = sum_ij g_ij^2 r_i^2 c_j^2 = mean(v_row) * sum_j (1 / v_col_j) * T_j,   T_j = sum_i g_ij^2 / v_row_i
//
// which holds because r_i^2 = mean(v_row) / v_row_i and c_j^2 = 1 / v_col_j when no 1e-30 clamp is active
// (tensors carrying CAME_F_SQ_CLAMP take the two-pass kernels instead).  v_row_i needs the complete row,
// so the unit of work is a strip of 128 whole rows, staged through shared memory in batches of `rb` rows by
// bulk asynchronous copies into a 192 KB ring of slots and swept twice from shared memory.
//
// Replaces kUpdateSqRowQuantized, the column walk of kUpdateSqColQuantizedFinalize and kSumUpdateSq
// (came_kernels.cu:61-96, 198-243, 596-619), which read g three times.
#include "common.cuh"
#include "launch.h"
#include "pipeline.cuh"

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

constexpr int FA_MAX_SLOTS = 8;
constexpr int FA_RING_BYTES = 192 * 1024;         // ring = slots x slot bytes; a batch (rb rows) fits one slot
constexpr int FA_ALL_THREADS = FA_THREADS + 64;   // 16 computing warps, the copy-issuing warp, the row-finalize warp

// What the computing warps and the row-finalize warp need to know about a strip, written to shared memory by
// the copy-issuing warp before it starts the strip's copies (reading it from the tables in global memory would
// put a chain of dependent loads at the start of every strip).
struct FaStrip {
    float* vr;              // fresh v_row of the tensor
    float* colpart;         // this strip's first row of column partials (row set 0)
    float* tpart;
    int C, row0, nrows, rb, nbatch, pad;
    float eps0C, fC, beta2, om_beta2, gs2;      // gs2: grad_scale squared, applied to every sum of g^2
};

// Shared bookkeeping of one CTA.  Ring: full / empty per slot.  Strips alternate between two buffers (record +
// old row state): `ready` = the copy-issuing warp has filled the buffer, `done` = every computing warp and the
// row-finalize warp are through with it.  `wready` = the row weights 1 / v_row of a batch are in shared memory
// (two buffers, alternating by batch); `rowdone` = the row partials of a batch are complete.
struct FaShared {
    uint64_t full[FA_MAX_SLOTS];
    uint64_t empty[FA_MAX_SLOTS];
    uint64_t ready[2];
    uint64_t done[2];
    uint64_t wready[2];
    uint64_t rowdone[2];     // every computing warp has left its row partial of a batch (two buffers, alternating by batch)
    int abort;
    int pad;
};

__device__ __forceinline__ bool fa_wait(uint64_t* bar, uint32_t parity, FaShared* sh, const StepArgs& a, int lane) {
    volatile int* abort = &sh->abort;
    for (uint32_t i = 0; i < MBAR_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 15u && *abort) return false;
    }
    if (lane == 0) { atomicExch(a.status, STATUS_MBAR_TIMEOUT); atomicExch(&sh->abort, 1); }
    return false;
}

// Persistent CTA, one per SM; work item = a strip of 128 whole rows of one matrix.  Warps 0..15 compute, warp 16
// issues the bulk copies for strip after strip (a bulk-copy instruction blocks while the copy engine's queue is
// full, which would otherwise stall a computing warp), warp 17 completes the row sums.
//
// A batch of rb rows (a power of two, at most 16, at most 64 KB) is swept twice from shared memory with two
// different thread mappings:
//   row sweep     the 16 computing warps split the batch into 16 row pieces (16 / rb pieces per row); a warp sums
//                 the squares of its piece and leaves one partial in shared memory;
//   row finalize  warp 17, lane r: sums the partials of row r in a fixed order, forms the new v_row (mean of
//                 g^2 + eps0 over the row, came_kernels.cu:77-88, EMA with the old state), publishes it and leaves
//                 1 / v_row in shared memory -- a chain of dependent divisions that the computing warps never see;
//   column sweep  a thread owns the same 8 consecutive columns (NG such groups) for every row and accumulates
//                 g^2 and g^2 / v_row down the columns.  RS = 2 (matrices of at most 2048 columns): the
//                 threads form two sets that take the even and the odd rows of a batch, which keeps every
//                 thread busy; each set leaves its own column partials.
// Software pipeline: the row sweep of batch i+1 is issued before the column sweep of batch i; a computing warp
// therefore holds two ring slots.  The warps meet only through mbarriers (data landed, row partials complete, row
// weights ready, strip done), all with bounded, abort-aware waits: a warp whose wait runs out records it and leaves,
// the others follow at their next wait, and the copy-issuing warp stays until the copies in flight have landed.
template <typename TG, int NG, int RS>
__global__ void __launch_bounds__(FA_ALL_THREADS, 1) k_sqstat_fused(StepArgs a, const Work* __restrict__ work, int n_items,
                                                                    int n_slots, int slot_bytes) {
    extern __shared__ __align__(128) unsigned char smem[];
    FaShared* sh = reinterpret_cast<FaShared*>(smem + FA_RING_BYTES);
    float* s_part = reinterpret_cast<float*>(sh + 1);                // [2][FA_WARPS] row-piece sums, alternating by batch
    float* s_w = s_part + 2 * FA_WARPS;                              // [2][FA_RB]    1 / v_row of a batch's rows
    float* s_old = s_w + 2 * FA_RB;                                  // [2][K_TR]     dequantised old v_row of a strip's rows
    FaStrip* s_strip = reinterpret_cast<FaStrip*>(s_old + 2 * K_TR); // [2]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < n_slots; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], FA_WARPS); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh->ready[i], 1);
            mbar_init(&sh->done[i], FA_WARPS + 1);
            mbar_init(&sh->wready[i], 1);
            mbar_init(&sh->rowdone[i], FA_WARPS);
        }
        sh->abort = 0;
        mbar_init_fence();
    }
    __syncthreads();

    if (warp == FA_WARPS) {
        // copy-issuing warp: per strip, fill the strip buffer, then stream the strip's batches (lane r: row r)
        int slot = 0, issued = 0, n = 0;
        uint32_t phase = 1;      // parity of the slot's previous use (meaningless during the first lap)
        bool ok = true;
        for (int i = blockIdx.x; ok && i < n_items; i += gridDim.x, ++n) {
            const int sb = n & 1;
            if (n >= 2 && !fa_wait(&sh->done[sb], ((n >> 1) - 1) & 1, sh, a, lane)) { ok = false; break; }
            const Work w = work[i];
            const CameTensorDesc& d = a.descs[w.tensor];
            const Scratch& s = a.scr[w.tensor];
            const CameHyper& h = a.hyp[d.group];
            const int R = (int)d.rows, C = (int)d.cols, rb = s.fa_rb;
            const int row0 = w.tile * K_TR, nrows = min(K_TR, R - row0), nbatch = (nrows + rb - 1) / rb;
            for (int r = lane; r < nrows; r += 32) {
                const int row = row0 + r;
                s_old[sb * K_TR + r] = d.mode != CAME_MODE_FP32
                    ? (float)reinterpret_cast<const uint8_t*>(d.sq_row)[row] * (d.sq_row_absmax[row >> 8] / QMAX_U8)
                    : reinterpret_cast<const float*>(d.sq_row)[row];
            }
            if (lane == 0) {
                if (w.tile == 0) s.scal[3] = 0.0f;      // "a clamp binds": set by the finalize of this step, if at all
                FaStrip& t = s_strip[sb];
                t.vr = s.vr;
                t.colpart = s.colpart + (int64_t)w.tile * RS * C;
                t.tpart = s.tpart + (int64_t)w.tile * RS * C;
                t.C = C; t.row0 = row0; t.nrows = nrows; t.rb = rb; t.nbatch = nbatch;
                t.eps0C = (float)C * h.eps0; t.fC = (float)C; t.beta2 = h.beta2; t.om_beta2 = h.om_beta2;
                t.gs2 = h.grad_scale * h.grad_scale;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->ready[sb]);
            const uint32_t row_bytes = (uint32_t)C * (uint32_t)sizeof(TG);
            const unsigned char* g_src = reinterpret_cast<const unsigned char*>(d.g) + (int64_t)row0 * row_bytes;
            for (int b = 0; b < nbatch; ++b, ++issued, ++slot) {
                if (slot == n_slots) { slot = 0; phase ^= 1u; }
                if (issued >= n_slots && !fa_wait(&sh->empty[slot], phase, sh, a, lane)) { ok = false; break; }
                const int rows = min(rb, nrows - b * rb);
                if (lane == 0) mbar_arrive_expect_tx(&sh->full[slot], (uint32_t)rows * row_bytes);
                __syncwarp();
                if (lane < rows)
                    bulk_g2s(smem + slot * slot_bytes + lane * row_bytes, g_src + (int64_t)(b * rb + lane) * row_bytes,
                             row_bytes, &sh->full[slot]);
            }
        }
        if (!ok) {      // let the copies in flight land before the CTA's shared memory is released
            for (int i = 0; i < n_slots; ++i)
                for (uint32_t t = 0; t < (1u << 16); ++t)
                    if (mbar_try_wait(&sh->full[i], 0) || mbar_try_wait(&sh->full[i], 1)) break;
        }
        return;
    }

    if (warp == FA_WARPS + 1) {
        // row-finalize warp
        int gb = 0, n = 0;      // batches / strips gone through (buffer and phase selectors)
        for (int i = blockIdx.x; i < n_items; i += gridDim.x, ++n) {
            const int sb = n & 1;
            if (!fa_wait(&sh->ready[sb], (n >> 1) & 1, sh, a, lane)) return;
            const FaStrip& t = s_strip[sb];
            const int nbatch = t.nbatch, rb = t.rb, ppr = FA_WARPS / rb;
            for (int b = 0; b < nbatch; ++b, ++gb) {
                if (!fa_wait(&sh->rowdone[gb & 1], (gb >> 1) & 1, sh, a, lane)) return;      // the row partials of batch b
                const int rows = min(rb, t.nrows - b * rb);
                if (lane < rows) {
                    const float* part = s_part + (gb & 1) * FA_WARPS + lane * ppr;
                    float sum = 0.0f;
                    for (int q = 0; q < ppr; ++q) sum += part[q];
                    const float mean = (sum * t.gs2 + t.eps0C) / t.fC;
                    const float v = s_old[sb * K_TR + b * rb + lane] * t.beta2 + t.om_beta2 * mean;
                    t.vr[t.row0 + b * rb + lane] = v;
                    s_w[(gb & 1) * FA_RB + lane] = v > 0.0f ? 1.0f / v : 0.0f;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->wready[gb & 1]);
            }
            if (lane == 0) mbar_arrive(&sh->done[sb]);      // through with the strip's record and old row state
        }
        return;
    }

    // ---- computing warps ----
    constexpr int ST = FA_THREADS / RS;          // threads of a row set of the column sweep
    const int rset = threadIdx.x / ST, tis = threadIdx.x - rset * ST;
    int slot = 0, gb = 0, n = 0;      // ring position (advanced without a division), batches and strips gone through
    uint32_t phase = 0;

    for (int i = blockIdx.x; i < n_items; i += gridDim.x, ++n) {
        const int sb = n & 1;
        if (!fa_wait(&sh->ready[sb], (n >> 1) & 1, sh, a, lane)) return;      // the status word is set
        const FaStrip& t = s_strip[sb];
        const int C = t.C, rb = t.rb, nrows = t.nrows, nbatch = t.nbatch;
        const int row_bytes = C * (int)sizeof(TG);
        // row sweep: this warp's row of a batch and its span of 8-column groups within the row
        const int ncg = C >> 3;                      // 8-column groups per row
        const int ppr = FA_WARPS / rb;               // pieces per row (rb is a power of two <= 16)
        const int my_row = warp / ppr, my_piece = warp - my_row * ppr;
        const int cg_lo = (int)((int64_t)my_piece * ncg / ppr), cg_hi = (int)((int64_t)(my_piece + 1) * ncg / ppr);
        const int piece_chunks = (cg_hi - cg_lo) >> 5, piece_rem = (cg_hi - cg_lo) & 31;
        // column sweep: 8-column groups of this thread.  A thread whose group lies beyond the last column sweeps
        // group 0 instead and drops the result: the sweep itself then needs no per-group test (wide rows keep the
        // test: without it the offsets cost registers they lack)
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

        auto row_sweep = [&](int b, int sl, float* part, uint64_t* rowdone) {
            const int rows = min(rb, nrows - b * rb);
            float acc_t = 0.0f;
            if (my_row < rows) {
                const TG* src = reinterpret_cast<const TG*>(smem + sl * slot_bytes + my_row * row_bytes);
                u64 acc[4] = {F2ZERO, F2ZERO, F2ZERO, F2ZERO};
                // whole 32-group chunks without a per-lane test, then the ragged end of the piece
                const TG* p = src + (cg_lo + lane) * 8;
#pragma unroll 4
                for (int c = 0; c < piece_chunks; ++c, p += 256) {
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
                acc_t = q.x + q.y;
            }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) acc_t += __shfl_xor_sync(0xffffffffu, acc_t, m);
            if (lane == 0) { part[warp] = acc_t; mbar_arrive(rowdone); }      // same thread: the partial comes first
        };
        auto col_sweep = [&](int b, int sl, const float* wv) {
            const int rows = min(rb, nrows - b * rb);
            const TG* src = reinterpret_cast<const TG*>(smem + sl * slot_bytes + rset * row_bytes);
#pragma unroll 2
            for (int r = rset; r < rows; r += RS, src += RS * C) {
                const u64 w2 = splat(wv[r]);
#pragma unroll
                for (int j = 0; j < NG; ++j) {
                    if (NG <= 2 || gvalid[j]) {
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
            if (lane == 0) mbar_arrive(&sh->empty[sl]);
        };

        // No CTA-wide barrier in the batch loop: a warp waits for its data (`full`), for the row weights of the batch it
        // is about to sweep by columns (`wready`), and for nothing else, so the warps drift apart by up to a batch and
        // their row sweeps (shared-memory loads, shuffles) overlap other warps' column sweeps (arithmetic).  Buffer
        // reuse is safe without one: the partial / weight buffers of batch b are written again for batch b + 2, and a
        // warp gets there only after its column sweep of batch b, i.e. after `wready` of batch b, which the
        // row-finalize warp raises after reading the partials; it writes the weights of batch b + 2 only after every
        // warp's row sweep of b + 2 (`rowdone`), which each warp issues after its column sweep of batch b.
        if (!fa_wait(&sh->full[slot], phase, sh, a, lane)) return;
        row_sweep(0, slot, s_part + (gb & 1) * FA_WARPS, &sh->rowdone[gb & 1]);
        for (int b = 0; b < nbatch; ++b, ++gb) {
            int nslot = slot + 1;
            uint32_t nphase = phase;
            if (nslot == n_slots) { nslot = 0; nphase ^= 1u; }
            if (b + 1 < nbatch) {
                if (!fa_wait(&sh->full[nslot], nphase, sh, a, lane)) return;
                row_sweep(b + 1, nslot, s_part + ((gb + 1) & 1) * FA_WARPS, &sh->rowdone[(gb + 1) & 1]);
            }
            if (!fa_wait(&sh->wready[gb & 1], (gb >> 1) & 1, sh, a, lane)) return;
            col_sweep(b, slot, s_w + (gb & 1) * FA_RB);
            slot = nslot; phase = nphase;
        }
        // one set of column partials per (strip, row set)
#pragma unroll
        for (int j = 0; j < NG; ++j) {
            if (gvalid[j]) {
                float* cp = t.colpart + (int64_t)rset * C + coff[j];
                float* tp = t.tpart + (int64_t)rset * C + coff[j];
                reinterpret_cast<float4*>(cp)[0] = make_float4(colb[j][0].x, colb[j][0].y, colb[j][1].x, colb[j][1].y);
                reinterpret_cast<float4*>(cp)[1] = make_float4(colb[j][2].x, colb[j][2].y, colb[j][3].x, colb[j][3].y);
                reinterpret_cast<float4*>(tp)[0] = make_float4(colT[j][0].x, colT[j][0].y, colT[j][1].x, colT[j][1].y);
                reinterpret_cast<float4*>(tp)[1] = make_float4(colT[j][2].x, colT[j][2].y, colT[j][3].x, colT[j][3].y);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->done[sb]);
    }
}

// Geometry of the fused first pass for a matrix of `cols` columns of `elem_bytes` each:
//   groups   row sets of the column sweep: 2 up to 2048 columns, else 1
//   ng       8-column groups per thread in the column sweep (1..4)
//   slot_kb  ring slot size in KB (the 192 KB ring holds 192 / slot_kb slots; all tensors of a launch share it)
//   rb       rows per staged batch: the largest power of two that fits a slot, between 1 and 16 (the cost of a
//            batch is mostly fixed, so large batches pay)
void fused_sq_geometry(int64_t cols, int elem_bytes, int* groups, int* ng, int* rb, int* slot_kb) {
    const int64_t ncg = cols / 8;
    const int g = ncg <= FA_THREADS / 2 ? 2 : 1;
    const int n = g == 2 ? 1 : (int)((ncg + FA_THREADS - 1) / FA_THREADS);
    const int64_t row_bytes = cols * elem_bytes;
    int kb = 64;
#ifdef CAME_TUNE      // build-time experiment switch: geometry overrides from the environment
    if (const char* e = getenv(n >= 3 ? "CAME_FA_SLOT_KB_WIDE" : "CAME_FA_SLOT_KB")) kb = atoi(e);
    if (row_bytes > (int64_t)kb * 1024) kb = 64;
#endif
    int64_t r = 1;
    while (r < FA_RB && 2 * r * row_bytes <= (int64_t)kb * 1024) r *= 2;
    *groups = g; *ng = n < 1 ? 1 : n; *rb = (int)r; *slot_kb = kb;
}

bool fused_sq_eligible(int64_t cols, int elem_bytes) {
    return cols % 8 == 0 && cols <= (int64_t)FA_THREADS * 8 * 4 && cols * elem_bytes <= 64 * 1024;
}

template <typename TG, int NG, int RS>
static cudaError_t launch_one(const StepArgs& a, const Work* work, int n, int slot_kb, cudaStream_t st) {
    const int sms = persistent_grid_limit();
    const size_t smem = (size_t)FA_RING_BYTES + sizeof(FaShared) +
                        (2 * FA_WARPS + 2 * FA_RB + 2 * K_TR) * sizeof(float) + 2 * sizeof(FaStrip);
    cudaError_t e = cudaFuncSetAttribute(k_sqstat_fused<TG, NG, RS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const int slot_bytes = slot_kb * 1024;
    int n_slots = FA_RING_BYTES / slot_bytes;
    if (n_slots > FA_MAX_SLOTS) n_slots = FA_MAX_SLOTS;
    k_sqstat_fused<TG, NG, RS><<<n < sms ? n : sms, FA_ALL_THREADS, smem, st>>>(a, work, n, n_slots, slot_bytes);
    return cudaGetLastError();
}

template <typename TG>
static cudaError_t launch_ng(int ng, int groups, int slot_kb, const StepArgs& a, const Work* work, int n, cudaStream_t st) {
    if (groups == 2) return launch_one<TG, 1, 2>(a, work, n, slot_kb, st);      // at most 2048 columns: one column group per thread
    switch (ng) {
        case 1: return launch_one<TG, 1, 1>(a, work, n, slot_kb, st);
        case 2: return launch_one<TG, 2, 1>(a, work, n, slot_kb, st);
        case 3: return launch_one<TG, 3, 1>(a, work, n, slot_kb, st);
        default: return launch_one<TG, 4, 1>(a, work, n, slot_kb, st);
    }
}

// key.mode carries ng | (groups << 4) | (slot KB << 8); all tensors of one launch share it
cudaError_t launch_fused_sq(const KernelKey& key, const StepArgs& a, const Work* work, int n, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    const int ng = key.mode & 15, groups = (key.mode >> 4) & 15, slot_kb = key.mode >> 8;
    switch (key.g_dtype) {
        case CAME_DT_F32: return launch_ng<float>(ng, groups, slot_kb, a, work, n, st);
        case CAME_DT_F16: return launch_ng<__half>(ng, groups, slot_kb, a, work, n, st);
        default: return launch_ng<__nv_bfloat16>(ng, groups, slot_kb, a, work, n, st);
    }
}

}  // namespace came
