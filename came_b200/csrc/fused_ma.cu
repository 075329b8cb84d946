// Momentum pass, residual finalize and apply pass of the tile layout (and of the flat layout whose column count is a
// multiple of 256) as ONE persistent kernel.
//
// Run as three launches over all tensors, each pass ends in a tail (a work item keeps an SM for 12 us) and the
// issue-bound momentum pass and the DRAM-bound apply pass never share the GPU.  Here the work items of every tensor
// form two lists that one launch consumes:
//
//   M  momentum tile (128 x 1024): g, m -> m, residual row / column partials      (k_moment_tile8_wide's item)
//   A  apply tile: m, p -> p                                                        (k_apply_tile8_wide's item)
//   F  one block of 256 entries of the residual row or column vector: partials -> state, fresh fp32 values,
//      C'_j; the tensor's last block adds the mean of the row vector        (k_vec_finalize<true>'s item)
//
//   list 1:  M(t0) M(t1)[`lag` items] A(t0) M(t1)[rest] M(t2)[...] A(t1) ...      computing warps, through the ring
//            (once a tensor's apply items are due they are dealt out one per momentum item, so that the DRAM-bound
//            and the issue-bound items share the GPU at all times)
//   list 2:  F(t0) F(t1) ...                                                        one finalizer warp per CTA
//
// Push mode (StepArgs::n_push > 0, several GPUs): an A item stores every new parameter into the local buffer and, at
// the same offset, into the mapped buffers of the peers: the weight exchange of a data-parallel job becomes part of the
// step.  Plain stores; no kernel here reads a peer's memory.
//
// A CTA takes the next item of a list whenever it has room for it (two cursors in global memory), so the load
// balances itself.  An F item needs every M item of its tensor, an A item every F item: per-tensor counters in global
// memory, incremented after a fence by the warp that finished an item and polled (acquire) by the warp about to run or
// publish a dependent one.  `lag` momentum items of later tensors separate a tensor's last M item from its first A
// item, which covers the M items still in flight and the finalize (about 40 us on Llama-7B shapes); the helper warp
// holds an A item whose tensor is not ready while the CTA's other warps work on the items already published.
// Dependencies only point backwards in the lists and a grid never exceeds one CTA per SM (cooperative launch: all CTAs
// are resident), so the waits cannot deadlock; they are bounded all the same (status word, abort flag).
//
// Measured on Llama-7B shapes: 9.9 ms against 10.7 ms for the three launches, 94 % of the copy bandwidth for the bytes
// actually moved.  L2: every stream that is read once carries an evict-first policy; the codes of the last quarter of a
// tensor's momentum tiles are written evict-last and the apply items run through the tiles in reverse order, which
// lets them find about 70 % of that quarter in L2 (1.2 GB of 6.7 GB of codes per step).  Protecting every tile does not
// work: with the apply items as far behind as the dependency needs (40 us times the bandwidth), more protected lines
// are alive than the L2 keeps, and they crowd out each other; measured, it is slower than protecting none.
//
// The arithmetic of every item is that of the three separate kernels, operation for operation: the results are
// bit-identical to theirs.
#include "wide.cuh"

#include <cstdlib>

namespace came {

constexpr int MA_PRODUCERS = 2;
constexpr int MA_HELPER = W_WARPS + MA_PRODUCERS;                 // warp index of the helper
constexpr int MA_FINALIZER = MA_HELPER + 1;                       // warp that runs the F items
constexpr int MA_ALL_THREADS = W_THREADS + 32 * (MA_PRODUCERS + 2);
constexpr uint32_t MA_POLL_LIMIT = 1u << 26;                      // helper polls (a few seconds) before it gives up

struct MaItem {
    int kind, tensor;
    int R, C, row0, col0, wcols, nbands, tr, tc;
    // copy stream: operand A (g for M, p for A), codes, and (A only) the band's tile absmax
    const unsigned char* a_src;
    const unsigned char* m_src;
    const unsigned char* x_src;
    const unsigned char* b_src;      // flat-layout A item: the parameter rows (a_src holds the gradient rows)
    int64_t a_pitch, m_pitch, x_pitch;
    // M
    int8_t* m;
    float* m_absmax;
    float* colpart;
    float om_beta1, dq_beta1, beta1;
    int keep;             // the codes this item writes are marked evict-last in L2
    // A
    void* p;
    float lr, wd_lr, decay_mul;
    int wd_mode;
};

struct MaShared {
    uint64_t full[4];
    uint64_t empty[4];
    uint64_t ready[2];
    uint64_t done[2];
    int abort;
    int pad[3];             // 112 bytes: what follows in shared memory stays 16-byte aligned (bulk-copy destinations)
};
static_assert(sizeof(MaShared) % 16 == 0, "factor slices are bulk-copy destinations");

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// bounded, abort-aware wait on one of the CTA's barriers (same contract as wide_wait)
__device__ __forceinline__ bool ma_wait(uint64_t* bar, uint32_t parity, MaShared* sh, const StepArgs& a, int lane) {
    volatile int* abort = &sh->abort;
    for (uint32_t i = 0; i < MBAR_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return *abort == 0;
        if ((i & 15u) == 15u && *abort) return false;
    }
    if (lane == 0) { atomicExch(a.status, STATUS_MBAR_TIMEOUT); atomicExch(&sh->abort, 1); }
    return false;
}

// One block of 256 entries of the residual row or column vector of a tensor, by ONE warp (the helper warp of the CTA
// that took the item): partial sums -> new state value (EMA with the dequantised old state), fresh fp32 copy,
// requantisation, the block's share of the row mean / the column factors C'_j of the apply items.  Arithmetic and
// summation order are those of k_vec_finalize<true> (reference: came_kernels.cu:2685-2779, 298-333): lane l holds the
// entries w * 32 + l (w = 0..7), i.e. what thread l of warp w holds there.
__device__ __forceinline__ void ma_finalize_block(const StepArgs& a, int tensor, int fblock, int lane) {
    const CameTensorDesc& d = a.descs[tensor];
    const Scratch& s = a.scr[tensor];
    const CameHyper& h = a.hyp[d.group];
    const int R = (int)d.rows, C = (int)d.cols;
    const bool is_col = fblock >= s.nbR;
    const int b = is_col ? fblock - s.nbR : fblock;
    const int nvec = is_col ? C : R;
    const int base = b * QBLOCK + lane;
    uint8_t* state = reinterpret_cast<uint8_t*>(is_col ? d.res_col : d.res_row);
    float* absmax = is_col ? d.res_col_absmax : d.res_row_absmax;
    float* fresh = is_col ? s.Rc : s.Rr;
    // Partial sums of the block's entries, entry by entry with 32 loads in flight (one warp has to cover the latency of
    // parts x 256 loads).  Columns: partials [ptiles_r][C], eight chains over the rows t = w, w + 8, ..., added in the
    // order w = 0..7.  Rows: partials [ptiles_c][R], one chain in the order t = 0, 1, ...  (Adding the 0.0f of a
    // masked load leaves a sum unchanged, so the chunking does not alter the result.)
    const float* part = is_col ? s.colpart : s.rowpart;
    const int parts = is_col ? s.ptiles_r : s.ptiles_c;
    float tot[8];
#pragma unroll 1
    for (int e = 0; e < 8; ++e) {
        const int idx = base + 32 * e;
        const bool valid = idx < nvec;
        const float* col = part + (valid ? idx : 0);
        float chain[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) chain[k] = 0.0f;
        for (int t0 = 0; t0 < parts; t0 += 32) {
            float x[32];
#pragma unroll
            for (int k = 0; k < 32; ++k) x[k] = (valid && t0 + k < parts) ? __ldcg(col + (int64_t)(t0 + k) * nvec) : 0.0f;   // written by other SMs: past L1
            if (is_col) {
#pragma unroll
                for (int k = 0; k < 32; ++k) chain[k & 7] += x[k];
            } else {
#pragma unroll
                for (int k = 0; k < 32; ++k) chain[0] += x[k];
            }
        }
        float r = chain[0];
        if (is_col) {
            r = 0.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) r += chain[k];
        }
        tot[e] = r;
    }
    const float old_scale = absmax[b] / QMAX_U8;
    const float fn = (float)(is_col ? R : C);      // entries a sum ran over
    float v[8], vmax = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const int idx = base + 32 * e;
        v[e] = 0.0f;
        if (idx < nvec) {
            const float acc = mean_plus_eps(tot[e], fn, h.eps1);
            const float old = (float)state[idx] * old_scale;
            v[e] = ema_update(old, h.beta3, h.om_beta3, acc);
            fresh[idx] = v[e];
        }
        vmax = fmaxf(vmax, v[e]);
    }
    const float bmax = fix_absmax(warp_max(vmax));
    __syncwarp();      // every lane has read the old absmax
    if (lane == 0) absmax[b] = bmax;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const int idx = base + 32 * e;
        if (idx < nvec) state[idx] = (uint8_t)quant_u8_div(v[e], bmax);
    }
    if (!is_col) {
        float t = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) t += warp_sum(v[e]);      // the sum of "warp" e, then the eight in order
        if (lane == 0) s.rowblk2[b] = t;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int idx = base + 32 * e;
            // C'_j for the tensor's A items (the flat layout still needs c_j there: a vector of its own)
            if (idx < nvec) (s.mfac_c2 ? s.mfac_c2 : s.mfac_c)[idx] = col_factor(v[e], d.flags & CAME_F_RESCOL_CLAMP);
        }
    }
}

#ifdef CAME_MA_PROFILE      // build-time experiment: per-CTA cycle counters (slot meanings at the use sites)
__device__ unsigned long long g_ma_prof[160][16];
#define MA_PROF_ADD(slot, cycles) atomicAdd(&g_ma_prof[blockIdx.x][slot], (unsigned long long)(cycles))
#define MA_CLOCK() clock64()
extern "C" int came_b200_debug_ma_profile(unsigned long long* out, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out, g_ma_prof, sizeof(g_ma_prof));
    if (e == cudaSuccess && reset) {
        static unsigned long long zero[160][16];
        e = cudaMemcpyToSymbol(g_ma_prof, zero, sizeof(zero));
    }
    return e == cudaSuccess ? 0 : -3;
}
#else
#define MA_PROF_ADD(slot, cycles)
#define MA_CLOCK() 0ll
#endif

// After a failed wait: give the bulk copies that may still be in flight a bounded chance to land before the warp
// leaves (the CTA's shared memory must not be released under them).  Every warp that gives up calls this.
__device__ __forceinline__ void ma_drain(MaShared* sh, int stages) {
    for (int i = 0; i < stages; ++i)
        for (uint32_t t = 0; t < (1u << 16); ++t)
            if (mbar_try_wait(&sh->full[i], 0) || mbar_try_wait(&sh->full[i], 1)) break;
}

// FLAT = false: tile layout (the momentum is re-quantised per 16 x 16 tile by the M items; the A items read the new
// codes).  FLAT = true: flat layout, column count a multiple of 256 (absmax per 256-column row segment): the M items
// only produce the residual sums; the A items recompute the momentum from g and the old codes so that its un-quantised
// value feeds the update, re-quantise it and update p (k_apply_flat8_wide's item: bands of 8 rows of g, p and codes).
template <typename T, bool FLAT>
__global__ void __launch_bounds__(MA_ALL_THREADS, 1) k_moment_apply_tile8(StepArgs a, const Work* __restrict__ work, int n_items,
                                                                          int* __restrict__ mcount, int* __restrict__ fcount,
                                                                          int* __restrict__ next_item, const Work* __restrict__ fwork,
                                                                          int n_fitems, int* __restrict__ next_fitem, int keep_pct) {
    constexpr int STAGES = WideCfg<T>::STAGES, STAGE = WideCfg<T>::STAGE, ROW = WideCfg<T>::ROW;
    constexpr int FLB = 8;                                  // rows of a band of a flat-layout A item
    static_assert(FLB * (2 * ROW + W_MROW) <= STAGE, "a flat A band fits a ring slot");
    extern __shared__ __align__(128) unsigned char smem[];
    MaShared* sh = reinterpret_cast<MaShared*>(smem + STAGES * STAGE);
    float* s_r = reinterpret_cast<float*>(sh + 1);      // [2][W_TR]   row factors of an item (M: r_i / clip, A: R'_i)
    float* s_c = s_r + 2 * W_TR;                        // [2][W_TC]   column factors (M: c_j, A: C'_j)
    float* s_row = s_c + 2 * W_TC;                      // [2][W_WARPS][W_TR]  M: per-warp row partials; F: reduction scratch
    MaItem* s_item = reinterpret_cast<MaItem*>(s_row + 2 * W_WARPS * W_TR);    // [2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], W_WARPS); }
        // `done`: every computing warp and every producer warp is through with the record
        for (int i = 0; i < 2; ++i) { mbar_init(&sh->ready[i], 1); mbar_init(&sh->done[i], W_WARPS + MA_PRODUCERS); }
        sh->abort = 0;
        mbar_init_fence();
    }
    __syncthreads();

    // ------------------------------------------------------------------------------------------------
    // producer warps: the copy stream of the CTA's M and A items, alternate bands each
    // ------------------------------------------------------------------------------------------------
    if (warp >= W_WARPS && warp < MA_HELPER) {
        const int which = warp - W_WARPS;
        const uint64_t stream_policy = l2_policy_evict_first();
        int q = 0;
        bool ok = true;
        for (int n = 0; ok; ++n) {
            const int buf = n & 1;
            if (!ma_wait(&sh->ready[buf], (n >> 1) & 1, sh, a, lane)) { ok = false; break; }
            if (s_item[buf].kind == MA_KIND_END) break;
            const MaItem& it = s_item[buf];
            // the codes (and p) were written by ordinary stores of other CTAs: order them before this CTA's bulk copies
            fence_async_global();
            const unsigned char* a_src = it.a_src;
            const unsigned char* m_src = it.m_src;
            const unsigned char* x_src = it.x_src;
            const int64_t a_pitch = it.a_pitch, m_pitch = it.m_pitch, x_pitch = it.x_pitch;
            const int nbands = it.nbands, nrows = it.R - it.row0;
            const uint32_t a_bytes = (uint32_t)it.wcols * sizeof(T), m_bytes = (uint32_t)it.wcols;
            const uint32_t x_bytes = x_src ? (uint32_t)(it.wcols >> 4) * sizeof(float) : 0u;
            if (FLAT && it.kind == MA_KIND_A) {
                // bands of 8 rows, three operands: lanes 0-7 the gradient rows, 8-15 the code rows, 16-23 the parameter rows
                const unsigned char* b_src = it.b_src;
                for (int band = 0; band < nbands; ++band, ++q) {
                    if (q % MA_PRODUCERS != which) continue;
                    const int slot = q % STAGES;
                    if (q >= STAGES && !ma_wait(&sh->empty[slot], ((q / STAGES) - 1) & 1, sh, a, lane)) { ok = false; break; }
                    const int rows = min(FLB, nrows - band * FLB);
                    if (lane == 0) mbar_arrive_expect_tx(&sh->full[slot], (uint32_t)rows * (2 * a_bytes + m_bytes));
                    __syncwarp();
                    const int r = lane & 7, op = lane >> 3;
                    if (r < rows && op < 3) {
                        const int64_t row = band * FLB + r;
                        unsigned char* st = smem + slot * STAGE;
                        if (op == 0) bulk_g2s_hint(st + r * ROW, a_src + row * a_pitch, a_bytes, &sh->full[slot], stream_policy);
                        else if (op == 1) bulk_g2s_hint(st + 2 * FLB * ROW + r * W_MROW, m_src + row * m_pitch, m_bytes, &sh->full[slot], stream_policy);
                        else bulk_g2s_hint(st + FLB * ROW + r * ROW, b_src + row * a_pitch, a_bytes, &sh->full[slot], stream_policy);
                    }
                }
                __syncwarp();
                if (ok && lane == 0) mbar_arrive(&sh->done[buf]);
                continue;
            }
            for (int band = 0; band < nbands; ++band, ++q) {
                if (q % MA_PRODUCERS != which) continue;
                const int slot = q % STAGES;
                if (q >= STAGES && !ma_wait(&sh->empty[slot], ((q / STAGES) - 1) & 1, sh, a, lane)) { ok = false; break; }
                const int rows = min(W_BAND, nrows - band * W_BAND);
                if (lane == 0) {
                    mbar_arrive_expect_tx(&sh->full[slot], (uint32_t)rows * (a_bytes + m_bytes) + x_bytes);
                    if (x_bytes) bulk_g2s_hint(smem + slot * STAGE + WideCfg<T>::AMAX_OFF, x_src + band * x_pitch, x_bytes, &sh->full[slot], stream_policy);
                }
                __syncwarp();
                const int r = lane & 15;
                if (r < rows) {
                    const int64_t row = band * W_BAND + r;
                    if (lane < 16) bulk_g2s_hint(smem + slot * STAGE + r * ROW, a_src + row * a_pitch, a_bytes, &sh->full[slot], stream_policy);
                    else bulk_g2s_hint(smem + slot * STAGE + W_BAND * ROW + r * W_MROW, m_src + row * m_pitch, m_bytes, &sh->full[slot], stream_policy);
                }
            }
            // the record has been read for the last time (the helper reuses its buffer once everybody has said so)
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(&sh->done[buf]);
        }
        // after a failed wait somewhere in the CTA: let the copies in flight land before shared memory is released
        if (*reinterpret_cast<volatile int*>(&sh->abort)) ma_drain(sh, STAGES);
        return;
    }

    // ------------------------------------------------------------------------------------------------
    // finalizer warp: takes the F items of the launch in list order (a cursor of its own), waits until the tensor's
    // M items are all in, runs the block and counts it.  148 such warps share the 59 blocks of a 4096 x 11008 tensor.
    // ------------------------------------------------------------------------------------------------
    if (warp == MA_FINALIZER) {
        while (true) {
            int idx = 0;
            if (lane == 0) idx = atomicAdd(next_fitem, 1);
            idx = __shfl_sync(0xffffffffu, idx, 0);
            if (idx >= n_fitems) return;
            const Work wf = fwork[idx];
            const Scratch& s = a.scr[wf.tensor];
            const int need = s.ptiles_r * s.ptiles_c;
            uint32_t polls = 0;
            while (true) {
                int got = 0;
                if (lane == 0) got = ld_acquire(mcount + wf.tensor);
                got = __shfl_sync(0xffffffffu, got, 0);
                if (got >= need) break;
                if (*reinterpret_cast<volatile int*>(&sh->abort)) return;
                if (++polls > MA_POLL_LIMIT) {
                    if (lane == 0) { atomicExch(a.status, STATUS_MBAR_TIMEOUT); atomicExch(&sh->abort, 1); }
                    return;
                }
                __nanosleep(256);
            }
            const long long t0 = MA_CLOCK();
            ma_finalize_block(a, wf.tensor, wf.tile, lane);
            if (lane == 0) { MA_PROF_ADD(11, MA_CLOCK() - t0); MA_PROF_ADD(12, 1); }      // 11: F cycles, 12: F items
            __threadfence();
            __syncwarp();
            int before = 0;
            if (lane == 0) before = atomicAdd(fcount + wf.tensor, 1);
            before = __shfl_sync(0xffffffffu, before, 0);
            if (before + 1 == s.nbR + s.nbC) {
                // The tensor's last block: every row block's share of the mean is in.  mean(Rr), guarded as the apply
                // pass guards it, goes to the tensor's scalar scratch; then one more count: the A items wait for
                // blocks + 1.
                __threadfence();      // acquire side of the counter: the other finalizers' writes are visible
                const CameTensorDesc& d = a.descs[wf.tensor];
                float part = 0.0f;      // warp_vector_sum's order, with loads that bypass L1 (other SMs wrote the values)
                for (int i = lane; i < s.nbR; i += 32) part += __ldcg(s.rowblk2 + i);
                float mean = warp_sum(part) / (float)d.rows;
                mean = guard_mean(mean, d.flags & CAME_F_RESROW_FIX, d.flags & CAME_F_RESROW_CLAMP);
                if (lane == 0) s.scal[2] = mean;
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicAdd(fcount + wf.tensor, 1);
            }
        }
    }

    // ------------------------------------------------------------------------------------------------
    // helper warp: publishes the CTA's items one by one (two record buffers), after their dependencies are met;
    // finishes the items the computing warps are through with (row partials of an M item, the tensor's counters)
    // ------------------------------------------------------------------------------------------------
    if (warp == MA_HELPER) {
        // What an item needs to know about its tensor, cached per kind (consecutive M items mostly share a tensor, and
        // so do consecutive A items): filling an entry is a chain of dependent global loads, done once per tensor.
        struct TensorInfo {
            int tensor, R, C, ptiles_c, ntiles;
            const unsigned char* a_base;      // g (M, flat A) or p (tile A)
            const unsigned char* b_base;      // p (flat A)
            const float* fac_c2;              // flat A: C'_j (fac_c keeps c_j)
            const float* fac_r0;              // flat A: mfac rows (r_i / clip)
            const unsigned char* m_base;
            const unsigned char* x_base;      // tile absmax
            float* colpart;
            const float* fac_r;               // M: mfac (r_i / clip); A: the fresh residual row vector Rr
            const float* fac_c;               // mfac_c
            float om_beta1, dq_beta1, beta1, lr, wd_lr, decay_mul;
            int wd_mode;
            float mean;                       // A: guarded mean(Rr)
            bool clamp_row;
        };
        TensorInfo ti[2];      // [0]: M items, [1]: A items (registers; every lane holds a copy)
        ti[0].tensor = ti[1].tensor = -1;
        auto prepare = [&](const Work& w, int buf) {
            const int kind = (int)((uint32_t)w.tile >> 28), tile = w.tile & 0x0fffffff;
            TensorInfo& t = ti[kind == MA_KIND_M ? 0 : 1];
            if (t.tensor != w.tensor) {
                const CameTensorDesc& d = a.descs[w.tensor];
                const Scratch& s = a.scr[w.tensor];
                const CameHyper& h = a.hyp[d.group];
                t.tensor = w.tensor;
                t.R = (int)d.rows; t.C = (int)d.cols; t.ptiles_c = s.ptiles_c; t.ntiles = s.ptiles_r * s.ptiles_c;
                t.a_base = reinterpret_cast<const unsigned char*>((kind == MA_KIND_M || FLAT) ? d.g : d.p);
                t.b_base = reinterpret_cast<const unsigned char*>(d.p);
                t.fac_c2 = s.mfac_c2; t.fac_r0 = s.mfac;
                t.m_base = reinterpret_cast<const unsigned char*>(d.m);
                t.x_base = reinterpret_cast<const unsigned char*>(d.m_absmax);
                t.colpart = s.colpart; t.fac_r = kind == MA_KIND_M ? s.mfac : s.Rr; t.fac_c = s.mfac_c;
                t.mean = kind == MA_KIND_A ? s.scal[2] : 1.0f;
                t.clamp_row = d.flags & CAME_F_RESROW_CLAMP;
                t.om_beta1 = h.om_beta1; t.dq_beta1 = h.beta1 / QMAX_I8; t.beta1 = h.beta1;
                t.lr = h.lr; t.wd_lr = h.wd_lr; t.decay_mul = h.decay_mul;
                t.wd_mode = h.weight_decay == 0.0f ? 0 : ((d.flags & CAME_F_WD_MUL2) ? 2 : ((d.flags & CAME_F_WD_ADD2) ? 3 : 1));
            }
            const int R = t.R, C = t.C;
            float* sr = s_r + buf * W_TR;
            float* sc = s_c + buf * W_TC;
            const int tr = tile / t.ptiles_c, tc = tile - tr * t.ptiles_c;
            const int row0 = tr * W_TR, col0 = tc * W_TC;
            const int wcols = min(W_TC, C - col0);
            const bool flat_a = FLAT && kind == MA_KIND_A;
            const int nbands = flat_a ? min(W_TR / FLB, (R - row0 + FLB - 1) / FLB) : min(W_BANDS, (R - row0 + W_BAND - 1) / W_BAND);
            // The factor slices of the item come by bulk copies that complete on the record's `ready` barrier (the
            // waiters see them with the record): the column factors (c_j for M, C'_j for A) of the tile's columns and
            // the row factors (r_i / clip, R'_i) of its rows.  Rows past the end of the matrix receive whatever follows
            // in the scratch (the copy is rounded up to 16 bytes); the computing warps never use them.
            const uint32_t c_bytes = (uint32_t)wcols * sizeof(float);
            const uint32_t r_bytes = (kind == MA_KIND_M || flat_a) ? (uint32_t)((min(W_TR, R - row0) + 3) & ~3) * sizeof(float) : 0u;
            // a flat A item needs both pairs of factors: r_i / clip and c_j (bulk copies, as for an M item) in the record's
            // first slices, R'_i (computed here) and C'_j (bulk copy) in the record's row-partial area, which an A item
            // does not use otherwise
            float* sr2 = s_row + buf * (W_WARPS * W_TR);
            float* sc2 = sr2 + W_TR;
            if (flat_a) sr = sr2;      // where the R'_i computed below go
            if (kind == MA_KIND_A) {
                // R'_i = rsqrt(Rr_i / mean(Rr)) for the tile's rows (came_kernels.cu:313-332)
                float rr[W_TR / 32];
#pragma unroll
                for (int k = 0; k < W_TR / 32; ++k) rr[k] = (row0 + lane + 32 * k < R) ? t.fac_r[row0 + lane + 32 * k] : 1.0f;
#pragma unroll
                for (int k = 0; k < W_TR / 32; ++k)
                    sr[lane + 32 * k] = (row0 + lane + 32 * k < R) ? row_factor(rr[k], t.mean, t.clamp_row) : 0.0f;
            }
            __syncwarp();      // the row factors written above come before lane 0's arrival
            if (lane == 0) {
                MaItem& mi = s_item[buf];
                mi.kind = kind; mi.tensor = w.tensor;
                mi.R = R; mi.C = C; mi.row0 = row0; mi.col0 = col0; mi.wcols = wcols; mi.nbands = nbands; mi.tr = tr; mi.tc = tc;
                mi.a_pitch = (int64_t)C * sizeof(T); mi.m_pitch = C; mi.x_pitch = (int64_t)(C >> 4) * sizeof(float);
                mi.a_src = t.a_base + (int64_t)row0 * mi.a_pitch + (int64_t)col0 * sizeof(T);
                mi.m_src = t.m_base + (int64_t)row0 * mi.m_pitch + col0;
                mi.x_src = (kind == MA_KIND_A && !FLAT) ? t.x_base + (int64_t)(row0 >> 4) * mi.x_pitch + (col0 >> 4) * sizeof(float) : nullptr;
                mi.b_src = t.b_base + (int64_t)row0 * mi.a_pitch + (int64_t)col0 * sizeof(T);
                mi.m = reinterpret_cast<int8_t*>(const_cast<unsigned char*>(t.m_base));
                mi.m_absmax = reinterpret_cast<float*>(const_cast<unsigned char*>(t.x_base));
                mi.colpart = t.colpart;
                mi.om_beta1 = t.om_beta1; mi.dq_beta1 = t.dq_beta1; mi.beta1 = t.beta1;
                mi.keep = (int64_t)tile * 100 >= (int64_t)t.ntiles * (100 - keep_pct);
                mi.p = const_cast<unsigned char*>(flat_a ? t.b_base : t.a_base); mi.lr = t.lr; mi.wd_lr = t.wd_lr; mi.decay_mul = t.decay_mul;
                mi.wd_mode = t.wd_mode;
                // the record written above comes before the arrival (same thread); the factor vectors were written by
                // ordinary stores of other CTAs: order them before the bulk copies
                fence_async_global();
                mbar_arrive_expect_tx(&sh->ready[buf], c_bytes + r_bytes + (flat_a ? c_bytes : 0u));   // the one arrival `ready` waits for
                bulk_g2s(sc, t.fac_c + col0, c_bytes, &sh->ready[buf]);
                if (flat_a) {
                    bulk_g2s(s_r + buf * W_TR, t.fac_r0 + row0, r_bytes, &sh->ready[buf]);
                    bulk_g2s(sc2, t.fac_c2 + col0, c_bytes, &sh->ready[buf]);
                } else if (r_bytes) {
                    bulk_g2s(sr, t.fac_r + row0, r_bytes, &sh->ready[buf]);
                }
            }
        };
        auto epilogue = [&](int buf) {
            const MaItem& mi = s_item[buf];
            if (mi.kind != MA_KIND_M) return;
            float* rowpart = a.scr[mi.tensor].rowpart;
            const float* prow = s_row + buf * (W_WARPS * W_TR);
            const int nw = (mi.wcols + 63) >> 6, nrows = min(W_TR, mi.R - mi.row0);
            for (int i = lane; i < nrows; i += 32) {
                float t = 0.0f;
                for (int ww = 0; ww < nw; ++ww) t += prow[ww * W_TR + i];
                rowpart[(int64_t)mi.tc * mi.R + mi.row0 + i] = t;
            }
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(mcount + mi.tensor, 1);
        };
        // Items are handed out dynamically: whoever has a free record buffer takes the next item of the list (a cursor
        // in global memory), so a CTA that was held up simply takes fewer.
        auto dep_met = [&](const Work& x) {
            const int kind = (int)((uint32_t)x.tile >> 28);
            if (kind == MA_KIND_M) return true;
            const Scratch& s = a.scr[x.tensor];
            int got = 0, need = 0;
            if (lane == 0) {
                got = ld_acquire(fcount + x.tensor);
                need = s.nbR + s.nbC + 1;      // every block, and the mean the last one leaves
            }
            return __shfl_sync(0xffffffffu, got >= need ? 1 : 0, 0) != 0;
        };
        bool pending[2] = {false, false};
        int pend_n[2] = {0, 0};
        int n = 0;
        bool have = false, end_sent = false;
        Work w{0, 0};
        uint32_t idle = 0;
        while (true) {
            bool progress = false;
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                if (pending[b] && mbar_test_wait(&sh->done[b], (pend_n[b] >> 1) & 1)) {
                    const long long t0 = MA_CLOCK();
                    epilogue(b);
                    if (lane == 0) MA_PROF_ADD(8, MA_CLOCK() - t0);      // 8: helper epilogues
                    pending[b] = false;
                    progress = true;
                }
            }
            if (!end_sent) {
                const int buf = n & 1;
                if (!have && !pending[buf]) {
                    int idx = 0;
                    if (lane == 0) idx = atomicAdd(next_item, 1);
                    idx = __shfl_sync(0xffffffffu, idx, 0);
                    if (idx < n_items) w = work[idx];
                    else w = Work{0, (int32_t)((uint32_t)MA_KIND_END << 28)};
                    have = true;
                    progress = true;
                }
                if (have) {
                    const int kind = (int)((uint32_t)w.tile >> 28);
                    if (!pending[buf]) {
                        if (kind == MA_KIND_END) {
                            if (lane == 0) s_item[buf].kind = MA_KIND_END;
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&sh->ready[buf]);
                            end_sent = true;
                            have = false;
                            progress = true;
                        } else if (dep_met(w)) {
                            const long long t0 = MA_CLOCK();
                            prepare(w, buf);      // fills the record and arrives on `ready` (release: the waiters see it)
                            if (lane == 0) MA_PROF_ADD(9, MA_CLOCK() - t0);      // 9: helper prepares
                            pending[buf] = true;
                            pend_n[buf] = n;
                            ++n;
                            have = false;
                            progress = true;
                        }
                    }
                }
            } else if (!pending[0] && !pending[1]) {
                break;
            }
            if (progress) {
                idle = 0;
            } else {
                if (have && !pending[n & 1] && lane == 0) MA_PROF_ADD(10, 1);      // 10: polls with an item held for its dependency
                if (*reinterpret_cast<volatile int*>(&sh->abort)) return;
                if (++idle > MA_POLL_LIMIT) {
                    if (lane == 0) { atomicExch(a.status, STATUS_MBAR_TIMEOUT); atomicExch(&sh->abort, 1); }
                    return;
                }
                __nanosleep(128);
            }
        }
        return;
    }

    // ------------------------------------------------------------------------------------------------
    // computing warps
    // ------------------------------------------------------------------------------------------------
    const int c8 = lane & 7, rsub = lane >> 3;
    const int cl = warp * 64 + c8 * 8;          // this lane's first column inside a tile
    const u64 magic = splat(ROUND_MAGIC);
    const uint64_t keep_last = l2_policy_evict_last(), keep_first = l2_policy_evict_first();
    int q = 0;            // position of the next band to consume in this CTA's band stream
    int n = 0;            // items this CTA has gone through

    const bool prof = threadIdx.x == 0;
    long long t_item0 = MA_CLOCK();
    (void)prof; (void)t_item0;
    for (;; ++n) {
        const int buf = n & 1;
        const long long t_r0 = MA_CLOCK();
        if (!ma_wait(&sh->ready[buf], (n >> 1) & 1, sh, a, lane)) { ma_drain(sh, STAGES); return; }
        const MaItem& mi = s_item[buf];
        const int kind = mi.kind;
        if (prof) { MA_PROF_ADD(0 + (kind & 3), MA_CLOCK() - t_r0); MA_PROF_ADD(4, 1); }      // 0..3: wait for a record of kind k
        if (kind == MA_KIND_END) { if (prof) MA_PROF_ADD(5, MA_CLOCK() - t_item0); return; }     // 5: consumer lifetime
        const int R = mi.R, C = mi.C, row0 = mi.row0, nbands = mi.nbands;
        const bool active = cl < mi.wcols;        // warps beyond a ragged tile width idle
        const int col = mi.col0 + cl;
        const float* sr = s_r + buf * W_TR;
        const float* sc = s_c + buf * W_TC;

        if (kind == MA_KIND_M) {
            // ---- momentum tile (reference: kUpdateExpAvgQuantAndResSumsTiled came_kernels.cu:2584-2683) ----
            const int tile_cols = C >> 4;
            float* srow = s_row + buf * (W_WARPS * W_TR);
            u64 cf2[4], colacc[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                cf2[j] = active ? pk(sc[cl + 2 * j], sc[cl + 2 * j + 1]) : F2ZERO;
                colacc[j] = F2ZERO;
            }
            const u64 om2 = splat(mi.om_beta1);
            const float dq_beta1 = mi.dq_beta1;
            const uint64_t keep_policy = mi.keep ? keep_last : keep_first;
            int8_t* mdst = mi.m + (int64_t)(row0 + rsub) * C + col;
            float* amax_dst = mi.m_absmax + (int64_t)(row0 >> 4) * tile_cols + (col >> 4);
            const int64_t band_bytes = (int64_t)W_BAND * C;
            float a_next = (active && !FLAT) ? amax_dst[0] : 0.0f;
            // flat layout: one absmax per (row, 256-column segment); this lane's 4 rows of the band, one band ahead
            const float* amax_flat = mi.m_absmax + (((int64_t)(row0 + rsub) * C + col) >> 8);
            const int64_t flat_row_step = C >> 8;       // absmax entries per row
            float af_next[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (FLAT && active) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (row0 + rsub + 4 * i < R) af_next[i] = amax_flat[(int64_t)(4 * i) * flat_row_step];
            }
            const float* sr_k = sr + rsub;
            float* srow_k = srow + warp * W_TR + rsub;

#pragma unroll 1
            for (int k = 0; k < nbands; ++k, ++q) {
                const int slot = q % STAGES;
                const long long t_f0 = MA_CLOCK();
                if (!ma_wait(&sh->full[slot], (uint32_t)((q / STAGES) & 1), sh, a, lane)) { ma_drain(sh, STAGES); return; }
                if (prof) MA_PROF_ADD(6, MA_CLOCK() - t_f0);      // 6: M bands, wait for data
                if (!active) { __syncwarp(); if (lane == 0) mbar_arrive(&sh->empty[slot]); continue; }
                const unsigned char* sg = smem + slot * STAGE + cl * (int)sizeof(T);
                const unsigned char* sm = smem + slot * STAGE + W_BAND * ROW + cl;
                const int brow = row0 + k * W_BAND;
                const float a_old = a_next;
                if (!FLAT && k + 1 < nbands) a_next = amax_dst[tile_cols];
                const u64 scb2 = splat(a_old * dq_beta1);      // a tile that was never written has absmax 0: scale 0
                float af[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) af[i] = af_next[i];
                if (FLAT && k + 1 < nbands) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (brow + W_BAND + rsub + 4 * i < R)
                            af_next[i] = amax_flat[(int64_t)((k + 1) * W_BAND + 4 * i) * flat_row_step];
                }
                const bool full_band = brow + W_BAND <= R;
                float rsum[4];
                float A = 1.0f;
                auto band = [&](auto full_tag) {
                    constexpr bool FULL = decltype(full_tag)::value;
                    u64 m2[4][4];
                    float amax = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int r = rsub + 4 * i;
                        const bool live = FULL || (brow + r < R);
                        u64 g2[4];
                        wide_run8(reinterpret_cast<const T*>(sg + r * ROW), g2);
                        uint2 mv = *reinterpret_cast<const uint2*>(sm + r * W_MROW);
                        mv.x ^= 0x80808080u; mv.y ^= 0x80808080u;
                        const u64 ra2 = splat(live ? sr_k[4 * i] : 0.0f);
                        const u64 sc_row2 = FLAT ? splat(af[i] * dq_beta1) : scb2;
                        u64 rs2 = F2ZERO;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const u64 u2 = mul2(mul2(g2[j], ra2), cf2[j]);
                            const u64 mo2 = mul2(codes_to_f2(j < 2 ? mv.x : mv.y, (j & 1) * 2), sc_row2);
                            u64 mn = fma2(om2, u2, mo2);
                            u64 df2 = sub2(u2, mn);
                            if (!FULL && !live) { df2 = F2ZERO; mn = F2ZERO; }
                            colacc[j] = fma2(df2, df2, colacc[j]);
                            rs2 = fma2(df2, df2, rs2);
                            if (!FLAT) {
                                amax = fmaxf(amax, fmaxf(fabsf(mn.x), fabsf(mn.y)));
                                m2[i][j] = mn;
                            }
                        }
                        rsum[i] = rs2.x + rs2.y;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->empty[slot]);      // the slot's bytes are in registers now
                    if (FLAT) return;                  // nothing is written in the flat layout
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 16));
                    A = fix_absmax(amax);
                    if (__all_sync(0xffffffffu, recip_safe(A))) {
                        const u64 s127 = splat(QMAX_I8 / A);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            u64 y[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) y[j] = fma2(m2[i][j], s127, magic);
                            if (FULL || brow + rsub + 4 * i < R)
                                st_global_v2_hint(mdst + (int64_t)(4 * i) * C, make_uint2(pack_codes4(y[0], y[1]), pack_codes4(y[2], y[3])), keep_policy);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t out[2];
#pragma unroll
                            for (int t = 0; t < 2; ++t) {
                                const u64 lo2 = m2[i][2 * t], hi2 = m2[i][2 * t + 1];
                                out[t] = ((uint32_t)quant_i8_div(lo2.x, A) & 0xffu) | (((uint32_t)quant_i8_div(lo2.y, A) & 0xffu) << 8) |
                                         (((uint32_t)quant_i8_div(hi2.x, A) & 0xffu) << 16) | (((uint32_t)quant_i8_div(hi2.y, A) & 0xffu) << 24);
                            }
                            if (FULL || brow + rsub + 4 * i < R)
                                st_global_v2_hint(mdst + (int64_t)(4 * i) * C, make_uint2(out[0], out[1]), keep_policy);
                        }
                    }
                };
                if (full_band) band(std::true_type{});
                else band(std::false_type{});
                if (!FLAT && rsub == 0 && (c8 & 1) == 0) *amax_dst = A;     // one lane per tile
                {
                    const bool up4 = (c8 & 4) != 0, up2 = (c8 & 2) != 0;
                    const float a0 = (up4 ? rsum[2] : rsum[0]) + __shfl_xor_sync(0xffffffffu, up4 ? rsum[0] : rsum[2], 4);
                    const float a1 = (up4 ? rsum[3] : rsum[1]) + __shfl_xor_sync(0xffffffffu, up4 ? rsum[1] : rsum[3], 4);
                    float v = (up2 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, up2 ? a0 : a1, 2);
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    const int irow = (up4 ? 2 : 0) + (up2 ? 1 : 0);
                    if ((c8 & 1) == 0) srow_k[4 * irow] = v;
                }
                mdst += band_bytes; amax_dst += tile_cols; sr_k += W_BAND; srow_k += W_BAND;
            }
            if (active) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float lo, hi;
                    upk(colacc[j], lo, hi);
                    lo += __shfl_xor_sync(0xffffffffu, lo, 8);  hi += __shfl_xor_sync(0xffffffffu, hi, 8);
                    lo += __shfl_xor_sync(0xffffffffu, lo, 16); hi += __shfl_xor_sync(0xffffffffu, hi, 16);
                    if (rsub == 0) *reinterpret_cast<float2*>(mi.colpart + (int64_t)mi.tr * C + col + 2 * j) = make_float2(lo, hi);
                }
            }
        } else if (FLAT) {
            // ---- flat-layout apply tile (reference: kCameFactoredExpAvgResPrepare + kCameFactoredParamUpdate,
            //      came_kernels.cu:2246-2305, 2487-2511): bands of 8 rows; warp w owns the 256-column segment (w & 3) of
            //      rows 2 * (w >> 2) and 2 * (w >> 2) + 1 of the band: a warp = one flat block at a time ----
            const int chunk = warp & 3, rpair = warp >> 2;
            const int fcl = chunk * 256 + lane * 8;
            const bool factive = fcl < mi.wcols;
            const int fcol = mi.col0 + fcl;
            const float* sr2 = s_row + buf * (W_WARPS * W_TR);      // R'_i
            const float* sc2 = sr2 + W_TR;                          // C'_j
            u64 cf2[4], cr2[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                cf2[j] = factive ? pk(sc[fcl + 2 * j], sc[fcl + 2 * j + 1]) : F2ZERO;
                cr2[j] = factive ? pk(sc2[fcl + 2 * j], sc2[fcl + 2 * j + 1]) : F2ZERO;
            }
            const int wd_mode = mi.wd_mode;
            const u64 om2 = splat(mi.om_beta1), dmul2 = splat(mi.decay_mul), nwdlr2 = splat(-mi.wd_lr), nlr2 = splat(-mi.lr);
            const float beta1 = mi.beta1;
            const int64_t blocks_per_row = C >> 8;
            float* amax_blk = mi.m_absmax + (int64_t)(row0 + 2 * rpair) * blocks_per_row + (fcol >> 8);
            int8_t* const m_base = mi.m;
            T* const p_base = reinterpret_cast<T*>(mi.p);
            float an[2] = {1.0f, 1.0f};
            if (factive) {
#pragma unroll
                for (int t = 0; t < 2; ++t)
                    if (row0 + 2 * rpair + t < R) an[t] = amax_blk[(int64_t)t * blocks_per_row];
            }
#pragma unroll 1
            for (int k = 0; k < nbands; ++k, ++q) {
                const int slot = q % STAGES;
                const long long t_f0 = MA_CLOCK();
                if (!ma_wait(&sh->full[slot], (uint32_t)((q / STAGES) & 1), sh, a, lane)) { ma_drain(sh, STAGES); return; }
                if (prof) MA_PROF_ADD(7, MA_CLOCK() - t_f0);      // 7: A bands, wait for data
                if (!factive) { __syncwarp(); if (lane == 0) mbar_arrive(&sh->empty[slot]); continue; }
                const unsigned char* st = smem + slot * STAGE;
                const int brow = row0 + k * FLB + 2 * rpair;
                float a_old[2] = {an[0], an[1]};
                if (k + 1 < nbands) {
#pragma unroll
                    for (int t = 0; t < 2; ++t)
                        if (brow + FLB + t < R) an[t] = amax_blk[(int64_t)((k + 1) * FLB + t) * blocks_per_row];
                }
                u64 g2[2][4], p2[2][4];
                uint2 mv[2];
                float ra[2], rr[2];
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const int r = 2 * rpair + t;
                    wide_run8(reinterpret_cast<const T*>(st + r * ROW) + fcl, g2[t]);
                    wide_run8(reinterpret_cast<const T*>(st + FLB * ROW + r * ROW) + fcl, p2[t]);
                    mv[t] = *reinterpret_cast<const uint2*>(st + 2 * FLB * ROW + r * W_MROW + fcl);
                    ra[t] = sr[k * FLB + r];
                    rr[t] = sr2[k * FLB + r];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->empty[slot]);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (brow + t >= R) continue;       // uniform over the warp
                    const uint32_t mx = mv[t].x ^ 0x80808080u, my = mv[t].y ^ 0x80808080u;
                    const u64 ra2 = splat(ra[t]), scb2 = splat((a_old[t] / QMAX_I8) * beta1), rr2 = splat(rr[t]);
                    u64 mn[4];
                    float amax = 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const u64 u2 = mul2(mul2(g2[t][j], ra2), cf2[j]);
                        mn[j] = fma2(om2, u2, mul2(codes_to_f2(j < 2 ? mx : my, (j & 1) * 2), scb2));
                        amax = fmaxf(amax, fmaxf(fabsf(mn[j].x), fabsf(mn[j].y)));
                    }
                    amax = warp_max(amax);
                    const float A = fix_absmax(amax);
                    const int64_t off = (int64_t)(brow + t) * C + fcol;
                    uint32_t out[2];
                    if (recip_safe(A)) {      // uniform: A is a warp-wide value
                        const u64 s127 = splat(QMAX_I8 / A);
                        u64 y[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) y[j] = fma2(mn[j], s127, magic);
                        out[0] = pack_codes4(y[0], y[1]);
                        out[1] = pack_codes4(y[2], y[3]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 2; ++e)
                            out[e] = ((uint32_t)quant_i8_div(mn[2 * e].x, A) & 0xffu) | (((uint32_t)quant_i8_div(mn[2 * e].y, A) & 0xffu) << 8) |
                                     (((uint32_t)quant_i8_div(mn[2 * e + 1].x, A) & 0xffu) << 16) | (((uint32_t)quant_i8_div(mn[2 * e + 1].y, A) & 0xffu) << 24);
                    }
                    *reinterpret_cast<uint2*>(m_base + off) = make_uint2(out[0], out[1]);
                    if (lane == 0) amax_blk[(int64_t)(k * FLB + t) * blocks_per_row] = A;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const u64 upd = mul2(mul2(mn[j], rr2), cr2[j]);
                        u64 pv = p2[t][j];
                        if (wd_mode == 1) pv = fma2(nwdlr2, pv, pv);
                        else if (wd_mode == 2) pv = round_pair<T>(mul2(pv, dmul2));
                        else if (wd_mode == 3) pv = round_pair<T>(fma2(nwdlr2, pv, pv));
                        p2[t][j] = fma2(nlr2, upd, pv);
                    }
                    wide_store8_push(p_base + off, p2[t], a);
                }
            }
        } else {
            // ---- apply tile (reference: kParamUpdateTiled came_kernels.cu:3332-3366, decay of :2678-2682) ----
            u64 cf2[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) cf2[j] = active ? pk(sc[cl + 2 * j], sc[cl + 2 * j + 1]) : F2ZERO;
            const int wd_mode = mi.wd_mode;
            const u64 dmul2 = splat(mi.decay_mul), nwdlr2 = splat(-mi.wd_lr), nlr2 = splat(-mi.lr);
            T* const p_base = reinterpret_cast<T*>(mi.p);
#pragma unroll 1
            for (int k = 0; k < nbands; ++k, ++q) {
                const int slot = q % STAGES;
                const long long t_f0 = MA_CLOCK();
                if (!ma_wait(&sh->full[slot], (uint32_t)((q / STAGES) & 1), sh, a, lane)) { ma_drain(sh, STAGES); return; }
                if (prof) MA_PROF_ADD(7, MA_CLOCK() - t_f0);      // 7: A bands, wait for data
                if (!active) { __syncwarp(); if (lane == 0) mbar_arrive(&sh->empty[slot]); continue; }
                const unsigned char* sp = smem + slot * STAGE + cl * (int)sizeof(T);
                const unsigned char* sm = smem + slot * STAGE + W_BAND * ROW + cl;
                const int brow = row0 + k * W_BAND;
                const bool full_band = brow + W_BAND <= R;
                const float A = *reinterpret_cast<const float*>(smem + slot * STAGE + WideCfg<T>::AMAX_OFF + (cl >> 4) * 4);
                const float scl = A > 0.0f ? A / QMAX_I8 : 0.0f;
                auto band = [&](auto wd_tag, auto full_tag) {
                    constexpr int WD = decltype(wd_tag)::value;
                    constexpr bool FULL = decltype(full_tag)::value;
                    u64 p2[4][4];
                    uint2 mv[4];
                    float rfac[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int r = rsub + 4 * i;
                        wide_run8(reinterpret_cast<const T*>(sp + r * ROW), p2[i]);
                        mv[i] = *reinterpret_cast<const uint2*>(sm + r * W_MROW);
                        rfac[i] = sr[k * W_BAND + r];
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->empty[slot]);
                    T* pdst = p_base + (int64_t)(brow + rsub) * C + col;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t mx = mv[i].x ^ 0x80808080u, my = mv[i].y ^ 0x80808080u;
                        const u64 scr2 = splat(scl * rfac[i]);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const u64 upd = mul2(mul2(codes_to_f2(j < 2 ? mx : my, (j & 1) * 2), scr2), cf2[j]);
                            u64 pv = p2[i][j];
                            if (WD == 2) pv = round_pair<T>(mul2(pv, dmul2));
                            else if (WD == 3) pv = round_pair<T>(fma2(nwdlr2, pv, pv));
                            else if (WD == 1) pv = fma2(nwdlr2, pv, pv);
                            p2[i][j] = fma2(nlr2, upd, pv);
                        }
                        if (FULL || brow + rsub + 4 * i < R) wide_store8_push(pdst + (int64_t)(4 * i) * C, p2[i], a);
                    }
                };
                auto band_wd = [&](auto wd_tag) {
                    if (full_band) band(wd_tag, std::true_type{});
                    else band(wd_tag, std::false_type{});
                };
                switch (wd_mode) {
                    case 0: band_wd(std::integral_constant<int, 0>{}); break;
                    case 1: band_wd(std::integral_constant<int, 1>{}); break;
                    case 2: band_wd(std::integral_constant<int, 2>{}); break;
                    default: band_wd(std::integral_constant<int, 3>{}); break;
                }
            }
        }
        // this warp is through with the item (the helper's fence after `done` orders the warps' global writes before its
        // counter update, as the single fencing thread of a grid barrier does)
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->done[buf]);
    }
}

// ------------------------------------------------------------------------------------------------
// launcher
// ------------------------------------------------------------------------------------------------
template <typename T> static constexpr size_t ma_smem() {
    return (size_t)WideCfg<T>::STAGES * WideCfg<T>::STAGE + sizeof(MaShared) +
           2 * (W_TR + W_TC + W_WARPS * W_TR) * sizeof(float) + 2 * sizeof(MaItem);
}

template <typename T, bool FLAT>
static cudaError_t launch_ma(const StepArgs& a, const Work* work, int n, const Work* fwork, int nf, int* mcount, int* fcount,
                             int* next_item, cudaStream_t st) {
    // CAME_B200_MA_KEEP_PCT: share of a tensor's momentum tiles (the last written) whose codes are marked evict-last
    static const int keep_pct = [] { const char* e = getenv("CAME_B200_MA_KEEP_PCT"); return e ? atoi(e) : 25; }();
    const int sms = persistent_grid_limit();
    const size_t smem = ma_smem<T>();
    cudaError_t e = cudaFuncSetAttribute(k_moment_apply_tile8<T, FLAT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    StepArgs args = a;
    int* next_fitem = next_item + 1;
    int keep = keep_pct;
    void* params[] = {&args, &work, &n, &mcount, &fcount, &next_item, &fwork, &nf, &next_fitem, &keep};
    // cooperative launch: every CTA of the grid is resident at once (CTAs wait for items other CTAs finish)
    return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(k_moment_apply_tile8<T, FLAT>), dim3(n < sms ? n : sms),
                                       dim3(MA_ALL_THREADS), params, smem, st);
}

cudaError_t launch_fused_ma(const KernelKey& key, const StepArgs& a, const Work* work, int n, const Work* fwork, int nf,
                            int* mcount, int* fcount, int* next_item, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    switch (key.g_dtype) {
        case CAME_DT_F32: return key.mode == CAME_MODE_FLAT8 ? launch_ma<float, true>(a, work, n, fwork, nf, mcount, fcount, next_item, st)
                                                  : launch_ma<float, false>(a, work, n, fwork, nf, mcount, fcount, next_item, st);
        case CAME_DT_F16: return key.mode == CAME_MODE_FLAT8 ? launch_ma<__half, true>(a, work, n, fwork, nf, mcount, fcount, next_item, st)
                                                  : launch_ma<__half, false>(a, work, n, fwork, nf, mcount, fcount, next_item, st);
        default: return key.mode == CAME_MODE_FLAT8 ? launch_ma<__nv_bfloat16, true>(a, work, n, fwork, nf, mcount, fcount, next_item, st)
                                                  : launch_ma<__nv_bfloat16, false>(a, work, n, fwork, nf, mcount, fcount, next_item, st);
    }
}

}  // namespace came
