// fp32-state layout (CAMECUDA): momentum and apply passes staged through shared memory, for matrices whose column
// count is a multiple of 64 and whose buffers are 16-byte aligned.
//
// Same organisation as the tile-layout passes (persistent CTAs, one per SM; tiles of 128 rows x up to 1024 columns;
// bulk asynchronous copies through a ring of mbarriers; packed fp32x2 arithmetic), with the momentum as fp32: a band
// is 8 rows (a row of 1024 fp32 values is 4 KB), a lane owns 8 consecutive columns (lane & 7) of 2 rows (lane >> 3,
// +4), a warp 64 columns.  The new momentum goes from registers to global memory (32 bytes per lane and row).
//
// Results equal those of k_moment / k_apply in factored.cu up to the order of a few fp32 roundings.
// Reference: kCameFactoredExpAvgRes (came_kernels.cu:2307-2342), kCameFactoredParamUpdate (came_kernels.cu:2487-2511).
#include "wide.cuh"

namespace came {

constexpr int FP_BAND = 8;
constexpr int FP_BANDS = W_TR / FP_BAND;          // 16
constexpr int FP_MROW = W_TC * (int)sizeof(float);
template <typename T> struct FpCfg {
    static constexpr int ROW = W_TC * (int)sizeof(T);                 // staged row of the gradient / the parameter
    static constexpr int STAGE = FP_BAND * (ROW + FP_MROW);
    static constexpr int STAGES = sizeof(T) == 2 ? 4 : 3;             // 192 KB either way
};
constexpr int FPM_PRODUCERS = 2;
constexpr int FPM_ALL_THREADS = W_THREADS + 32 * (FPM_PRODUCERS + 1);      // + the helper warp

// The copy stream of one CTA: every band of every work item of the CTA, in consumption order (operand A = gradient
// or parameter rows, then the fp32 momentum rows).
template <typename TA>
struct FpProducer {
    static constexpr int STAGES = FpCfg<TA>::STAGES, STAGE = FpCfg<TA>::STAGE, ROW = FpCfg<TA>::ROW;
    int item, band, q, nbands;
    bool live;
    WideItem it;
    uint64_t stream_policy;
    __device__ __forceinline__ void load(const StepArgs& a, const Work* work, bool a_is_grad) {
        it = wide_item<TA>(a, work[item], a_is_grad);
        it.m_pitch = (int64_t)it.C * sizeof(float);
        it.m_src = reinterpret_cast<const unsigned char*>(a.descs[it.tensor].m) + (int64_t)it.row0 * it.m_pitch +
                   (int64_t)it.col0 * sizeof(float);
        nbands = min(FP_BANDS, (it.R - it.row0 + FP_BAND - 1) / FP_BAND);
    }
    __device__ __forceinline__ void init(const StepArgs& a, const Work* work, int n_items, bool a_is_grad) {
        stream_policy = l2_policy_evict_first();
        item = blockIdx.x; band = 0; q = 0;
        live = item < n_items;
        if (live) load(a, work, a_is_grad);
    }
    __device__ __forceinline__ bool issue(const StepArgs& a, const Work* work, int n_items, bool a_is_grad,
                                          unsigned char* smem, WideShared* sh, int lane, int which = 0, int nprod = 1) {
        if (!live) return true;
        if (nprod == 1 || q % nprod == which) {
            const int slot = q % STAGES;
            if (q >= STAGES) {
                if (!wide_wait(&sh->empty[slot], ((q / STAGES) - 1) & 1, sh, a, lane)) return false;
            }
            const int rows = min(FP_BAND, it.R - it.row0 - band * FP_BAND);
            const uint32_t a_bytes = (uint32_t)it.wcols * sizeof(TA), m_bytes = (uint32_t)it.wcols * sizeof(float);
            if (lane == 0) mbar_arrive_expect_tx(&sh->full[slot], (uint32_t)rows * (a_bytes + m_bytes));
            __syncwarp();
            const int r = lane & 7;
            if (r < rows && lane < 16) {
                const int64_t row = band * FP_BAND + r;
                unsigned char* st = smem + slot * STAGE;
                if (lane < 8) bulk_g2s_hint(st + r * ROW, it.a_src + row * it.a_pitch, a_bytes, &sh->full[slot], stream_policy);
                else bulk_g2s_hint(st + FP_BAND * ROW + r * FP_MROW, it.m_src + row * it.m_pitch, m_bytes, &sh->full[slot], stream_policy);
            }
        }
        ++q;
        if (++band == nbands) {
            band = 0;
            item += gridDim.x;
            live = item < n_items;
            if (live) load(a, work, a_is_grad);
        }
        return true;
    }
};

// ------------------------------------------------------------------------------------------------
// momentum pass: u = g r c / clip, m = beta1 m + (1 - beta1) u (written), sums of (u - m)^2 per row and column
// ------------------------------------------------------------------------------------------------
struct FpMomentItem {
    float* m;
    float* colpart;
    int R, C, row0, col0, wcols, nbands, tr, pad;
    float om_beta1, beta1;
};

template <typename TG>
__global__ void __launch_bounds__(FPM_ALL_THREADS, 1) k_moment_fp32_wide(StepArgs a, const Work* __restrict__ work, int n_items) {
    constexpr int STAGES = FpCfg<TG>::STAGES, STAGE = FpCfg<TG>::STAGE, ROW = FpCfg<TG>::ROW;
    extern __shared__ __align__(128) unsigned char smem[];
    WideShared* sh = reinterpret_cast<WideShared*>(smem + STAGES * STAGE);
    float* s_r = reinterpret_cast<float*>(sh + 1);      // [2][W_TR]   row factors (times 1/clip), double-buffered by item
    float* s_c = s_r + 2 * W_TR;                        // [2][W_TC]   column factors
    float* s_row = s_c + 2 * W_TC;                      // [2][W_WARPS][W_TR]  per-warp row partials of the residual
    FpMomentItem* s_item = reinterpret_cast<FpMomentItem*>(s_row + 2 * W_WARPS * W_TR);    // [2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], W_WARPS); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sh->ready[i], 1); mbar_init(&sh->done[i], W_WARPS); }
        sh->abort = 0;
        mbar_init_fence();
    }
    __syncthreads();
    // No CTA-wide barrier from here on (see k_moment_tile8_wide): bounded, abort-aware waits only.
    if (warp >= W_WARPS && warp < W_WARPS + FPM_PRODUCERS) {
        FpProducer<TG> prod;
        prod.init(a, work, n_items, true);
        while (prod.live && prod.issue(a, work, n_items, true, smem, sh, lane, warp - W_WARPS, FPM_PRODUCERS)) {}
        if (*reinterpret_cast<volatile int*>(&sh->abort)) wide_drain(sh, STAGES);
        return;
    }
    if (warp == W_WARPS + FPM_PRODUCERS) {
        // helper warp: publishes item n + 2 into the buffer item n has left (record + factor slices by bulk copy on the
        // record's `ready` barrier), after summing item n's per-warp row partials in a fixed order
        auto prepare = [&](int item, int buf) {
            const WideItem it = wide_item<TG>(a, work[item], true);
            const CameTensorDesc& d = a.descs[it.tensor];
            const Scratch& s = a.scr[it.tensor];
            const CameHyper& h = a.hyp[d.group];
            const uint32_t c_bytes = (uint32_t)it.wcols * sizeof(float);
            const uint32_t r_bytes = (uint32_t)((min(W_TR, it.R - it.row0) + 3) & ~3) * sizeof(float);
            if (lane == 0) {
                FpMomentItem& mi = s_item[buf];
                mi.m = reinterpret_cast<float*>(d.m); mi.colpart = s.colpart;
                mi.R = it.R; mi.C = it.C; mi.row0 = it.row0; mi.col0 = it.col0; mi.wcols = it.wcols;
                mi.nbands = min(FP_BANDS, (it.R - it.row0 + FP_BAND - 1) / FP_BAND); mi.tr = it.tr;
                mi.om_beta1 = h.om_beta1; mi.beta1 = h.beta1;
                mbar_arrive_expect_tx(&sh->ready[buf], c_bytes + r_bytes);
                bulk_g2s(s_c + buf * W_TC, s.mfac_c + it.col0, c_bytes, &sh->ready[buf]);
                bulk_g2s(s_r + buf * W_TR, s.mfac + it.row0, r_bytes, &sh->ready[buf]);
            }
        };
        auto row_epilogue = [&](int item, int buf) {
            const WideItem it = wide_item<TG>(a, work[item], true);
            float* rowpart = a.scr[it.tensor].rowpart;
            const float* prow = s_row + buf * (W_WARPS * W_TR);
            const int nw = (it.wcols + 63) >> 6, nrows = min(W_TR, it.R - it.row0);
            for (int i = lane; i < nrows; i += 32) {
                float t = 0.0f;
                for (int ww = 0; ww < nw; ++ww) t += prow[ww * W_TR + i];
                rowpart[(int64_t)it.tc * it.R + it.row0 + i] = t;
            }
        };
        for (int j = 0; j < 2; ++j)
            if ((int)(blockIdx.x + j * gridDim.x) < n_items) prepare(blockIdx.x + j * gridDim.x, j);
        int n = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n) {
            const int buf = n & 1;
            if (!wide_wait(&sh->done[buf], (n >> 1) & 1, sh, a, lane)) return;
            row_epilogue(item, buf);
            __syncwarp();      // the partials are read before the buffer is handed out again
            const int64_t next = (int64_t)item + 2 * (int64_t)gridDim.x;
            if (next < n_items) prepare((int)next, buf);
        }
        return;
    }
    const int c8 = lane & 7, rsub = lane >> 3;
    const int cl = warp * 64 + c8 * 8;
    int q = 0, n = 0;

    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n) {
        const int buf = n & 1;
        if (!wide_wait(&sh->ready[buf], (n >> 1) & 1, sh, a, lane)) { wide_drain(sh, STAGES); return; }
        const FpMomentItem& mi = s_item[buf];
        const int R = mi.R, C = mi.C, row0 = mi.row0, nbands = mi.nbands;
        const bool active = cl < mi.wcols;
        const int col = mi.col0 + cl;
        const float* sr = s_r + buf * W_TR;
        const float* sc = s_c + buf * W_TC;
        float* srow = s_row + buf * (W_WARPS * W_TR);
        u64 cf2[4], colacc[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            cf2[j] = active ? pk(sc[cl + 2 * j], sc[cl + 2 * j + 1]) : F2ZERO;
            colacc[j] = F2ZERO;
        }
        const u64 om2 = splat(mi.om_beta1), b2 = splat(mi.beta1);
        float* mdst = mi.m + (int64_t)(row0 + rsub) * C + col;
        const int64_t band_elems = (int64_t)FP_BAND * C;
        const float* sr_k = sr + rsub;
        float* srow_k = srow + warp * W_TR + rsub;

#pragma unroll 1
        for (int k = 0; k < nbands; ++k, ++q) {
            const int slot = q % STAGES;
            if (!wide_wait_full(a, sh, slot, (q / STAGES) & 1, lane)) { wide_drain(sh, STAGES); return; }
            if (!active) { wide_release(sh, slot, lane); continue; }
            const unsigned char* sg = smem + slot * STAGE + cl * (int)sizeof(TG);
            const unsigned char* sm = smem + slot * STAGE + FP_BAND * ROW + cl * (int)sizeof(float);
            const int brow = row0 + k * FP_BAND;
            u64 mn[2][4];
            float rsum[2];
            bool live[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = rsub + 4 * i;
                live[i] = brow + r < R;
                u64 g2[4], m2[4];
                wide_run8(reinterpret_cast<const TG*>(sg + r * ROW), g2);
                wide_run8(reinterpret_cast<const float*>(sm + r * FP_MROW), m2);
                const u64 ra2 = splat(live[i] ? sr_k[4 * i] : 0.0f);
                u64 rs2 = F2ZERO;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const u64 u2 = mul2(mul2(g2[j], ra2), cf2[j]);
                    const u64 x = fma2(om2, u2, mul2(m2[j], b2));
                    u64 df2 = sub2(u2, x);
                    if (!live[i]) df2 = F2ZERO;      // rows past the end hold stale bytes in shared memory
                    // sums of (u - m)^2; eps1 is added once per row / column when the partials are finalised
                    colacc[j] = fma2(df2, df2, colacc[j]);
                    rs2 = fma2(df2, df2, rs2);
                    mn[i][j] = x;
                }
                rsum[i] = rs2.x + rs2.y;
            }
            wide_release(sh, slot, lane);      // the slot's bytes are in registers now
#pragma unroll
            for (int i = 0; i < 2; ++i)
                if (live[i]) wide_store8(mdst + (int64_t)(4 * i) * C, mn[i]);
            // row sums over this warp's 64 columns: halving butterfly over the 8 column groups; lane c8 = 0 ends up with
            // the sum of row rsub, lane c8 = 4 with that of row rsub + 4
            {
                const bool up4 = (c8 & 4) != 0;
                float v = (up4 ? rsum[1] : rsum[0]) + __shfl_xor_sync(0xffffffffu, up4 ? rsum[0] : rsum[1], 4);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                if ((c8 & 3) == 0) srow_k[4 * (c8 >> 2)] = v;
            }
            mdst += band_elems; sr_k += FP_BAND; srow_k += FP_BAND;
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
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->done[buf]);
    }
}

// ------------------------------------------------------------------------------------------------
// apply pass: p -= lr * m * R'_i * C'_j, with the weight-decay forms of apply_one
// ------------------------------------------------------------------------------------------------
template <typename TP>
__global__ void __launch_bounds__(W_ALL_THREADS, 1) k_apply_fp32_wide(StepArgs a, const Work* __restrict__ work, int n_items) {
    constexpr int STAGES = FpCfg<TP>::STAGES, STAGE = FpCfg<TP>::STAGE, ROW = FpCfg<TP>::ROW;
    extern __shared__ __align__(128) unsigned char smem[];
    WideShared* sh = reinterpret_cast<WideShared*>(smem + STAGES * STAGE);
    float* s_r = reinterpret_cast<float*>(sh + 1);      // [2][W_TR]
    float* s_c = s_r + 2 * W_TR;                        // [2][W_TC]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], W_WARPS); }
        sh->abort = 0;
        mbar_init_fence();
    }
    __syncthreads();
    if (warp == W_WARPS) {
        FpProducer<TP> prod;
        prod.init(a, work, n_items, false);
        while (prod.live && prod.issue(a, work, n_items, false, smem, sh, lane)) {}
        return;
    }
    const int c8 = lane & 7, rsub = lane >> 3;
    const int cl = warp * 64 + c8 * 8;
    int q = 0, buf = 0;
    bool aborted = false;

    for (int item = blockIdx.x; item < n_items; item += gridDim.x, buf ^= 1) {
        const WideItem it = wide_item<TP>(a, work[item], false);
        const CameTensorDesc& d = a.descs[it.tensor];
        const Scratch& s = a.scr[it.tensor];
        const CameHyper& h = a.hyp[d.group];
        const int R = it.R, C = it.C;
        const bool active = cl < it.wcols;
        const int col = it.col0 + cl;
        const int nbands = min(FP_BANDS, (R - it.row0 + FP_BAND - 1) / FP_BAND);
        float* sr = s_r + buf * W_TR;
        float* sc = s_c + buf * W_TC;
        if (!aborted) {
            const bool cr = d.flags & CAME_F_RESROW_CLAMP;
            float mean = warp_vector_sum(s.rowblk2, s.nbR, lane) / (float)R;
            mean = guard_mean(mean, d.flags & CAME_F_RESROW_FIX, cr);
            for (int i = threadIdx.x; i < W_TR; i += W_CONSUMERS)
                sr[i] = (it.row0 + i < R) ? row_factor(s.Rr[it.row0 + i], mean, cr) : 0.0f;
            for (int i = threadIdx.x; i < it.wcols; i += W_CONSUMERS)
                sc[i] = col_factor(s.Rc[it.col0 + i], d.flags & CAME_F_RESCOL_CLAMP);
        }
        // hardware barrier among the consumer warps, met once per item even after a failed wait
        named_sync(1, W_CONSUMERS);
        if (aborted || *reinterpret_cast<volatile int*>(&sh->abort)) { aborted = true; continue; }
        u64 cf2[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) cf2[j] = active ? pk(sc[cl + 2 * j], sc[cl + 2 * j + 1]) : F2ZERO;
        const int wd_mode = h.weight_decay == 0.0f ? 0 : ((d.flags & CAME_F_WD_MUL2) ? 2 : ((d.flags & CAME_F_WD_ADD2) ? 3 : 1));
        const u64 dmul2 = splat(h.decay_mul), nwdlr2 = splat(-h.wd_lr), nlr2 = splat(-h.lr);
        TP* const p_base = reinterpret_cast<TP*>(d.p);
        bool ok = true;

#pragma unroll 1
        for (int k = 0; k < nbands; ++k, ++q) {
            const int slot = q % STAGES;
            if (!wide_wait_full(a, sh, slot, (q / STAGES) & 1, lane)) { ok = false; break; }
            if (!active) { wide_release(sh, slot, lane); continue; }
            const unsigned char* sp = smem + slot * STAGE + cl * (int)sizeof(TP);
            const unsigned char* sm = smem + slot * STAGE + FP_BAND * ROW + cl * (int)sizeof(float);
            const int brow = it.row0 + k * FP_BAND;
            u64 p2[2][4], m2[2][4];
            float rfac[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = rsub + 4 * i;
                wide_run8(reinterpret_cast<const TP*>(sp + r * ROW), p2[i]);
                wide_run8(reinterpret_cast<const float*>(sm + r * FP_MROW), m2[i]);
                rfac[i] = sr[k * FP_BAND + r];
            }
            wide_release(sh, slot, lane);
            TP* pdst = p_base + (int64_t)(brow + rsub) * C + col;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const u64 rr2 = splat(rfac[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const u64 upd = mul2(mul2(m2[i][j], rr2), cf2[j]);
                    u64 pv = p2[i][j];
                    if (wd_mode == 1) pv = fma2(nwdlr2, pv, pv);
                    else if (wd_mode == 2) pv = round_pair<TP>(mul2(pv, dmul2));
                    else if (wd_mode == 3) pv = round_pair<TP>(fma2(nwdlr2, pv, pv));
                    p2[i][j] = fma2(nlr2, upd, pv);
                }
                if (brow + rsub + 4 * i < R) wide_store8(pdst + (int64_t)(4 * i) * C, p2[i]);
            }
        }
        if (!ok) { aborted = true; continue; }
    }
    if (aborted && warp == 0) wide_drain(sh, STAGES);
}

// ------------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------------
template <typename T> static constexpr size_t fp_moment_smem() {
    return (size_t)FpCfg<T>::STAGES * FpCfg<T>::STAGE + sizeof(WideShared) +
           2 * (W_TR + W_TC + W_WARPS * W_TR) * sizeof(float) + 2 * sizeof(FpMomentItem);
}
template <typename T> static constexpr size_t fp_apply_smem() {
    return (size_t)FpCfg<T>::STAGES * FpCfg<T>::STAGE + sizeof(WideShared) + 2 * (W_TR + W_TC) * sizeof(float);
}
static_assert(fp_moment_smem<float>() <= 227 * 1024 && fp_moment_smem<__half>() <= 227 * 1024, "shared memory of a CTA");

template <typename K>
static cudaError_t launch_fp_persistent(K kernel, size_t smem, const StepArgs& a, const Work* work, int n, cudaStream_t st, int threads) {
    const int sms = persistent_grid_limit();
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kernel<<<n < sms ? n : sms, threads, smem, st>>>(a, work, n);
    return cudaGetLastError();
}

cudaError_t launch_fp32_wide(int kernel, const KernelKey& key, const StepArgs& a, const Work* work, int n, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    if (kernel == KID_MOMENT) {
        switch (key.g_dtype) {
            case CAME_DT_F32: return launch_fp_persistent(k_moment_fp32_wide<float>, fp_moment_smem<float>(), a, work, n, st, FPM_ALL_THREADS);
            case CAME_DT_F16: return launch_fp_persistent(k_moment_fp32_wide<__half>, fp_moment_smem<__half>(), a, work, n, st, FPM_ALL_THREADS);
            default: return launch_fp_persistent(k_moment_fp32_wide<__nv_bfloat16>, fp_moment_smem<__nv_bfloat16>(), a, work, n, st, FPM_ALL_THREADS);
        }
    }
    if (kernel == KID_APPLY) {
        switch (key.p_dtype) {
            case CAME_DT_F32: return launch_fp_persistent(k_apply_fp32_wide<float>, fp_apply_smem<float>(), a, work, n, st, W_ALL_THREADS);
            case CAME_DT_F16: return launch_fp_persistent(k_apply_fp32_wide<__half>, fp_apply_smem<__half>(), a, work, n, st, W_ALL_THREADS);
            default: return launch_fp_persistent(k_apply_fp32_wide<__nv_bfloat16>, fp_apply_smem<__nv_bfloat16>(), a, work, n, st, W_ALL_THREADS);
        }
    }
    return cudaErrorInvalidValue;
}

}  // namespace came
