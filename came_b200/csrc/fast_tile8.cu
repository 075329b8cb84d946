// Tile-layout (CAME8bit / CAME8bit2D) momentum and apply passes for matrices whose column count is a
// multiple of 64 and whose buffers are 16-byte aligned.
//
// Persistent CTAs (one per SM: 16 computing warps, one or two copy-issuing warps and, in the momentum pass, a
// helper warp) walk a strided share of the work list.  A work item is a tile of
// 128 rows x up to 1024 columns, consumed in 8 bands of 16 rows.  Bands are staged in shared memory by bulk
// asynchronous copies (TMA, one copy per row per operand: 2 KB / 1 KB, the size at which the copy engine
// reaches full bandwidth) through a ring of mbarriers that runs ahead across item boundaries.  Arithmetic
// uses packed fp32x2 instructions; int8 <-> fp32 conversion goes through byte permutes.
//
// Warp w owns columns [64w, 64w+64) of the tile (four exp_avg tiles).  Within a band a lane owns 8
// consecutive columns (lane & 7) of 4 rows (lane >> 3, +4, +8, +12): column sums stay in 8 registers across
// the bands, row sums need a 3-step shuffle, a 16x16 tile is shared by 8 lanes.
//
// Results equal those of k_moment / k_apply in factored.cu up to the order of a few fp32 roundings.
#include "wide.cuh"

namespace came {

// ------------------------------------------------------------------------------------------------
// momentum pass (reference: kUpdateExpAvgQuantAndResSumsTiled came_kernels.cu:2584-2683)
// ------------------------------------------------------------------------------------------------
// FLAT = false: tile layout, the momentum is re-quantised and written here.  FLAT = true: flat layout (absmax per
// 256 consecutive elements = per 256-column row segment, the column count being a multiple of 256): only the
// residual sums are produced; the flat apply pass recomputes the momentum so that its un-quantised value feeds
// the update (came_kernels.cu:2246-2305 keeps it in fp32 scratch instead).
// What the computing warps need to know about a work item, prepared in shared memory by the helper warp while
// the previous item is being computed (reading it from the tables in global memory would put a chain of
// dependent loads at the start of every item, which the computing warps cannot hide).
constexpr int M_PRODUCERS = 2;                                          // copy-issuing warps of the momentum pass
constexpr int M_ALL_THREADS = W_THREADS + 32 * (M_PRODUCERS + 1);       // + the helper warp

struct MomentItem {
    int8_t* m;              // codes of the tensor
    float* m_absmax;
    float* colpart;
    int R, C, row0, col0, wcols, nbands, tr, pad;
    float om_beta1, dq_beta1;     // 1 - beta1;  beta1 / 127
};

template <typename TG, bool FLAT>
__global__ void __launch_bounds__(M_ALL_THREADS, 1) k_moment_tile8_wide(StepArgs a, const Work* __restrict__ work, int n_items) {
    constexpr int STAGES = WideCfg<TG>::STAGES, STAGE = WideCfg<TG>::STAGE, ROW = WideCfg<TG>::ROW;
    extern __shared__ __align__(128) unsigned char smem[];
    WideShared* sh = reinterpret_cast<WideShared*>(smem + STAGES * STAGE);
    float* s_r = reinterpret_cast<float*>(sh + 1);      // [2][W_TR]   row factors (times 1/clip), double-buffered by item
    float* s_c = s_r + 2 * W_TR;                        // [2][W_TC]   column factors
    float* s_row = s_c + 2 * W_TC;                      // [2][W_WARPS][W_TR]  per-warp row partials of the residual
    MomentItem* s_item = reinterpret_cast<MomentItem*>(s_row + 2 * W_WARPS * W_TR);    // [2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], W_WARPS); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sh->ready[i], 1); mbar_init(&sh->done[i], W_WARPS); }
        sh->abort = 0;
        mbar_init_fence();
    }
    __syncthreads();
    // No CTA-wide barrier from here on: the warps meet only through the ring and the item barriers below, all with
    // bounded, abort-aware waits, so a warp that gives up simply leaves and the others follow at their next wait.
    if (warp < W_WARPS + M_PRODUCERS && warp >= W_WARPS) {
        // producer warps: run the copy stream as far ahead as the ring allows, alternate bands each
        WideProducer<TG> prod;
        prod.init(a, work, n_items, true);
        while (prod.live && prod.issue(a, work, n_items, true, smem, sh, lane, warp - W_WARPS, M_PRODUCERS)) {}
        // after a failed wait somewhere in the CTA: let the copies in flight land before shared memory is released
        if (*reinterpret_cast<volatile int*>(&sh->abort)) wide_drain(sh, STAGES);
        return;
    }
    if (warp == W_WARPS + M_PRODUCERS) {
        // Helper warp.  Items alternate between two buffers (factor slices, item record, per-warp row partials).
        // For the n-th item of this CTA the helper waits until every computing warp has finished it (`done`), sums
        // its per-warp row partials in a fixed order, then prepares item n+2 in the same buffer and publishes it
        // (`ready`).  The computing warps thus never wait for each other at an item boundary, only for `ready`,
        // which normally completed a whole item earlier.
        auto prepare = [&](int item, int buf) {
            const WideItem it = wide_item<TG>(a, work[item], true);
            const CameTensorDesc& d = a.descs[it.tensor];
            const Scratch& s = a.scr[it.tensor];
            const CameHyper& h = a.hyp[d.group];
            float* sr = s_r + buf * W_TR;
            float* sc = s_c + buf * W_TC;
            // The factor slices (r_i / clip and c_j, prepared once per tensor by k_s_finalize) come by bulk copies that
            // complete on the record's `ready` barrier: a loop of dependent global loads in this warp takes as long as
            // the item itself under load.  Rows past the end of the matrix receive whatever follows in the scratch (the
            // copy is rounded up to 16 bytes); the computing warps never use them.
            const uint32_t c_bytes = (uint32_t)it.wcols * sizeof(float);
            const uint32_t r_bytes = (uint32_t)((min(W_TR, it.R - it.row0) + 3) & ~3) * sizeof(float);
            if (lane == 0) {
                MomentItem& mi = s_item[buf];
                mi.m = reinterpret_cast<int8_t*>(d.m); mi.m_absmax = d.m_absmax; mi.colpart = s.colpart;
                mi.R = it.R; mi.C = it.C; mi.row0 = it.row0; mi.col0 = it.col0; mi.wcols = it.wcols;
                mi.nbands = it.nbands; mi.tr = it.tr;
                mi.om_beta1 = h.om_beta1; mi.dq_beta1 = h.beta1 / QMAX_I8;
                // the record written above comes before the arrival (same thread)
                mbar_arrive_expect_tx(&sh->ready[buf], c_bytes + r_bytes);      // the one arrival `ready` waits for
                bulk_g2s(sc, s.mfac_c + it.col0, c_bytes, &sh->ready[buf]);
                bulk_g2s(sr, s.mfac + it.row0, r_bytes, &sh->ready[buf]);
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
        auto publish = [&](int) {};      // `prepare` arrives on `ready` itself (with the factor slices' bytes)
        for (int j = 0; j < 2; ++j)
            if ((int)(blockIdx.x + j * gridDim.x) < n_items) { prepare(blockIdx.x + j * gridDim.x, j); publish(j); }
        int n = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n) {
            const int buf = n & 1;
            if (!wide_wait(&sh->done[buf], (n >> 1) & 1, sh, a, lane)) return;
            row_epilogue(item, buf);
            const int64_t next = (int64_t)item + 2 * (int64_t)gridDim.x;
            if (next < n_items) { prepare((int)next, buf); publish(buf); }
        }
        return;
    }
    const int c8 = lane & 7, rsub = lane >> 3;
    const int cl = warp * 64 + c8 * 8;          // this lane's first column inside the tile
    const u64 magic = splat(ROUND_MAGIC);
    const uint64_t keep_policy = l2_policy_evict_last();      // the new codes are read back by the apply pass
    int q = 0;            // position of the next band to consume in this CTA's band stream
    int n = 0;            // items this CTA has gone through

    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n) {
        const int buf = n & 1;
        if (!wide_wait(&sh->ready[buf], (n >> 1) & 1, sh, a, lane)) { wide_drain(sh, STAGES); return; }
        const MomentItem& mi = s_item[buf];
        const int R = mi.R, C = mi.C, row0 = mi.row0, nbands = mi.nbands;
        const bool active = cl < mi.wcols;        // warps beyond a ragged tile width idle
        const int col = mi.col0 + cl;
        const int tile_cols = C >> 4;
        const float* sr = s_r + buf * W_TR;
        const float* sc = s_c + buf * W_TC;
        float* srow = s_row + buf * (W_WARPS * W_TR);
        u64 cf2[4], colacc[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            cf2[j] = active ? pk(sc[cl + 2 * j], sc[cl + 2 * j + 1]) : F2ZERO;
            colacc[j] = F2ZERO;
        }
        // flat layout: one absmax per (row, 256-column segment); this lane's 4 rows of the band, one band ahead
        const float* amax_flat = mi.m_absmax + (((int64_t)(row0 + rsub) * C + col) >> 8);
        const int64_t flat_row_step = C >> 8;       // absmax entries per row
        float af_next[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (FLAT && active) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (row0 + rsub + 4 * i < R) af_next[i] = amax_flat[(int64_t)(4 * i) * flat_row_step];
        }
        const u64 om2 = splat(mi.om_beta1);
        // old code -> beta1 * (code * absmax / 127) as one scale per tile: absmax * (beta1 / 127)
        const float dq_beta1 = mi.dq_beta1;
        // Pointers that walk down the tile one band at a time (one 64-bit add per band instead of index arithmetic
        // from the table entries, which the barriers in the loop would make the compiler reload on every band)
        int8_t* mdst = mi.m + (int64_t)(row0 + rsub) * C + col;                               // this lane's first row
        float* amax_dst = mi.m_absmax + (int64_t)(row0 >> 4) * tile_cols + (col >> 4);        // this lane's tile
        const int64_t band_bytes = (int64_t)W_BAND * C;
        float a_next = (active && !FLAT) ? amax_dst[0] : 0.0f;
        const float* sr_k = sr + rsub;                                                         // row factors of the band
        float* srow_k = srow + warp * W_TR + rsub;

#pragma unroll 1
        for (int k = 0; k < nbands; ++k, ++q) {
            const int slot = q % STAGES;
            if (!wide_wait_full(a, sh, slot, (q / STAGES) & 1, lane)) { wide_drain(sh, STAGES); return; }      // the status word is set
            if (!active) { wide_release(sh, slot, lane); continue; }
            const unsigned char* sg = smem + slot * STAGE + cl * (int)sizeof(TG);
            const unsigned char* sm = smem + slot * STAGE + W_BAND * ROW + cl;
            const int brow = row0 + k * W_BAND;
            // old absmax of this lane's tile, fetched one band ahead (a dependent global load here would sit on the
            // critical path)
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
            const bool full_band = brow + W_BAND <= R;     // uniform over the CTA
            float rsum[4];
            float A = 1.0f;
            // FULL: all 16 rows of the band exist: no per-row predicate anywhere.  Otherwise (only the last band
            // of a matrix whose row count is not a multiple of 16) rows past the end hold stale bytes in shared
            // memory; whatever they produce is kept out of the sums, the absmax and the stores.
            auto band = [&](auto full_tag) {
                constexpr bool FULL = decltype(full_tag)::value;
                u64 m2[4][4];
                float amax = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int r = rsub + 4 * i;
                    const bool live = FULL || (brow + r < R);
                    u64 g2[4];
                    wide_run8(reinterpret_cast<const TG*>(sg + r * ROW), g2);
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
                        // sums of (u - m)^2; eps1 is added once per row / column when the partials are finalised
                        colacc[j] = fma2(df2, df2, colacc[j]);
                        rs2 = fma2(df2, df2, rs2);
                        if (!FLAT) {
                            amax = fmaxf(amax, fmaxf(fabsf(mn.x), fabsf(mn.y)));
                            m2[i][j] = mn;
                        }
                    }
                    rsum[i] = rs2.x + rs2.y;
                }
                wide_release(sh, slot, lane);      // the slot's bytes are in registers now
                if (FLAT) return;                  // nothing is written in the flat layout
                // tile absmax: the 8 lanes {c8 ^ 1} x {4 row groups} share a 16x16 tile
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 16));
                A = fix_absmax(amax);
                // the reciprocal form needs a normal 1/A: decided per warp so that the branch never diverges
                if (__all_sync(0xffffffffu, recip_safe(A))) {
                    // code = rint((m / A) * 127) computed as rint(m * (127 / A)) in one FMA with the rounding constant:
                    // the argument may differ from the two-step IEEE value in its last bits, which moves a code only
                    // when it lies within ~1e-5 of a rounding boundary (the reference kernel multiplies by a
                    // reciprocal as well, came_kernels.cu:833-836).  The sum's low mantissa byte is the
                    // two's-complement code.
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
                            *reinterpret_cast<uint2*>(mdst + (int64_t)(4 * i) * C) = make_uint2(out[0], out[1]);
                    }
                }
            };
            if (full_band) band(std::true_type{});
            else band(std::false_type{});
            if (!FLAT && rsub == 0 && (c8 & 1) == 0) *amax_dst = A;     // one lane per tile
            // row sums over this warp's 64 columns: halving butterfly over the 8 column groups (4 shuffles instead
            // of 12); lane c8 ends up with the sum of row rsub + 4 * ((c8 >> 1) & 3) when c8 is even
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
        // column partials: the 4 row groups of a warp hold partial sums of the same 8 columns
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
        // this warp is through with the item: its row partials are in shared memory for the helper warp
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->done[buf]);
    }
}

// ------------------------------------------------------------------------------------------------
// apply pass (reference: kParamUpdateTiled came_kernels.cu:3332-3366, weight decay of :2678-2682)
// ------------------------------------------------------------------------------------------------
template <typename TP>
__global__ void __launch_bounds__(W_ALL_THREADS, 1) k_apply_tile8_wide(StepArgs a, const Work* __restrict__ work, int n_items) {
    constexpr int STAGES = WideCfg<TP>::STAGES, STAGE = WideCfg<TP>::STAGE, ROW = WideCfg<TP>::ROW;
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
    if (warp == W_WARPS) {      // producer warp: run the copy stream as far ahead as the ring allows
        WideProducer<TP> prod;
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
        TP* const p_base = reinterpret_cast<TP*>(d.p);      // read once per item, not once per band
        bool ok = true;

#pragma unroll 1
        for (int k = 0; k < it.nbands; ++k, ++q) {
            const int slot = q % STAGES;
            if (!wide_wait_full(a, sh, slot, (q / STAGES) & 1, lane)) { ok = false; break; }
            if (!active) { wide_release(sh, slot, lane); continue; }
            const unsigned char* sp = smem + slot * STAGE + cl * (int)sizeof(TP);
            const unsigned char* sm = smem + slot * STAGE + W_BAND * ROW + cl;
            const int brow = it.row0 + k * W_BAND;
            const bool full_band = brow + W_BAND <= R;
            // absmax of this lane's tile: it came with the band
            const float A = *reinterpret_cast<const float*>(smem + slot * STAGE + WideCfg<TP>::AMAX_OFF + (cl >> 4) * 4);
            const float scl = A > 0.0f ? A / QMAX_I8 : 0.0f;
            // WD: 0 no decay, 1 one rounding, 2 multiply form with a rounding, 3 add form with a rounding.
            // FULL: all 16 rows of the band exist.  Both are uniform over the item, so the inner loops carry no
            // branches.
            auto band = [&](auto wd_tag, auto full_tag) {
                constexpr int WD = decltype(wd_tag)::value;
                constexpr bool FULL = decltype(full_tag)::value;
                u64 p2[4][4];
                uint2 mv[4];
                float rfac[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int r = rsub + 4 * i;
                    wide_run8(reinterpret_cast<const TP*>(sp + r * ROW), p2[i]);
                    mv[i] = *reinterpret_cast<const uint2*>(sm + r * W_MROW);
                    rfac[i] = sr[k * W_BAND + r];
                }
                wide_release(sh, slot, lane);
                TP* pdst = p_base + (int64_t)(brow + rsub) * C + col;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t mx = mv[i].x ^ 0x80808080u, my = mv[i].y ^ 0x80808080u;
                    const u64 scr2 = splat(scl * rfac[i]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const u64 upd = mul2(mul2(codes_to_f2(j < 2 ? mx : my, (j & 1) * 2), scr2), cf2[j]);
                        u64 pv = p2[i][j];
                        if (WD == 2) pv = round_pair<TP>(mul2(pv, dmul2));
                        else if (WD == 3) pv = round_pair<TP>(fma2(nwdlr2, pv, pv));
                        else if (WD == 1) pv = fma2(nwdlr2, pv, pv);
                        p2[i][j] = fma2(nlr2, upd, pv);
                    }
                    if (FULL || brow + rsub + 4 * i < R) wide_store8(pdst + (int64_t)(4 * i) * C, p2[i]);
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
        if (!ok) { aborted = true; continue; }
    }
    if (aborted && warp == 0) wide_drain(sh, STAGES);
}

// ------------------------------------------------------------------------------------------------
// flat-layout apply pass (CAME8bitFull / CAME8bitMemory, column count a multiple of 256): g, m, p -> m, p.
// The momentum is recomputed from g and the old codes (the un-quantised value feeds the update, as in
// kCameFactoredExpAvgResPrepare + kCameFactoredParamUpdate, came_kernels.cu:2246-2305, 2487-2511), re-quantised
// with one absmax per 256-column row segment, and the parameter is updated in the same pass.
// Bands of 8 rows x up to 1024 columns; warp w owns the 256-column segment (w & 3) of rows 2*(w >> 2) and
// 2*(w >> 2) + 1 of the band: a warp = one flat block at a time, its absmax is a warp reduction.
// ------------------------------------------------------------------------------------------------
constexpr int FL_BAND = 8;
constexpr int FL_BANDS = W_TR / FL_BAND;      // 16
template <typename T> struct FlatCfg {
    static constexpr int ROW = W_TC * (int)sizeof(T);
    static constexpr int STAGE = FL_BAND * (2 * ROW + W_MROW);       // g rows, p rows, code rows
    static constexpr int STAGES = sizeof(T) == 2 ? 4 : 2;
};

template <typename T>
__global__ void __launch_bounds__(W_ALL_THREADS, 1) k_apply_flat8_wide(StepArgs a, const Work* __restrict__ work, int n_items) {
    constexpr int STAGES = FlatCfg<T>::STAGES, STAGE = FlatCfg<T>::STAGE, ROW = FlatCfg<T>::ROW;
    extern __shared__ __align__(128) unsigned char smem[];
    WideShared* sh = reinterpret_cast<WideShared*>(smem + STAGES * STAGE);
    float* s_rows = reinterpret_cast<float*>(sh + 1);   // [2][2][W_TR]  per item: r_i / clip, R'_i
    float* s_cols = s_rows + 4 * W_TR;                  // [2][2][W_TC]  per item: c_j, C'_j

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], W_WARPS); }
        sh->abort = 0;
        mbar_init_fence();
    }
    __syncthreads();
    if (warp == W_WARPS) {      // producer: lanes 0-7 copy the band's g rows, 8-15 its code rows, 16-23 its p rows
        int q = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const WideItem it = wide_item<T>(a, work[item], true);
            const unsigned char* p_src = reinterpret_cast<const unsigned char*>(a.descs[it.tensor].p) +
                                         (int64_t)it.row0 * it.a_pitch + (int64_t)it.col0 * sizeof(T);
            const uint32_t a_bytes = (uint32_t)it.wcols * sizeof(T), m_bytes = (uint32_t)it.wcols;
            const int nb = min(FL_BANDS, (it.R - it.row0 + FL_BAND - 1) / FL_BAND);
            for (int band = 0; band < nb; ++band, ++q) {
                const int slot = q % STAGES;
                if (q >= STAGES && !wide_wait(&sh->empty[slot], ((q / STAGES) - 1) & 1, sh, a, lane)) return;
                const int rows = min(FL_BAND, it.R - it.row0 - band * FL_BAND);
                if (lane == 0) mbar_arrive_expect_tx(&sh->full[slot], (uint32_t)rows * (2 * a_bytes + m_bytes));
                __syncwarp();
                const int r = lane & 7, which = lane >> 3;
                if (r < rows && which < 3) {
                    const int64_t row = band * FL_BAND + r;
                    unsigned char* st = smem + slot * STAGE;
                    if (which == 0) bulk_g2s(st + r * ROW, it.a_src + row * it.a_pitch, a_bytes, &sh->full[slot]);
                    else if (which == 1) bulk_g2s(st + 2 * FL_BAND * ROW + r * W_MROW, it.m_src + row * it.m_pitch, m_bytes, &sh->full[slot]);
                    else bulk_g2s(st + FL_BAND * ROW + r * ROW, p_src + row * it.a_pitch, a_bytes, &sh->full[slot]);
                }
            }
        }
        return;
    }
    const int chunk = warp & 3, rpair = warp >> 2;
    const int cl = chunk * 256 + lane * 8;
    const u64 magic = splat(ROUND_MAGIC);
    int q = 0, buf = 0;
    bool aborted = false;

    for (int item = blockIdx.x; item < n_items; item += gridDim.x, buf ^= 1) {
        const WideItem it = wide_item<T>(a, work[item], true);
        const CameTensorDesc& d = a.descs[it.tensor];
        const Scratch& s = a.scr[it.tensor];
        const CameHyper& h = a.hyp[d.group];
        const int R = it.R, C = it.C;
        const bool active = cl < it.wcols;
        const int col = it.col0 + cl;
        float* sr = s_rows + buf * 2 * W_TR;       // [0]: r / clip, [1]: R'
        float* sc = s_cols + buf * 2 * W_TC;       // [0]: c, [1]: C'
        if (!aborted) {
            // r_i / clip and c_j come from the factor vectors k_s_finalize prepared for the momentum pass
            const bool cr = d.flags & CAME_F_RESROW_CLAMP;
            float mean2 = warp_vector_sum(s.rowblk2, s.nbR, lane) / (float)R;
            mean2 = guard_mean(mean2, d.flags & CAME_F_RESROW_FIX, cr);
            for (int i = threadIdx.x; i < W_TR; i += W_CONSUMERS) {
                const bool in = it.row0 + i < R;
                sr[i] = in ? s.mfac[it.row0 + i] : 0.0f;
                sr[W_TR + i] = in ? row_factor(s.Rr[it.row0 + i], mean2, cr) : 0.0f;
            }
            for (int i = threadIdx.x; i < it.wcols; i += W_CONSUMERS) {
                sc[i] = s.mfac_c[it.col0 + i];
                sc[W_TC + i] = col_factor(s.Rc[it.col0 + i], d.flags & CAME_F_RESCOL_CLAMP);
            }
        }
        named_sync(1, W_CONSUMERS);     // met once per item by every consumer warp, also after a failed wait
        if (aborted || *reinterpret_cast<volatile int*>(&sh->abort)) { aborted = true; continue; }
        u64 cf2[4], cr2[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            cf2[j] = active ? pk(sc[cl + 2 * j], sc[cl + 2 * j + 1]) : F2ZERO;
            cr2[j] = active ? pk(sc[W_TC + cl + 2 * j], sc[W_TC + cl + 2 * j + 1]) : F2ZERO;
        }
        const int nb = min(FL_BANDS, (R - it.row0 + FL_BAND - 1) / FL_BAND);
        const int wd_mode = h.weight_decay == 0.0f ? 0 : ((d.flags & CAME_F_WD_MUL2) ? 2 : ((d.flags & CAME_F_WD_ADD2) ? 3 : 1));
        const u64 om2 = splat(h.om_beta1), dmul2 = splat(h.decay_mul), nwdlr2 = splat(-h.wd_lr), nlr2 = splat(-h.lr);
        const float beta1 = h.beta1;
        // absmax of this warp's two flat blocks, one band ahead
        const int64_t blocks_per_row = C >> 8;
        float* amax_blk = d.m_absmax + (int64_t)(it.row0 + 2 * rpair) * blocks_per_row + (col >> 8);
        int8_t* const m_base = reinterpret_cast<int8_t*>(d.m);      // read once per item, not once per band
        T* const p_base = reinterpret_cast<T*>(d.p);
        float an[2] = {1.0f, 1.0f};
        if (active) {
#pragma unroll
            for (int t = 0; t < 2; ++t)
                if (it.row0 + 2 * rpair + t < R) an[t] = amax_blk[(int64_t)t * blocks_per_row];
        }
        bool ok = true;
#pragma unroll 1
        for (int k = 0; k < nb; ++k, ++q) {
            const int slot = q % STAGES;
            if (!wide_wait_full(a, sh, slot, (q / STAGES) & 1, lane)) { ok = false; break; }
            if (!active) { wide_release(sh, slot, lane); continue; }
            const unsigned char* st = smem + slot * STAGE;
            const int brow = it.row0 + k * FL_BAND + 2 * rpair;
            float a_old[2] = {an[0], an[1]};
            if (k + 1 < nb) {
#pragma unroll
                for (int t = 0; t < 2; ++t)
                    if (brow + FL_BAND + t < R) an[t] = amax_blk[(int64_t)((k + 1) * FL_BAND + t) * blocks_per_row];
            }
            u64 g2[2][4], p2[2][4];
            uint2 mv[2];
            float ra[2], rr[2];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const int r = 2 * rpair + t;
                wide_run8(reinterpret_cast<const T*>(st + r * ROW) + cl, g2[t]);
                wide_run8(reinterpret_cast<const T*>(st + FL_BAND * ROW + r * ROW) + cl, p2[t]);
                mv[t] = *reinterpret_cast<const uint2*>(st + 2 * FL_BAND * ROW + r * W_MROW + cl);
                ra[t] = sr[k * FL_BAND + r];
                rr[t] = sr[W_TR + k * FL_BAND + r];
            }
            wide_release(sh, slot, lane);
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
                const int64_t off = (int64_t)(brow + t) * C + col;
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
                if (lane == 0) amax_blk[(int64_t)(k * FL_BAND + t) * blocks_per_row] = A;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const u64 upd = mul2(mul2(mn[j], rr2), cr2[j]);
                    u64 pv = p2[t][j];
                    if (wd_mode == 1) pv = fma2(nwdlr2, pv, pv);
                    else if (wd_mode == 2) pv = round_pair<T>(mul2(pv, dmul2));
                    else if (wd_mode == 3) pv = round_pair<T>(fma2(nwdlr2, pv, pv));
                    p2[t][j] = fma2(nlr2, upd, pv);
                }
                wide_store8(p_base + off, p2[t]);
            }
        }
        if (!ok) { aborted = true; continue; }
    }
    if (aborted && warp == 0) wide_drain(sh, STAGES);
}

// ------------------------------------------------------------------------------------------------
// self-test of the bounded wait: one CTA of two warps waits, through wide_wait with a small limit, on a barrier that
// nothing ever completes.  The first warp to run out records STATUS_MBAR_TIMEOUT in *status and raises the CTA's abort
// flag; the other one leaves at its next poll of the flag; the kernel returns.  Nothing is in flight, nothing faults.
// ------------------------------------------------------------------------------------------------
__global__ void k_selftest_bounded_wait(int* status, int* observed) {
    __shared__ WideShared sh;
    if (threadIdx.x == 0) {
        mbar_init(&sh.full[0], 1);
        sh.abort = 0;
        mbar_init_fence();
    }
    __syncthreads();
    StepArgs a{nullptr, nullptr, nullptr, status};
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // warp 0 runs out after 4096 polls; warp 1 has the full limit and must leave because of the abort flag
    const bool ok = wide_wait(&sh.full[0], 0, &sh, a, lane, warp == 0 ? 4096u : MBAR_SPIN_LIMIT);
    if (lane == 0) observed[warp] = ok ? 1 : 0;
}

cudaError_t launch_selftest_bounded_wait(int* status, int* observed, cudaStream_t st) {
    k_selftest_bounded_wait<<<1, 64, 0, st>>>(status, observed);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------------
template <typename T> static constexpr size_t moment_smem() {
    return (size_t)WideCfg<T>::STAGES * WideCfg<T>::STAGE + sizeof(WideShared) +
           2 * (W_TR + W_TC + W_WARPS * W_TR) * sizeof(float) + 2 * sizeof(MomentItem);
}
template <typename T> static constexpr size_t apply_smem() {
    return (size_t)WideCfg<T>::STAGES * WideCfg<T>::STAGE + sizeof(WideShared) + 2 * (W_TR + W_TC) * sizeof(float);
}

template <typename T> static constexpr size_t flat_smem() {
    return (size_t)FlatCfg<T>::STAGES * FlatCfg<T>::STAGE + sizeof(WideShared) + 4 * (W_TR + W_TC) * sizeof(float);
}

template <typename K>
static cudaError_t launch_persistent(K kernel, size_t smem, const StepArgs& a, const Work* work, int n, cudaStream_t st,
                                     int threads = W_ALL_THREADS) {
    const int sms = persistent_grid_limit();
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kernel<<<n < sms ? n : sms, threads, smem, st>>>(a, work, n);
    return cudaGetLastError();
}

cudaError_t launch_fast_tile8(int kernel, const KernelKey& key, const StepArgs& a, const Work* work, int n,
                              cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    if (kernel == KID_MOMENT) {
        if (key.mode == CAME_MODE_FLAT8) {
            switch (key.g_dtype) {
                case CAME_DT_F32: return launch_persistent(k_moment_tile8_wide<float, true>, moment_smem<float>(), a, work, n, st, M_ALL_THREADS);
                case CAME_DT_F16: return launch_persistent(k_moment_tile8_wide<__half, true>, moment_smem<__half>(), a, work, n, st, M_ALL_THREADS);
                default: return launch_persistent(k_moment_tile8_wide<__nv_bfloat16, true>, moment_smem<__nv_bfloat16>(), a, work, n, st, M_ALL_THREADS);
            }
        }
        switch (key.g_dtype) {
            case CAME_DT_F32: return launch_persistent(k_moment_tile8_wide<float, false>, moment_smem<float>(), a, work, n, st, M_ALL_THREADS);
            case CAME_DT_F16: return launch_persistent(k_moment_tile8_wide<__half, false>, moment_smem<__half>(), a, work, n, st, M_ALL_THREADS);
            default: return launch_persistent(k_moment_tile8_wide<__nv_bfloat16, false>, moment_smem<__nv_bfloat16>(), a, work, n, st, M_ALL_THREADS);
        }
    }
    if (kernel == KID_APPLY_FLAT) {
        switch (key.g_dtype) {
            case CAME_DT_F32: return launch_persistent(k_apply_flat8_wide<float>, flat_smem<float>(), a, work, n, st);
            case CAME_DT_F16: return launch_persistent(k_apply_flat8_wide<__half>, flat_smem<__half>(), a, work, n, st);
            default: return launch_persistent(k_apply_flat8_wide<__nv_bfloat16>, flat_smem<__nv_bfloat16>(), a, work, n, st);
        }
    }
    if (kernel == KID_APPLY) {
        switch (key.p_dtype) {
            case CAME_DT_F32: return launch_persistent(k_apply_tile8_wide<float>, apply_smem<float>(), a, work, n, st);
            case CAME_DT_F16: return launch_persistent(k_apply_tile8_wide<__half>, apply_smem<__half>(), a, work, n, st);
            default: return launch_persistent(k_apply_tile8_wide<__nv_bfloat16>, apply_smem<__nv_bfloat16>(), a, work, n, st);
        }
    }
    return cudaErrorInvalidValue;
}

}  // namespace came
