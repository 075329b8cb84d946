// CAME step for 2-D (factored) tensors: multi-tensor kernels over a device-side work list.
//
// Pass structure per step (every pass is one launch over all tensors of a kind):
//   sq_partials  : g          -> per-CTA row/col partial sums of g^2 + eps0
//   vec_finalize : partials   -> exp_avg_sq_row/col (EMA, requantised), fresh fp32 copies
//   sumsq        : g          -> per-CTA partials of S = sum (g r c)^2          (RMS clip)
//   s_finalize   : partials   -> S, clip
//   moment       : g, m       -> m (tile8 / fp32 layouts), per-CTA row/col partials of the residual
//   vec_finalize : partials   -> exp_avg_res_row/col
//   apply        : m, p       -> p                       (tile8 / fp32 layouts)
//   factors + apply_flat : g, m, p -> m, p               (flat8 layout: momentum recomputed so that
//                                                          the un-quantised value feeds the update)
// All reductions are two-level with a fixed order, so a step is bit-reproducible run to run.
#include "common.cuh"
#include "launch.h"

namespace came {

// ------------------------------------------------------------------------------------------
// shared: stage the row / column factors of one CTA tile into shared memory
// ------------------------------------------------------------------------------------------
template <int TR, int TC>
__device__ __forceinline__ void stage_factors(const float* __restrict__ vrow, const float* __restrict__ vcol,
                                              const float* __restrict__ rowblk, int nbR, int R, int C, int row0,
                                              int col0, bool fix, bool clamp_row, bool clamp_col, float* s_r,
                                              float* s_c, float* red) {
    float mean = block_vector_sum(rowblk, nbR, red) / (float)R;
    mean = guard_mean(mean, fix, clamp_row);
    for (int i = threadIdx.x; i < TR; i += THREADS) {
        const int row = row0 + i;
        s_r[i] = row < R ? row_factor(vrow[row], mean, clamp_row) : 0.0f;
    }
    for (int i = threadIdx.x; i < TC; i += THREADS) {
        const int col = col0 + i;
        s_c[i] = col < C ? col_factor(vcol[col], clamp_col) : 0.0f;
    }
    __syncthreads();
}

// ------------------------------------------------------------------------------------------
// pass 1: row / column partial sums of g^2 + eps0 over a K_TR x K_TC tile
// (reference: kUpdateSqRowQuantized came_kernels.cu:61-96 and the column walk of :198-243)
// ------------------------------------------------------------------------------------------
template <typename TG, bool VEC>
__global__ void __launch_bounds__(THREADS) k_sq_partials(StepArgs a, const Work* __restrict__ work) {
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const int R = (int)d.rows, C = (int)d.cols;
    const int tr = w.tile / s.tiles_c, tc = w.tile - tr * s.tiles_c;
    const int row0 = tr * K_TR, col0 = tc * K_TC;
    const float eps0 = a.hyp[d.group].eps0, gscale = a.hyp[d.group].grad_scale;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TG* __restrict__ g = reinterpret_cast<const TG*>(d.g);

    __shared__ float s_col[THREADS / 32][K_TC];
    float colacc[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) colacc[e] = 0.0f;

    for (int k = 0; k < K_TR / 8; ++k) {
        const int row = row0 + warp + 8 * k;
        if (row >= R) break;   // uniform per warp
        float racc = 0.0f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int col = col0 + h * 256 + lane * 8;
            if (col < C) {
                float v[8];
                load_run<8, VEC>(g, (int64_t)row * C + col, col, C, v);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    v[e] *= gscale;
                    float q = fmaf(v[e], v[e], eps0);
                    if (!VEC && col + e >= C) q = 0.0f;
                    racc += q;
                    colacc[h * 8 + e] += q;
                }
            }
        }
        racc = warp_sum(racc);
        if (lane == 0) s.rowpart[(int64_t)tc * R + row] = racc;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 8; ++e) s_col[warp][h * 256 + lane * 8 + e] = colacc[h * 8 + e];
    __syncthreads();
    for (int cc = threadIdx.x; cc < K_TC; cc += THREADS) {
        const int col = col0 + cc;
        if (col < C) {
            float t = 0.0f;
#pragma unroll
            for (int ww = 0; ww < THREADS / 32; ++ww) t += s_col[ww][cc];
            s.colpart[(int64_t)tr * C + col] = t;
        }
    }
}

// ------------------------------------------------------------------------------------------
// finalize one block of 256 entries of a row or column vector: EMA with the dequantised old state,
// fresh fp32 copy for the following passes, requantisation (uint8, absmax = block max, 0 -> 1).
// RES=false: second moment (beta2, partials of pass 1); RES=true: residual (beta3, partials of moment).
// (reference: came_kernels.cu:77-93, 215-242, 298-333, 2685-2706, 2742-2779, 524-593, 1436-1487)
// ------------------------------------------------------------------------------------------
// Sum of the `parts` rows of a [parts x n] matrix of column partials for the 256 columns of block b; the result
// for column b * 256 + threadIdx.x.  Warp w adds the rows w, w + 8, ... (a lane holds 8 columns: two 16-byte loads
// per row), then the eight per-warp sums are added in a fixed order: the chain of dependent loads is parts / 8
// long instead of parts, and the order of the additions does not depend on timing.
__device__ __forceinline__ float column_partial_sum(const float* __restrict__ part, int parts, int n, int b,
                                                    float (*s_acc)[QBLOCK]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c0 = b * QBLOCK + lane * 8;
    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    const bool vec = (n & 3) == 0 && (reinterpret_cast<uintptr_t>(part) & 15) == 0 && c0 + 8 <= n;
    if (vec) {
#pragma unroll 8
        for (int t = warp; t < parts; t += THREADS / 32) {
            const float4* p = reinterpret_cast<const float4*>(part + (int64_t)t * n + c0);
            const float4 x = p[0], y = p[1];
            acc[0] += x.x; acc[1] += x.y; acc[2] += x.z; acc[3] += x.w;
            acc[4] += y.x; acc[5] += y.y; acc[6] += y.z; acc[7] += y.w;
        }
    } else {
        for (int t = warp; t < parts; t += THREADS / 32)
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (c0 + e < n) acc[e] += part[(int64_t)t * n + c0 + e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) s_acc[warp][lane * 8 + e] = acc[e];
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) r += s_acc[w][threadIdx.x];
    __syncthreads();      // the buffer may be reused right away
    return r;
}

template <bool RES>
__global__ void __launch_bounds__(THREADS) k_vec_finalize(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    __shared__ float s_acc[THREADS / 32][QBLOCK];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const int R = (int)d.rows, C = (int)d.cols;
    const bool is_col = w.tile >= s.nbR;
    const int b = is_col ? w.tile - s.nbR : w.tile;
    const int n = is_col ? C : R;
    const int idx = b * QBLOCK + threadIdx.x;
    const bool valid = idx < n;
    const bool quant = d.mode != CAME_MODE_FP32;
    const float beta = RES ? h.beta3 : h.beta2;
    const float om = RES ? h.om_beta3 : h.om_beta2;

    void* state = RES ? (is_col ? d.res_col : d.res_row) : (is_col ? d.sq_col : d.sq_row);
    float* absmax = RES ? (is_col ? d.res_col_absmax : d.res_row_absmax) : (is_col ? d.sq_col_absmax : d.sq_row_absmax);
    float* fresh = RES ? (is_col ? s.Rc : s.Rr) : (is_col ? s.vc : s.vr);

    // the fused first pass delivers finished v_row values, column sums without eps0, and tpart
    const bool fused = !RES && s.fused_a;
    float v = 0.0f, tsum = 0.0f;
    // column partials: summed by the whole block together (every thread takes part, also beyond the last column)
    float colsum = 0.0f;
    if (is_col) {
        const int parts = RES ? s.ptiles_r : s.sq_col_parts;
        colsum = column_partial_sum(s.colpart, parts, C, b, s_acc);
        if (fused) {      // the fused first pass sums the raw gradient: the gradient scale enters here, squared
            const float gs2 = h.grad_scale * h.grad_scale;
            tsum = column_partial_sum(s.tpart, parts, C, b, s_acc) * gs2;
            colsum *= gs2;
        }
    }
    if (valid) {
        if (fused && !is_col) {
            v = s.vr[idx];
        } else {
            float acc = 0.0f;
            if (!is_col) {
                const int parts = RES ? s.ptiles_c : s.tiles_c;
                for (int t = 0; t < parts; ++t) acc += s.rowpart[(int64_t)t * R + idx];
                acc = (RES && s.res_eps_deferred) ? mean_plus_eps(acc, (float)C, h.eps1) : __fdiv_rn(acc, (float)C);
            } else {
                acc = colsum;
                if (fused) acc = __fadd_rn(acc, __fmul_rn((float)R, h.eps0));
                acc = (RES && s.res_eps_deferred) ? mean_plus_eps(acc, (float)R, h.eps1) : __fdiv_rn(acc, (float)R);
            }
            float old;
            if (quant) {
                old = (float)reinterpret_cast<const uint8_t*>(state)[idx] * (absmax[b] / QMAX_U8);
            } else {
                old = reinterpret_cast<const float*>(state)[idx];
            }
            v = ema_update(old, beta, om, acc);
            fresh[idx] = v;
        }
    }
    // The fused first pass gets the clip sum from a closed form that assumes r_i^2 = mean / v_row_i and c_j^2 = 1 / v_col_j,
    // i.e. that none of the 1e-30 clamps binds.  Far outside this range one could: the two-pass sum then runs instead.
    if (fused && (d.flags & CAME_F_SQ_CLAMP) && valid && !(v >= 1e-20f && v <= 1e8f)) s.scal[3] = 1.0f;
    if (quant) {
        const float bmax = fix_absmax(block_max(valid ? v : 0.0f, red));   // syncs: every old absmax read is done
        if (threadIdx.x == 0) absmax[b] = bmax;
        if (valid) reinterpret_cast<uint8_t*>(state)[idx] = (uint8_t)quant_u8_div(v, bmax);
    } else if (valid) {
        reinterpret_cast<float*>(state)[idx] = v;
    }
    if (!is_col) {
        const float bs = block_sum(valid ? v : 0.0f, red);
        if (threadIdx.x == 0) (RES ? s.rowblk2 : s.rowblk)[b] = bs;
    } else if (fused) {
        // this block's share of sum_j T_j / v_col_j  (S = mean(v_row) * that sum, see fused_sq.cu)
        const float bs = block_sum((valid && v > 0.0f) ? tsum / v : 0.0f, red);
        if (threadIdx.x == 0) s.spart[b] = bs;
    }
}

// ------------------------------------------------------------------------------------------
// pass 2: partials of S = sum (g * r_i * c_j)^2   (reference: kSumUpdateSq came_kernels.cu:596-619)
// ------------------------------------------------------------------------------------------
template <typename TG, bool VEC>
__global__ void __launch_bounds__(THREADS) k_sumsq(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    __shared__ float s_r[K_TR];
    __shared__ float s_c[K_TC];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    if (s.fused_a && s.scal[3] == 0.0f) return;      // the fused first pass's closed form stands: nothing to do
    const int R = (int)d.rows, C = (int)d.cols;
    const int tr = w.tile / s.tiles_c, tc = w.tile - tr * s.tiles_c;
    const int row0 = tr * K_TR, col0 = tc * K_TC;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TG* __restrict__ g = reinterpret_cast<const TG*>(d.g);
    const bool clamp = d.flags & CAME_F_SQ_CLAMP;
    const float gscale = a.hyp[d.group].grad_scale;
    stage_factors<K_TR, K_TC>(s.vr, s.vc, s.rowblk, s.nbR, R, C, row0, col0, d.flags & CAME_F_SQ_FIX, clamp, clamp,
                              s_r, s_c, red);
    float cf[16];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int e = 0; e < 8; ++e) cf[hh * 8 + e] = s_c[hh * 256 + lane * 8 + e];

    float acc = 0.0f;
    for (int k = 0; k < K_TR / 8; ++k) {
        const int rl = warp + 8 * k;
        const int row = row0 + rl;
        if (row >= R) break;
        const float r = s_r[rl];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int col = col0 + hh * 256 + lane * 8;
            if (col < C) {
                float v[8];
                load_run<8, VEC>(g, (int64_t)row * C + col, col, C, v);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float u = ((v[e] * gscale) * r) * cf[hh * 8 + e];   // masked elements: v = 0, cf = 0
                    acc = fmaf(u, u, acc);
                }
            }
        }
    }
    const float t = block_sum(acc, red);
    if (threadIdx.x == 0) s.spart[w.tile] = t;
}

// S and the clip divisor of one tensor (reference: kReducePartialSum came_kernels.cu:763-779 and
// clip = max(1, sqrt(S/n)/clip_threshold), came_kernels.cu:2619-2620)
__global__ void __launch_bounds__(THREADS) k_s_finalize(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    float S;
    if (s.fused_a && s.scal[3] == 0.0f) {
        float mean = block_vector_sum(s.rowblk, s.nbR, red) / (float)d.rows;
        mean = guard_mean(mean, d.flags & CAME_F_SQ_FIX, d.flags & CAME_F_SQ_CLAMP);
        S = mean * block_vector_sum(s.spart, s.nbC, red);
    } else {
        S = block_vector_sum(s.spart, s.tiles_r * s.tiles_c, red);
    }
    const float n = (float)((int64_t)d.rows * d.cols);
    const float clip = fmaxf(1.0f, sqrtf(S / n) / a.hyp[d.group].clip_threshold);   // S is the same in every thread
    if (threadIdx.x == 0 && w.tile == 0) {
        s.scal[0] = S;
        s.scal[1] = clip;
    }
    if (s.mfac) {
        // factor vectors of the momentum pass, once per tensor instead of once per tile: r_i / clip, then c_j
        const bool clamp = d.flags & CAME_F_SQ_CLAMP;
        float mean = block_vector_sum(s.rowblk, s.nbR, red) / (float)d.rows;
        mean = guard_mean(mean, d.flags & CAME_F_SQ_FIX, clamp);
        const float inv_clip = 1.0f / clip;
        const int R = (int)d.rows, C = (int)d.cols;
        const int hi = min(R + C, (w.tile + 1) * S_FIN_CHUNK);      // this CTA's chunk of the R + C entries
        for (int i = w.tile * S_FIN_CHUNK + threadIdx.x; i < hi; i += THREADS)
            if (i < R) s.mfac[i] = row_factor(s.vr[i], mean, clamp) * inv_clip * a.hyp[d.group].grad_scale;   // g enters u through it
            else s.mfac_c[i - R] = col_factor(s.vc[i - R], clamp);
    }
}

// ------------------------------------------------------------------------------------------
// pass 3: u = g r c / clip, m = beta1 m + (1-beta1) u, residual (u-m)^2 + eps1 -> row/col partials.
// A lane owns 16 consecutive columns of one row; a warp covers 16 rows x 32 columns (two exp_avg
// tiles) per iteration and walks down P_TR rows.
//   TILE8: m re-quantised per 16x16 tile and written        (came_kernels.cu:2584-2683)
//   FP32 : m written in place                                (came_kernels.cu:2307-2342)
//   FLAT8: nothing written; the flat apply pass recomputes m (came_kernels.cu:2246-2305 computes the
//          same values into fp32 scratch)
// ------------------------------------------------------------------------------------------
template <typename TG, int MODE, bool VEC>
__global__ void __launch_bounds__(THREADS) k_moment(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    __shared__ float s_r[P_TR];
    __shared__ float s_c[P_TC];
    __shared__ float s_row[THREADS / 32][P_TR];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const int R = (int)d.rows, C = (int)d.cols;
    const int tr = w.tile / s.ptiles_c, tc = w.tile - tr * s.ptiles_c;
    const int row0 = tr * P_TR, col0 = tc * P_TC;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rl = lane >> 1, half = lane & 1;
    const TG* __restrict__ g = reinterpret_cast<const TG*>(d.g);
    const bool clamp = d.flags & CAME_F_SQ_CLAMP;
    stage_factors<P_TR, P_TC>(s.vr, s.vc, s.rowblk, s.nbR, R, C, row0, col0, d.flags & CAME_F_SQ_FIX, clamp, clamp,
                              s_r, s_c, red);
    const float inv_clip = 1.0f / s.scal[1];
    const float beta1 = h.beta1, om1 = h.om_beta1, eps1 = h.eps1;
    const int cl = warp * 32 + half * 16;      // column offset inside the CTA tile
    const int col = col0 + cl;
    const int tile_cols = (C + TILE - 1) / TILE;
    float cf[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) cf[e] = s_c[cl + e];
    float colacc[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) colacc[e] = 0.0f;

    for (int k = 0; k < P_TR / TILE; ++k) {
        const int rloc = k * TILE + rl;
        const int row = row0 + rloc;
        if (row0 + k * TILE >= R) {            // uniform per CTA: the tile-row is entirely out of range
            if (half == 0) s_row[warp][rloc] = 0.0f;
            continue;
        }
        const bool live = row < R && col < C;
        const int64_t off = (int64_t)row * C + col;
        float gv[16], m[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) { gv[e] = 0.0f; m[e] = 0.0f; }
        if (live) {
            load_run<16, VEC>(g, off, col, C, gv);
            if (MODE == CAME_MODE_FP32) {
                load_run<16, VEC>(reinterpret_cast<const float*>(d.m), off, col, C, m);
            } else {
                load_codes<16, VEC>(reinterpret_cast<const int8_t*>(d.m), off, col, C, m);
                if (MODE == CAME_MODE_TILE8) {
                    const float a_old = d.m_absmax[(int64_t)(row >> 4) * tile_cols + (col >> 4)];
                    const float sc = a_old > 0.0f ? a_old / QMAX_I8 : 0.0f;
#pragma unroll
                    for (int e = 0; e < 16; ++e) m[e] *= sc;
                } else {
                    const int64_t last = ((int64_t)R * C - 1) >> 8;
                    const int64_t b0 = off >> 8, b1 = min((off + 15) >> 8, last);
                    const float sc0 = d.m_absmax[b0] / QMAX_I8;
                    const float sc1 = d.m_absmax[b1] / QMAX_I8;
#pragma unroll
                    for (int e = 0; e < 16; ++e) m[e] *= (((off + e) >> 8) == b0) ? sc0 : sc1;
                }
            }
        }
        const float r = s_r[rloc];
        float rs = 0.0f, amax = 0.0f;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const float u = (((gv[e] * h.grad_scale) * r) * cf[e]) * inv_clip;
            const float mn = m[e] * beta1 + om1 * u;
            const float df = u - mn;
            float res = fmaf(df, df, eps1);
            if (!live || (!VEC && col + e >= C)) res = 0.0f;
            rs += res;
            colacc[e] += res;
            m[e] = mn;
            amax = fmaxf(amax, fabsf(mn));
        }
        if (MODE == CAME_MODE_TILE8) {
#pragma unroll
            for (int o = 2; o <= 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float A = fix_absmax(amax);
            if (live) {
                int q[16];
                if (recip_safe(A)) {
                    const float inv = 1.0f / A;
#pragma unroll
                    for (int e = 0; e < 16; ++e) q[e] = quant_i8_fast(m[e], A, inv);
                } else {
#pragma unroll
                    for (int e = 0; e < 16; ++e) q[e] = quant_i8_div(m[e], A);
                }
                store_codes<16, VEC>(reinterpret_cast<int8_t*>(d.m), off, col, C, q);
            }
            // one lane per tile writes the absmax: the lane holding the tile's first row
            if (rl == 0 && col < C) d.m_absmax[(int64_t)((row0 + k * TILE) >> 4) * tile_cols + (col >> 4)] = A;
        } else if (MODE == CAME_MODE_FP32) {
            if (live) store_run<16, VEC>(reinterpret_cast<float*>(d.m), off, col, C, m);
        }
        rs += __shfl_xor_sync(0xffffffffu, rs, 1);
        if (half == 0) s_row[warp][rloc] = rs;
    }
    // column partials: sum over the 16 lanes that share `half`
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        float v = colacc[e];
#pragma unroll
        for (int o = 2; o <= 16; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        colacc[e] = v;
    }
    if (rl == 0) {
#pragma unroll
        for (int e = 0; e < 16; ++e)
            if (col + e < C) s.colpart[(int64_t)tr * C + col + e] = colacc[e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < P_TR; i += THREADS) {
        const int row = row0 + i;
        if (row < R) {
            float t = 0.0f;
#pragma unroll
            for (int ww = 0; ww < THREADS / 32; ++ww) t += s_row[ww][i];
            s.rowpart[(int64_t)tc * R + row] = t;
        }
    }
}

// ------------------------------------------------------------------------------------------
// pass 4 (tile8 / fp32 layouts): p -= lr * m * R'_i * C'_j, m read back from the state
// (tile8 uses the re-quantised momentum: kParamUpdateTiled came_kernels.cu:3332-3366;
//  fp32: kCameFactoredParamUpdate came_kernels.cu:2487-2511)
// ------------------------------------------------------------------------------------------
template <typename TP, int MODE, bool VEC>
__global__ void __launch_bounds__(THREADS) k_apply(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    __shared__ float s_r[P_TR];
    __shared__ float s_c[P_TC];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const int R = (int)d.rows, C = (int)d.cols;
    const int tr = w.tile / s.ptiles_c, tc = w.tile - tr * s.ptiles_c;
    const int row0 = tr * P_TR, col0 = tc * P_TC;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rl = lane >> 1, half = lane & 1;
    stage_factors<P_TR, P_TC>(s.Rr, s.Rc, s.rowblk2, s.nbR, R, C, row0, col0, d.flags & CAME_F_RESROW_FIX,
                              d.flags & CAME_F_RESROW_CLAMP, d.flags & CAME_F_RESCOL_CLAMP, s_r, s_c, red);
    const int cl = warp * 32 + half * 16;
    const int col = col0 + cl;
    if (col >= C) return;
    const int tile_cols = (C + TILE - 1) / TILE;
    TP* __restrict__ p = reinterpret_cast<TP*>(d.p);
    float cf[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) cf[e] = s_c[cl + e];

    for (int k = 0; k < P_TR / TILE; ++k) {
        const int rloc = k * TILE + rl;
        const int row = row0 + rloc;
        if (row >= R) continue;
        const int64_t off = (int64_t)row * C + col;
        float m[16], pv[16];
        if (MODE == CAME_MODE_FP32) {
            load_run<16, VEC>(reinterpret_cast<const float*>(d.m), off, col, C, m);
        } else {
            load_codes<16, VEC>(reinterpret_cast<const int8_t*>(d.m), off, col, C, m);
            const float A = d.m_absmax[(int64_t)(row >> 4) * tile_cols + (col >> 4)];
            const float sc = A > 0.0f ? A / QMAX_I8 : 0.0f;
#pragma unroll
            for (int e = 0; e < 16; ++e) m[e] *= sc;
        }
        load_run<16, VEC>(p, off, col, C, pv);
        const float r = s_r[rloc];
#pragma unroll
        for (int e = 0; e < 16; ++e) pv[e] = apply_one<TP>(pv[e], (m[e] * r) * cf[e], h, d.flags);
        store_run<16, VEC>(p, off, col, C, pv);
    }
}

// ------------------------------------------------------------------------------------------
// flat8 layout: factor arrays (r, c from the second moment; R', C' from the residual), then the
// apply pass in flat coordinates: a warp owns one block of 256 consecutive elements.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS) k_factors(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const int R = (int)d.rows, C = (int)d.cols;
    const bool is_col = w.tile >= s.nbR;
    const int b = is_col ? w.tile - s.nbR : w.tile;
    const int idx = b * QBLOCK + threadIdx.x;
    float* r = s.fac;
    float* c = r + R;
    float* rr = c + C;
    float* rc = rr + R;
    if (is_col) {
        if (idx < C) {
            c[idx] = col_factor(s.vc[idx], d.flags & CAME_F_SQ_CLAMP);
            rc[idx] = col_factor(s.Rc[idx], d.flags & CAME_F_RESCOL_CLAMP);
        }
        return;
    }
    float mean = block_vector_sum(s.rowblk, s.nbR, red) / (float)R;
    mean = guard_mean(mean, d.flags & CAME_F_SQ_FIX, d.flags & CAME_F_SQ_CLAMP);
    float mean2 = block_vector_sum(s.rowblk2, s.nbR, red) / (float)R;
    mean2 = guard_mean(mean2, d.flags & CAME_F_RESROW_FIX, d.flags & CAME_F_RESROW_CLAMP);
    if (idx < R) {
        r[idx] = row_factor(s.vr[idx], mean, d.flags & CAME_F_SQ_CLAMP);
        rr[idx] = row_factor(s.Rr[idx], mean2, d.flags & CAME_F_RESROW_CLAMP);
    }
}

// (reference: kCameFactoredExpAvgResPrepare came_kernels.cu:2246-2305 for m and its flat-256 absmax,
//  kCameFactoredParamUpdate came_kernels.cu:2487-2511 for p with the un-quantised m)
template <typename TG, typename TP, bool VEC>
__global__ void __launch_bounds__(THREADS) k_apply_flat(StepArgs a, const Work* __restrict__ work) {
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const int R = (int)d.rows, C = (int)d.cols;
    const int64_t n = (int64_t)R * C;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TG* __restrict__ g = reinterpret_cast<const TG*>(d.g);
    TP* __restrict__ p = reinterpret_cast<TP*>(d.p);
    int8_t* __restrict__ mq = reinterpret_cast<int8_t*>(d.m);
    const float* __restrict__ fr = s.fac;
    const float* __restrict__ fc = fr + R;
    const float* __restrict__ frr = fc + C;
    const float* __restrict__ frc = frr + R;
    const float inv_clip = 1.0f / s.scal[1];
    const float beta1 = h.beta1, om1 = h.om_beta1;

    for (int bi = warp; bi < FLAT_BLOCKS_PER_CTA; bi += THREADS / 32) {
        const int64_t blk = (int64_t)w.tile * FLAT_BLOCKS_PER_CTA + bi;
        const int64_t base = blk * QBLOCK;
        if (base >= n) break;
        const int64_t idx = base + lane * 8;
        // masking of the ragged tail goes through the (col, ncols) arguments of the run helpers
        const int rem = (int)((n - idx) > 8 ? 8 : (n - idx));   // may be <= 0
        float gv[8], m[8], pv[8], upd[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) { gv[e] = 0.0f; m[e] = 0.0f; pv[e] = 0.0f; }
        const bool live = rem > 0;
        if (live) {
            load_run<8, VEC>(g, idx, 0, rem, gv);
            load_codes<8, VEC>(mq, idx, 0, rem, m);
            load_run<8, VEC>(p, idx, 0, rem, pv);
        }
        const float sc = d.m_absmax[blk] / QMAX_I8;
        int row = (int)(idx / C);
        int col = (int)(idx - (int64_t)row * C);
        float amax = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float mn = 0.0f;
            upd[e] = 0.0f;
            if (e < rem) {
                const float u = (((gv[e] * h.grad_scale) * fr[row]) * fc[col]) * inv_clip;
                mn = (m[e] * sc) * beta1 + om1 * u;
                upd[e] = (mn * frr[row]) * frc[col];
            }
            m[e] = mn;
            amax = fmaxf(amax, fabsf(mn));
            if (++col == C) { col = 0; ++row; if (row >= R) row = R - 1; }
        }
        amax = warp_max(amax);
        const float A = fix_absmax(amax);
        if (live) {
            int q[8];
            if (recip_safe(A)) {
                const float inv = 1.0f / A;
#pragma unroll
                for (int e = 0; e < 8; ++e) q[e] = quant_i8_fast(m[e], A, inv);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) q[e] = quant_i8_div(m[e], A);
            }
            store_codes<8, VEC>(mq, idx, 0, rem, q);
#pragma unroll
            for (int e = 0; e < 8; ++e) pv[e] = apply_one<TP>(pv[e], upd[e], h, d.flags);
            store_run<8, VEC>(p, idx, 0, rem, pv);
        }
        if (lane == 0) d.m_absmax[blk] = A;
    }
}

// ------------------------------------------------------------------------------------------
// host-side launchers
// ------------------------------------------------------------------------------------------
template <typename F>
static cudaError_t go(F kernel, const StepArgs& a, const Work* work, int n, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    kernel<<<n, THREADS, 0, st>>>(a, work);
    return cudaGetLastError();
}

#define DISPATCH_G(FN, dt, ...)                                              \
    switch (dt) {                                                            \
        case CAME_DT_F32: return FN<float, __VA_ARGS__>;                     \
        case CAME_DT_F16: return FN<__half, __VA_ARGS__>;                    \
        default: return FN<__nv_bfloat16, __VA_ARGS__>;                      \
    }

using KernelFn = void (*)(StepArgs, const Work*);

static KernelFn pick_sq_partials(int g, bool vec) {
    if (vec) { DISPATCH_G(k_sq_partials, g, true) } else { DISPATCH_G(k_sq_partials, g, false) }
}
static KernelFn pick_sumsq(int g, bool vec) {
    if (vec) { DISPATCH_G(k_sumsq, g, true) } else { DISPATCH_G(k_sumsq, g, false) }
}
static KernelFn pick_moment(int g, int mode, bool vec) {
    switch (mode) {
        case CAME_MODE_FP32:
            if (vec) { DISPATCH_G(k_moment, g, CAME_MODE_FP32, true) } else { DISPATCH_G(k_moment, g, CAME_MODE_FP32, false) }
        case CAME_MODE_TILE8:
            if (vec) { DISPATCH_G(k_moment, g, CAME_MODE_TILE8, true) } else { DISPATCH_G(k_moment, g, CAME_MODE_TILE8, false) }
        default:
            if (vec) { DISPATCH_G(k_moment, g, CAME_MODE_FLAT8, true) } else { DISPATCH_G(k_moment, g, CAME_MODE_FLAT8, false) }
    }
}
static KernelFn pick_apply(int p, int mode, bool vec) {
    if (mode == CAME_MODE_FP32) {
        if (vec) { DISPATCH_G(k_apply, p, CAME_MODE_FP32, true) } else { DISPATCH_G(k_apply, p, CAME_MODE_FP32, false) }
    }
    if (vec) { DISPATCH_G(k_apply, p, CAME_MODE_TILE8, true) } else { DISPATCH_G(k_apply, p, CAME_MODE_TILE8, false) }
}
template <typename TG>
static KernelFn pick_apply_flat_p(int p, bool vec) {
    switch (p) {
        case CAME_DT_F32: return vec ? k_apply_flat<TG, float, true> : k_apply_flat<TG, float, false>;
        case CAME_DT_F16: return vec ? k_apply_flat<TG, __half, true> : k_apply_flat<TG, __half, false>;
        default: return vec ? k_apply_flat<TG, __nv_bfloat16, true> : k_apply_flat<TG, __nv_bfloat16, false>;
    }
}
static KernelFn pick_apply_flat(int g, int p, bool vec) {
    switch (g) {
        case CAME_DT_F32: return pick_apply_flat_p<float>(p, vec);
        case CAME_DT_F16: return pick_apply_flat_p<__half>(p, vec);
        default: return pick_apply_flat_p<__nv_bfloat16>(p, vec);
    }
}

cudaError_t launch_factored(int kernel, const KernelKey& key, const StepArgs& a, const Work* work, int n,
                            cudaStream_t st) {
    switch (kernel) {
        case KID_SQ_PARTIALS: return go(pick_sq_partials(key.g_dtype, (key.variant >= 1)), a, work, n, st);
        case KID_SQ_FINALIZE: return go(k_vec_finalize<false>, a, work, n, st);
        case KID_SUMSQ: return go(pick_sumsq(key.g_dtype, (key.variant >= 1)), a, work, n, st);
        case KID_S_FINALIZE: return go(k_s_finalize, a, work, n, st);
        case KID_MOMENT:
            if (key.variant == 2 && key.mode == CAME_MODE_FP32) return launch_fp32_wide(kernel, key, a, work, n, st);
            if (key.variant == 2) return launch_fast_tile8(kernel, key, a, work, n, st);
            return go(pick_moment(key.g_dtype, key.mode, (key.variant >= 1)), a, work, n, st);
        case KID_RES_FINALIZE: return go(k_vec_finalize<true>, a, work, n, st);
        case KID_APPLY:
            if (key.variant == 2 && key.mode == CAME_MODE_FP32) return launch_fp32_wide(kernel, key, a, work, n, st);
            if (key.variant == 2) return launch_fast_tile8(kernel, key, a, work, n, st);
            return go(pick_apply(key.p_dtype, key.mode, (key.variant >= 1)), a, work, n, st);
        case KID_FACTORS: return go(k_factors, a, work, n, st);
        case KID_APPLY_FLAT:
            if (key.variant == 2) return launch_fast_tile8(kernel, key, a, work, n, st);
            return go(pick_apply_flat(key.g_dtype, key.p_dtype, (key.variant >= 1)), a, work, n, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace came
