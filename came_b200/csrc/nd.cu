// CAME step for tensors of more than two dimensions: a batch of B contiguous [R, C] matrices (B = product of the
// leading dimensions) that share ONE RMS clip over the whole tensor, with row / column state vectors of B*R / B*C
// entries that are quantised in blocks of 256 over their flattened entries (a block may straddle matrices) and a
// momentum quantised in blocks of 256 flat elements.  This is what the reference's classes compute for such tensors on
// their generic paths (came_pytorch/CAME.py:117-172, CAMECUDA.py:275-326, CAME8bitFull.py:1006-1075: reductions over
// dim -1 / -2, `_rms` over the whole update, `quantize_blockwise` over the flattened state); its batched CUDA variants
// (came_kernels.cu:5707-6184, global RMS at :5880-5884) follow the same algebra.
//
// Such tensors are convolution kernels and stacked small matrices (thousands of 3 x 3 matrices, say), a negligible
// share of a model's elements: the kernels below favour simplicity over bandwidth.  One thread owns one entry of a
// state vector and walks its row (column); the element-wise passes own one flat block of 256 elements per CTA.
// Every reduction has a fixed order (bit-reproducible).  Launch sequence per step, each over all N-D tensors:
//
//   nd_sq     g              -> fresh v_row / v_col (EMA with the dequantised old state), requantised states
//   nd_mean   v_row          -> mean of v_row per matrix (guarded)
//   nd_sumsq  g              -> block partials of S = sum (g r c)^2
//   nd_s      partials       -> S, clip
//   nd_res    g, m           -> fresh residual row / column vectors, requantised states
//   nd_mean   Rr             -> mean per matrix
//   nd_apply  g, m, p        -> m (requantised per flat block), p
#include "common.cuh"
#include "launch.h"

namespace came {

namespace {

__device__ __forceinline__ float nd_load(const void* base, int dtype, int64_t i) {
    if (dtype == CAME_DT_F32) return reinterpret_cast<const float*>(base)[i];
    if (dtype == CAME_DT_F16) return __half2float(reinterpret_cast<const __half*>(base)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
}
__device__ __forceinline__ float nd_round(float x, int dtype) {
    if (dtype == CAME_DT_F32) return x;
    if (dtype == CAME_DT_F16) return __half2float(__float2half_rn(x));
    return __bfloat162float(__float2bfloat16_rn(x));
}
__device__ __forceinline__ void nd_store(void* base, int dtype, int64_t i, float x) {
    if (dtype == CAME_DT_F32) reinterpret_cast<float*>(base)[i] = x;
    else if (dtype == CAME_DT_F16) reinterpret_cast<__half*>(base)[i] = __float2half_rn(x);
    else reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(x);
}

struct NdShape {
    int64_t B, R, C, NR, NC, n;
};
__device__ __forceinline__ NdShape nd_shape(const CameTensorDesc& d) {
    NdShape s;
    s.B = d.batch; s.R = d.rows; s.C = d.cols;
    s.NR = s.B * s.R; s.NC = s.B * s.C; s.n = s.NR * s.C;
    return s;
}

// old value of entry e of a state vector (fp32 or uint8 with one absmax per 256 flat entries)
__device__ __forceinline__ float nd_old_vec(const void* state, const float* absmax, bool quant, int64_t e) {
    return quant ? (float)reinterpret_cast<const uint8_t*>(state)[e] * (absmax[e >> 8] / QMAX_U8)
                 : reinterpret_cast<const float*>(state)[e];
}

// fresh copy, requantisation of one block of 256 entries of a state vector (all 256 threads call)
__device__ __forceinline__ void nd_store_vec(void* state, float* absmax, float* fresh, bool quant, int64_t e, int blk, bool valid,
                                             float v, float* red) {
    if (valid) fresh[e] = v;
    if (quant) {
        const float bmax = fix_absmax(block_max(valid ? v : 0.0f, red));      // syncs: every old absmax read is done
        if (threadIdx.x == 0) absmax[blk] = bmax;
        if (valid) reinterpret_cast<uint8_t*>(state)[e] = (uint8_t)quant_u8_div(v, bmax);
    } else if (valid) {
        reinterpret_cast<float*>(state)[e] = v;
    }
}

// u0 = (g r_i) c_j and, from it, the new momentum value of element (b, i, j) at flat index f
struct NdElem {
    float u, m;
};
__device__ __forceinline__ float nd_u0(const CameTensorDesc& d, const Scratch& s, const NdShape& sh, int64_t b, int64_t i, int64_t j,
                                       int64_t f, float gscale) {
    const bool clamp = d.flags & CAME_F_SQ_CLAMP;
    const float r = row_factor(s.vr[b * sh.R + i], s.rowblk[b], clamp);
    const float c = col_factor(s.vc[b * sh.C + j], clamp);
    return ((nd_load(d.g, d.g_dtype, f) * gscale) * r) * c;
}
__device__ __forceinline__ NdElem nd_moment(const CameTensorDesc& d, const Scratch& s, const CameHyper& h, const NdShape& sh,
                                            int64_t b, int64_t i, int64_t j, int64_t f, float inv_clip) {
    NdElem o;
    o.u = nd_u0(d, s, sh, b, i, j, f, h.grad_scale) * inv_clip;
    const float m_old = d.mode == CAME_MODE_FP32 ? reinterpret_cast<const float*>(d.m)[f]
                                                 : (float)reinterpret_cast<const int8_t*>(d.m)[f] * (d.m_absmax[f >> 8] / QMAX_I8);
    o.m = m_old * h.beta1 + h.om_beta1 * o.u;
    return o;
}

}  // namespace

// RES = false: second moment of g (beta2, eps0); RES = true: residual (beta3, eps1).  Work item: one block of 256
// entries, the row vector's blocks first.
template <bool RES>
__global__ void __launch_bounds__(THREADS) k_nd_vec(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const NdShape sh = nd_shape(d);
    const int nbr = (int)((sh.NR + QBLOCK - 1) / QBLOCK);
    const bool is_col = w.tile >= nbr;
    const int blk = is_col ? w.tile - nbr : w.tile;
    const int64_t e = (int64_t)blk * QBLOCK + threadIdx.x;
    const bool valid = e < (is_col ? sh.NC : sh.NR);
    const bool quant = d.mode != CAME_MODE_FP32;
    const float inv_clip = RES ? 1.0f / s.scal[1] : 1.0f;
    const float eps = RES ? h.eps1 : h.eps0;
    float v = 0.0f;
    if (valid) {
        const int64_t len = is_col ? sh.R : sh.C;                  // entries the mean runs over
        const int64_t b = e / (is_col ? sh.C : sh.R), k = e - b * (is_col ? sh.C : sh.R);
        float acc = 0.0f;
        for (int64_t t = 0; t < len; ++t) {
            const int64_t i = is_col ? t : k, j = is_col ? k : t;
            const int64_t f = (b * sh.R + i) * sh.C + j;
            float x;
            if (RES) {
                const NdElem o = nd_moment(d, s, h, sh, b, i, j, f, inv_clip);
                const float df = o.u - o.m;
                x = fmaf(df, df, eps);
            } else {
                const float g = nd_load(d.g, d.g_dtype, f) * h.grad_scale;
                x = fmaf(g, g, eps);
            }
            acc += x;
        }
        const float mean = acc / (float)len;
        const void* state = RES ? (is_col ? d.res_col : d.res_row) : (is_col ? d.sq_col : d.sq_row);
        const float* absmax = RES ? (is_col ? d.res_col_absmax : d.res_row_absmax) : (is_col ? d.sq_col_absmax : d.sq_row_absmax);
        v = ema_update(nd_old_vec(state, absmax, quant, e), RES ? h.beta3 : h.beta2, RES ? h.om_beta3 : h.om_beta2, mean);
    }
    void* state = RES ? (is_col ? d.res_col : d.res_row) : (is_col ? d.sq_col : d.sq_row);
    float* absmax = RES ? (is_col ? d.res_col_absmax : d.res_row_absmax) : (is_col ? d.sq_col_absmax : d.sq_row_absmax);
    float* fresh = RES ? (is_col ? s.Rc : s.Rr) : (is_col ? s.vc : s.vr);
    nd_store_vec(state, absmax, fresh, quant, e, blk, valid, v, red);
}

// guarded mean of the fresh row vector of one matrix (work item: matrix index)
template <bool RES>
__global__ void __launch_bounds__(THREADS) k_nd_mean(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const int R = (int)d.rows;
    const float* v = (RES ? s.Rr : s.vr) + (int64_t)w.tile * R;
    float mean = block_vector_sum(v, R, red) / (float)R;
    mean = RES ? guard_mean(mean, d.flags & CAME_F_RESROW_FIX, d.flags & CAME_F_RESROW_CLAMP)
               : guard_mean(mean, d.flags & CAME_F_SQ_FIX, d.flags & CAME_F_SQ_CLAMP);
    if (threadIdx.x == 0) (RES ? s.rowblk2 : s.rowblk)[w.tile] = mean;
}

// block partials of S = sum (g r c)^2 (work item: flat block of 256 elements)
__global__ void __launch_bounds__(THREADS) k_nd_sumsq(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const NdShape sh = nd_shape(d);
    const int64_t f = (int64_t)w.tile * QBLOCK + threadIdx.x;
    float u = 0.0f;
    if (f < sh.n) {
        const int64_t b = f / (sh.R * sh.C), rem = f - b * sh.R * sh.C, i = rem / sh.C, j = rem - i * sh.C;
        u = nd_u0(d, s, sh, b, i, j, f, a.hyp[d.group].grad_scale);
    }
    const float t = block_sum(u * u, red);
    if (threadIdx.x == 0) s.spart[w.tile] = t;
}

// S and the clip divisor of one tensor (clip = max(1, sqrt(S/n)/clip_threshold), came_kernels.cu:2619-2620)
__global__ void __launch_bounds__(THREADS) k_nd_s(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const NdShape sh = nd_shape(d);
    const int nbe = (int)((sh.n + QBLOCK - 1) / QBLOCK);
    const float S = block_vector_sum(s.spart, nbe, red);
    if (threadIdx.x == 0) {
        s.scal[0] = S;
        s.scal[1] = fmaxf(1.0f, sqrtf(S / (float)sh.n) / a.hyp[d.group].clip_threshold);
    }
}

// momentum (requantised per flat block of 256) and parameter update (work item: flat block)
__global__ void __launch_bounds__(THREADS) k_nd_apply(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const NdShape sh = nd_shape(d);
    const int64_t f = (int64_t)w.tile * QBLOCK + threadIdx.x;
    const bool valid = f < sh.n;
    float m = 0.0f;
    if (valid) {
        const int64_t b = f / (sh.R * sh.C), rem = f - b * sh.R * sh.C, i = rem / sh.C, j = rem - i * sh.C;
        m = nd_moment(d, s, h, sh, b, i, j, f, 1.0f / s.scal[1]).m;
        const float rr = row_factor(s.Rr[b * sh.R + i], s.rowblk2[b], d.flags & CAME_F_RESROW_CLAMP);
        const float rc = col_factor(s.Rc[b * sh.C + j], d.flags & CAME_F_RESCOL_CLAMP);
        const float upd = (m * rr) * rc;
        float pv = nd_load(d.p, d.p_dtype, f);
        if (h.weight_decay != 0.0f) {
            if (d.flags & CAME_F_WD_MUL2) pv = nd_round(pv * h.decay_mul, d.p_dtype);
            else if (d.flags & CAME_F_WD_ADD2) pv = nd_round(pv - h.wd_lr * pv, d.p_dtype);
            else pv = pv - h.wd_lr * pv;
        }
        nd_store(d.p, d.p_dtype, f, pv - h.lr * upd);
    }
    if (d.mode == CAME_MODE_FP32) {
        if (valid) reinterpret_cast<float*>(d.m)[f] = m;
    } else {
        const float bmax = fix_absmax(block_max(valid ? fabsf(m) : 0.0f, red));   // syncs: every old absmax read is done
        if (threadIdx.x == 0) d.m_absmax[w.tile] = bmax;
        if (valid) reinterpret_cast<int8_t*>(d.m)[f] = (int8_t)quant_i8_div(m, bmax);
    }
}

cudaError_t launch_nd(int kernel, const StepArgs& a, const Work* work, int n, cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    switch (kernel) {
        case KID_ND_SQ: k_nd_vec<false><<<n, THREADS, 0, st>>>(a, work); break;
        case KID_ND_MEAN: k_nd_mean<false><<<n, THREADS, 0, st>>>(a, work); break;
        case KID_ND_SUMSQ: k_nd_sumsq<<<n, THREADS, 0, st>>>(a, work); break;
        case KID_ND_S: k_nd_s<<<n, THREADS, 0, st>>>(a, work); break;
        case KID_ND_RES: k_nd_vec<true><<<n, THREADS, 0, st>>>(a, work); break;
        case KID_ND_RESMEAN: k_nd_mean<true><<<n, THREADS, 0, st>>>(a, work); break;
        case KID_ND_APPLY: k_nd_apply<<<n, THREADS, 0, st>>>(a, work); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace came
