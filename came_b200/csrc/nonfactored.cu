// CAME step for 1-D (non-factored) tensors: two multi-tensor launches over blocks of 256 elements.
//
//   nf_partial : g, v        -> per-block partial of sum u^2,  u = g * rsqrt(v_new)
//   nf_reduce  : partials    -> S = sum u^2 of a tensor (one CTA per tensor, fixed order)
//   nf_apply   : g, v, m, p  -> v, m, p   (v_new and u are recomputed; no scratch tensor carries u)
//
// Reference: kCameNonfactoredSqUpdateAndQuant[TypedUpdate] came_kernels.cu:1013-1122 and
// kCameNonfactoredExpAvgParamUpdate[TypedUpdate] came_kernels.cu:1489-1601 (8-bit states);
// CAMECUDA._step_param_nonfactored_cuda CAMECUDA.py:247-273 (fp32 states).  There is no confidence
// term on 1-D tensors (CAME.py:163-164).
#include "common.cuh"
#include "launch.h"

namespace came {

template <typename TG>
__device__ __forceinline__ void nf_second_moment(const CameTensorDesc& d, const CameHyper& h, int b, int64_t idx,
                                                 bool valid, float& g, float& v, float& u) {
    g = 0.0f; v = 0.0f; u = 0.0f;
    if (!valid) return;
    g = to_f32(reinterpret_cast<const TG*>(d.g)[idx]) * h.grad_scale;
    float old;
    if (d.mode == CAME_MODE_FP32) {
        old = reinterpret_cast<const float*>(d.sq_row)[idx];
    } else {
        old = (float)reinterpret_cast<const uint8_t*>(d.sq_row)[idx] * (d.sq_row_absmax[b] / QMAX_U8);
    }
    v = old * h.beta2 + h.om_beta2 * fmaf(g, g, h.eps0);
    const float vv = (d.flags & CAME_F_RSQRT_CLAMP) ? fmaxf(v, 1e-30f) : v;
    u = (1.0f / sqrtf(vv)) * g;
}

template <typename TG>
__global__ void __launch_bounds__(THREADS) k_nf_partial(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const int64_t idx = (int64_t)w.tile * QBLOCK + threadIdx.x;
    float g, v, u;
    nf_second_moment<TG>(d, h, w.tile, idx, idx < d.rows, g, v, u);
    const float t = block_sum(u * u, red);
    if (threadIdx.x == 0) s.spart[w.tile] = t;
}

// S of one tensor, left behind its block partials: the apply CTAs read one float instead of summing all partials each
__global__ void __launch_bounds__(THREADS) k_nf_reduce(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    const Scratch& s = a.scr[work[blockIdx.x].tensor];
    const float S = block_vector_sum(s.spart, s.nbR, red);
    if (threadIdx.x == 0) s.spart[s.nbR] = S;
}

template <typename TG, typename TP>
__global__ void __launch_bounds__(THREADS) k_nf_apply(StepArgs a, const Work* __restrict__ work) {
    __shared__ float red[33];
    const Work w = work[blockIdx.x];
    const CameTensorDesc& d = a.descs[w.tensor];
    const Scratch& s = a.scr[w.tensor];
    const CameHyper& h = a.hyp[d.group];
    const int b = w.tile;
    const int64_t idx = (int64_t)b * QBLOCK + threadIdx.x;
    const bool valid = idx < d.rows;
    const bool quant = d.mode != CAME_MODE_FP32;

    const float S = s.spart[s.nbR];
    const float clip = fmaxf(1.0f, sqrtf(S / (float)d.rows) / h.clip_threshold);

    float g, v, u;
    nf_second_moment<TG>(d, h, b, idx, valid, g, v, u);
    if (d.flags & CAME_F_UPDATE_F16) u = __half2float(__float2half_rn(u));
    u = u / clip;

    float m_old = 0.0f;
    if (valid) {
        m_old = quant ? (float)reinterpret_cast<const int8_t*>(d.m)[idx] * (d.m_absmax[b] / QMAX_I8)
                      : reinterpret_cast<const float*>(d.m)[idx];
    }
    const float m = m_old * h.beta1 + h.om_beta1 * u;

    if (valid) {
        TP* p = reinterpret_cast<TP*>(d.p);
        p[idx] = from_f32<TP>(apply_one<TP>(to_f32(p[idx]), m, h, d.flags));
    }
    if (quant) {
        const float vmax = fix_absmax(block_max(valid ? v : 0.0f, red));
        const float mmax = fix_absmax(block_max(valid ? fabsf(m) : 0.0f, red));
        if (threadIdx.x == 0) {
            d.sq_row_absmax[b] = vmax;
            d.m_absmax[b] = mmax;
        }
        if (valid) {
            reinterpret_cast<uint8_t*>(d.sq_row)[idx] = (uint8_t)quant_u8_div(v, vmax);
            reinterpret_cast<int8_t*>(d.m)[idx] = (int8_t)quant_i8_div(m, mmax);
        }
    } else if (valid) {
        reinterpret_cast<float*>(d.sq_row)[idx] = v;
        reinterpret_cast<float*>(d.m)[idx] = m;
    }
}

using KernelFn = void (*)(StepArgs, const Work*);

template <typename TG>
static KernelFn pick_apply_p(int p) {
    switch (p) {
        case CAME_DT_F32: return k_nf_apply<TG, float>;
        case CAME_DT_F16: return k_nf_apply<TG, __half>;
        default: return k_nf_apply<TG, __nv_bfloat16>;
    }
}

cudaError_t launch_nonfactored(int kernel, const KernelKey& key, const StepArgs& a, const Work* work, int n,
                               cudaStream_t st) {
    if (n <= 0) return cudaSuccess;
    KernelFn fn = nullptr;
    if (kernel == KID_NF_PARTIAL) {
        fn = key.g_dtype == CAME_DT_F32 ? k_nf_partial<float>
             : key.g_dtype == CAME_DT_F16 ? k_nf_partial<__half> : k_nf_partial<__nv_bfloat16>;
    } else if (kernel == KID_NF_REDUCE) {
        fn = k_nf_reduce;
    } else if (kernel == KID_NF_APPLY) {
        fn = key.g_dtype == CAME_DT_F32 ? pick_apply_p<float>(key.p_dtype)
             : key.g_dtype == CAME_DT_F16 ? pick_apply_p<__half>(key.p_dtype) : pick_apply_p<__nv_bfloat16>(key.p_dtype);
    } else {
        return cudaErrorInvalidValue;
    }
    fn<<<n, THREADS, 0, st>>>(a, work);
    return cudaGetLastError();
}

}  // namespace came
