// Shared device helpers of the CAME step kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "came_b200.h"

namespace came {

constexpr int QBLOCK = 256;   // elements per absmax of the flat codec (blockwise_quantization.py)
constexpr int TILE = 16;      // edge of an exp_avg tile in CAME_MODE_TILE8 (came_kernels.cu:19)
constexpr float QMAX_I8 = 127.0f;
constexpr float QMAX_U8 = 255.0f;

// reduction tile of the gradient passes (rows x cols handled by one CTA)
constexpr int K_TR = 128;
constexpr int K_TC = 512;
// tile of the momentum / apply passes
constexpr int P_TR = 128;
constexpr int P_TC = 256;
constexpr int THREADS = 256;
// tile of the shared-memory staged (tile-layout) momentum / apply passes
constexpr int W_TR = 128;
constexpr int W_TC = 1024;
constexpr int W_THREADS = 512;
// flat blocks (of 256 elements) handled by one CTA of the flat-layout apply pass
constexpr int FLAT_BLOCKS_PER_CTA = 64;

// Per-tensor scratch, laid out in the caller's workspace by the plan.  All pointers are device
// pointers to fp32.
struct Scratch {
    float* vr;        // [rows]  fresh second-moment row vector (fp32, before requantisation)
    float* vc;        // [cols]
    float* Rr;        // [rows]  fresh residual row vector
    float* Rc;        // [cols]
    float* rowblk;    // [nbR]   sum of vr over each block of 256 rows
    float* rowblk2;   // [nbR]   same for Rr
    float* scal;      // [4]     {S = sum (g r c)^2, clip, -, -}
    float* rowpart;   // [max(tiles_c, ptiles_c) * rows]  per-CTA row partial sums
    float* colpart;   // [tiles_r * cols]                 per-CTA column partial sums
    float* spart;     // [tiles_r * tiles_c] partials of S; 1-D tensors: [nbR] block partials of sum u^2
    float* fac;       // flat layout only: r[rows], c[cols], R'[rows], C'[cols] factors, else nullptr
    float* tpart;     // fused first pass only: [tiles_r * cols] per-strip column sums of g^2 / v_row
    int32_t tiles_r, tiles_c;     // K_TR x K_TC grid
    int32_t ptiles_r, ptiles_c;   // P_TR x P_TC grid (W_TR x W_TC when the staged fast path runs)
    int32_t nbR, nbC;             // ceil(rows/256), ceil(cols/256)
    int32_t fused_a;              // 1: the fused first pass runs (complete row sums, v_row and tpart come from it)
    int32_t fa_rb;                // fused first pass: rows per staged batch
    float* mfac;                  // staged momentum pass: row factors r_i / clip [R]
    float* mfac_c;                // staged passes: column factors [C], 16-byte aligned (c_j; after the residual finalize C'_j)
    float* mfac_c2;               // flat layout on the staged path: C'_j (c_j stays in mfac_c for the apply items), else nullptr
    int32_t sq_col_parts;         // column partial sets the first pass leaves (strips, or strips x 2 warp groups)
    int32_t res_eps_deferred;     // 1: the residual partials hold sums of (u-m)^2 only; eps1 is added per row / column
                                  //    by the finalize kernel (cols * eps1, rows * eps1)
};

struct Work {
    int32_t tensor;
    int32_t tile;
};

// ------------------------------------------------------------------------------------------
// element conversion
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// round to T and back (the value a T-typed parameter holds after a store)
template <typename T> __device__ __forceinline__ float round_to(float x) { return to_f32(from_f32<T>(x)); }

// ------------------------------------------------------------------------------------------
// N contiguous elements -> fp32 registers.  VEC: 16-byte loads (caller guarantees alignment and
// that all N elements are in range).  !VEC: scalar loads, elements at col+e >= ncols read as 0.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack_bf16x8(const uint4& r, float* v) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void unpack_f16x8(const uint4& r, float* v) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

template <int N, bool VEC>
__device__ __forceinline__ void load_run(const float* p, int64_t off, int col, int ncols, float* v) {
    if (VEC) {
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            const float4 f = reinterpret_cast<const float4*>(p + off)[i];
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    } else {
#pragma unroll
        for (int e = 0; e < N; ++e) v[e] = (col + e < ncols) ? p[off + e] : 0.0f;
    }
}
template <int N, bool VEC>
__device__ __forceinline__ void load_run(const __nv_bfloat16* p, int64_t off, int col, int ncols, float* v) {
    if (VEC) {
#pragma unroll
        for (int i = 0; i < N / 8; ++i) {
            const uint4 r = reinterpret_cast<const uint4*>(p + off)[i];
            unpack_bf16x8(r, v + 8 * i);
        }
    } else {
#pragma unroll
        for (int e = 0; e < N; ++e) v[e] = (col + e < ncols) ? __bfloat162float(p[off + e]) : 0.0f;
    }
}
template <int N, bool VEC>
__device__ __forceinline__ void load_run(const __half* p, int64_t off, int col, int ncols, float* v) {
    if (VEC) {
#pragma unroll
        for (int i = 0; i < N / 8; ++i) {
            const uint4 r = reinterpret_cast<const uint4*>(p + off)[i];
            unpack_f16x8(r, v + 8 * i);
        }
    } else {
#pragma unroll
        for (int e = 0; e < N; ++e) v[e] = (col + e < ncols) ? __half2float(p[off + e]) : 0.0f;
    }
}

// N contiguous int8 codes -> fp32 (N = 8 or 16)
template <int N, bool VEC>
__device__ __forceinline__ void load_codes(const int8_t* p, int64_t off, int col, int ncols, float* v) {
    if (VEC) {
        uint32_t w[N / 4];
        if (N == 16) {
            const uint4 r = *reinterpret_cast<const uint4*>(p + off);
            w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w;
        } else {
            const uint2 r = *reinterpret_cast<const uint2*>(p + off);
            w[0] = r.x; w[1] = r.y;
        }
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
#pragma unroll
            for (int b = 0; b < 4; ++b) v[4 * i + b] = (float)(int)(int8_t)((w[i] >> (8 * b)) & 0xffu);
        }
    } else {
#pragma unroll
        for (int e = 0; e < N; ++e) v[e] = (col + e < ncols) ? (float)p[off + e] : 0.0f;
    }
}

template <int N, bool VEC>
__device__ __forceinline__ void store_codes(int8_t* p, int64_t off, int col, int ncols, const int* q) {
    if (VEC) {
        uint32_t w[N / 4];
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            w[i] = ((uint32_t)q[4 * i] & 0xffu) | (((uint32_t)q[4 * i + 1] & 0xffu) << 8) |
                   (((uint32_t)q[4 * i + 2] & 0xffu) << 16) | (((uint32_t)q[4 * i + 3] & 0xffu) << 24);
        }
        if (N == 16) {
            *reinterpret_cast<uint4*>(p + off) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            *reinterpret_cast<uint2*>(p + off) = make_uint2(w[0], w[1]);
        }
    } else {
#pragma unroll
        for (int e = 0; e < N; ++e)
            if (col + e < ncols) p[off + e] = (int8_t)q[e];
    }
}

template <int N, bool VEC>
__device__ __forceinline__ void store_run(float* p, int64_t off, int col, int ncols, const float* v) {
    if (VEC) {
#pragma unroll
        for (int i = 0; i < N / 4; ++i)
            reinterpret_cast<float4*>(p + off)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
        for (int e = 0; e < N; ++e)
            if (col + e < ncols) p[off + e] = v[e];
    }
}
template <int N, bool VEC>
__device__ __forceinline__ void store_run(__nv_bfloat16* p, int64_t off, int col, int ncols, const float* v) {
    if (VEC) {
#pragma unroll
        for (int i = 0; i < N / 8; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * i + 2 * k], v[8 * i + 2 * k + 1]);
                w[k] = *reinterpret_cast<const uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(p + off)[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
#pragma unroll
        for (int e = 0; e < N; ++e)
            if (col + e < ncols) p[off + e] = __float2bfloat16_rn(v[e]);
    }
}
template <int N, bool VEC>
__device__ __forceinline__ void store_run(__half* p, int64_t off, int col, int ncols, const float* v) {
    if (VEC) {
#pragma unroll
        for (int i = 0; i < N / 8; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const __half2 h = __floats2half2_rn(v[8 * i + 2 * k], v[8 * i + 2 * k + 1]);
                w[k] = *reinterpret_cast<const uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(p + off)[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
#pragma unroll
        for (int e = 0; e < N; ++e)
            if (col + e < ncols) p[off + e] = __float2half_rn(v[e]);
    }
}

// ------------------------------------------------------------------------------------------
// reductions (fixed order -> run-to-run identical results)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// all THREADS threads call; result valid in every thread.  `red` is a shared float[33].
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
        red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = red[0];
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) t = fmaxf(t, red[w]);
        red[32] = t;
    }
    __syncthreads();
    return red[32];
}
// sum of x[0..n) by the whole block
__device__ __forceinline__ float block_vector_sum(const float* x, int n, float* red) {
    float t = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) t += x[i];
    return block_sum(t, red);
}

// ------------------------------------------------------------------------------------------
// codec arithmetic.  Quantisation is rint((x / absmax) * qmax) with an IEEE quotient, as
// blockwise_quantization.py:73-80 computes it.  div_by() forms the correctly rounded quotient from
// a precomputed reciprocal with one residual correction (cheaper than a division per element).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float fix_absmax(float a) { return a > 0.0f ? a : 1.0f; }

__device__ __forceinline__ float div_by(float x, float d, float inv_d) {
    const float q0 = x * inv_d;
    const float r = fmaf(-q0, d, x);
    return fmaf(r, inv_d, q0);
}
__device__ __forceinline__ int quant_i8_div(float x, float absmax) {
    const float q = rintf((x / absmax) * QMAX_I8);
    return (int)fminf(QMAX_I8, fmaxf(-QMAX_I8, q));
}
__device__ __forceinline__ int quant_u8_div(float x, float absmax) {
    const float q = rintf((x / absmax) * QMAX_U8);
    return (int)fminf(QMAX_U8, fmaxf(0.0f, q));
}
__device__ __forceinline__ int quant_i8_fast(float x, float absmax, float inv) {
    const float q = rintf(div_by(x, absmax, inv) * QMAX_I8);
    return (int)fminf(QMAX_I8, fmaxf(-QMAX_I8, q));
}
// The reciprocal trick needs 1/absmax and the residual to stay normal; outside this range take the
// plain division (uniform per block, so no divergence inside a warp's block).
__device__ __forceinline__ bool recip_safe(float absmax) { return absmax > 1e-30f && absmax < 1e30f; }

// ------------------------------------------------------------------------------------------
// exponential moving average of a row / column statistic, with every rounding pinned (no contraction into
// fused multiply-adds): two kernels that finalize the same vector then agree bit for bit, and the value is the one
// the reference's separate multiply and add produce (came_kernels.cu:91, 546)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float ema_update(float old, float beta, float om, float x) {
    return __fadd_rn(__fmul_rn(old, beta), __fmul_rn(om, x));
}
// (sum + n * eps) / n
__device__ __forceinline__ float mean_plus_eps(float sum, float n, float eps) {
    return __fdiv_rn(__fadd_rn(sum, __fmul_rn(n, eps)), n);
}

// ------------------------------------------------------------------------------------------
// factor guards (one per reference code path, selected by CAME_F_* flags)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float guard_mean(float mean, bool fix, bool clamp) {
    if (clamp) return fmaxf(mean, 1e-30f);
    if (fix) return mean > 0.0f ? mean : 1.0f;
    return mean;
}
__device__ __forceinline__ float row_factor(float v, float mean, bool clamp) {
    float ratio = v / mean;
    if (clamp) ratio = fmaxf(ratio, 1e-30f);
    return 1.0f / sqrtf(ratio);
}
__device__ __forceinline__ float col_factor(float v, bool clamp) {
    if (clamp) v = fmaxf(v, 1e-30f);
    return 1.0f / sqrtf(v);
}

// ------------------------------------------------------------------------------------------
// weight decay + update of one parameter value, in the three forms the reference uses
// ------------------------------------------------------------------------------------------
template <typename TP>
__device__ __forceinline__ float apply_one(float pv, float upd, const CameHyper& h, uint32_t flags) {
    if (h.weight_decay != 0.0f) {
        if (flags & CAME_F_WD_MUL2) {
            pv = round_to<TP>(pv * h.decay_mul);
        } else if (flags & CAME_F_WD_ADD2) {
            pv = round_to<TP>(pv - h.wd_lr * pv);
        } else {
            pv = pv - h.wd_lr * pv;
        }
    }
    return pv - h.lr * upd;
}

}  // namespace came
