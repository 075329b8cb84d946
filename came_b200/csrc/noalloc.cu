// came_b200_step_vector_noalloc: one CAME step on a single 1-D (non-factored) tensor for callers that are
// not allowed to allocate device memory.
//
// Who that is: a host runtime that handed the whole device to its own arena at start-up (so cudaMalloc has
// nothing left to give, or would stall the device while the driver maps memory), and code running where an
// allocation is simply not permitted, e.g. a step function invoked between the stages of someone else's
// pre-planned memory schedule.  Those callers can hand over their tensors but cannot produce the workspace
// that came_b200_plan_create asks for.
//
// The per-block partial sums (and their total) that the kernels of the 1-D step pass to each other therefore live in a
// file-scope device array of fixed size.  Consequences, all of them part of the contract:
//   * the tensor may have at most CAME_B200_NOALLOC_MAX_ELEMS elements;
//   * every GPU that loads the library carries the array (64 KiB + one line) until the process exits;
//   * all calls on a device share it: two calls whose kernels overlap on the GPU (different streams) race;
//     calls on one stream are ordered and safe.  Nothing in it has to start at zero: a call first overwrites
//     every entry it later reads, whatever the previous call left there;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//     device current); make that first call outside any stream capture.
// The function calls no cudaMalloc / cudaFree and no allocating library routine.
#include <mutex>

#include "common.cuh"
#include "came_b200.h"

namespace came {

void set_last_error(const char* msg);   // capi.cu

constexpr int NOALLOC_MAX_BLOCKS = CAME_B200_NOALLOC_MAX_ELEMS / QBLOCK;   // 16384 partial sums = 64 KiB

// In host code this name is only a handle for cudaGetSymbolAddress, not a device address.
// 16384 block sums, then (one 256-byte line further) their total
static __device__ __align__(256) float g_noalloc_partials[NOALLOC_MAX_BLOCKS + 64];

struct NoallocArgs {
    void* p;
    const void* g;
    void* m;
    float* m_absmax;
    void* v;
    float* v_absmax;
    int64_t n;
    int quant;          // 1: int8 / uint8 codes with absmax per 256, 0: fp32 states
    int p_dtype, g_dtype;
    uint32_t flags;
    CameHyper h;
    float* partials;    // device address of g_noalloc_partials
};

__device__ __forceinline__ float load_any(const void* base, int dtype, int64_t i) {
    if (dtype == CAME_DT_F32) return reinterpret_cast<const float*>(base)[i];
    if (dtype == CAME_DT_F16) return __half2float(reinterpret_cast<const __half*>(base)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
}
__device__ __forceinline__ float round_any(float x, int dtype) {
    if (dtype == CAME_DT_F32) return x;
    if (dtype == CAME_DT_F16) return __half2float(__float2half_rn(x));
    return __bfloat162float(__float2bfloat16_rn(x));
}
__device__ __forceinline__ void store_any(void* base, int dtype, int64_t i, float x) {
    if (dtype == CAME_DT_F32) reinterpret_cast<float*>(base)[i] = x;
    else if (dtype == CAME_DT_F16) reinterpret_cast<__half*>(base)[i] = __float2half_rn(x);
    else reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(x);
}

// v = beta2 v + (1-beta2)(g^2 + eps0), u = g / sqrt(v)   (came_kernels.cu:1035-1042)
__device__ __forceinline__ void noalloc_second_moment(const NoallocArgs& a, int b, int64_t idx, bool valid, float& g,
                                                      float& v, float& u) {
    g = 0.0f; v = 0.0f; u = 0.0f;
    if (!valid) return;
    g = load_any(a.g, a.g_dtype, idx) * a.h.grad_scale;
    const float old = a.quant ? (float)reinterpret_cast<const uint8_t*>(a.v)[idx] * (a.v_absmax[b] / QMAX_U8)
                              : reinterpret_cast<const float*>(a.v)[idx];
    v = old * a.h.beta2 + a.h.om_beta2 * fmaf(g, g, a.h.eps0);
    const float vv = (a.flags & CAME_F_RSQRT_CLAMP) ? fmaxf(v, 1e-30f) : v;
    u = (1.0f / sqrtf(vv)) * g;
}

__global__ void __launch_bounds__(THREADS) k_noalloc_partial(NoallocArgs a) {
    __shared__ float red[33];
    const int b = blockIdx.x;
    const int64_t idx = (int64_t)b * QBLOCK + threadIdx.x;
    float g, v, u;
    noalloc_second_moment(a, b, idx, idx < a.n, g, v, u);
    const float t = block_sum(u * u, red);
    if (threadIdx.x == 0) a.partials[b] = t;      // every entry the second kernel reads is written here first
}

// S = sum of the block sums, by one CTA in the fixed order the workspace path uses; kept behind the partials
__global__ void __launch_bounds__(THREADS) k_noalloc_reduce(NoallocArgs a, int nblocks) {
    __shared__ float red[33];
    const float S = block_vector_sum(a.partials, nblocks, red);
    if (threadIdx.x == 0) a.partials[NOALLOC_MAX_BLOCKS] = S;
}

__global__ void __launch_bounds__(THREADS) k_noalloc_apply(NoallocArgs a, int nblocks) {
    __shared__ float red[33];
    const int b = blockIdx.x;
    const int64_t idx = (int64_t)b * QBLOCK + threadIdx.x;
    const bool valid = idx < a.n;
    const float S = a.partials[NOALLOC_MAX_BLOCKS];
    const float clip = fmaxf(1.0f, sqrtf(S / (float)a.n) / a.h.clip_threshold);
    float g, v, u;
    noalloc_second_moment(a, b, idx, valid, g, v, u);
    if (a.flags & CAME_F_UPDATE_F16) u = __half2float(__float2half_rn(u));
    u = u / clip;
    float m_old = 0.0f;
    if (valid)
        m_old = a.quant ? (float)reinterpret_cast<const int8_t*>(a.m)[idx] * (a.m_absmax[b] / QMAX_I8)
                        : reinterpret_cast<const float*>(a.m)[idx];
    const float m = m_old * a.h.beta1 + a.h.om_beta1 * u;
    if (valid) {
        float pv = load_any(a.p, a.p_dtype, idx);
        if (a.h.weight_decay != 0.0f) {
            if (a.flags & CAME_F_WD_MUL2) pv = round_any(pv * a.h.decay_mul, a.p_dtype);
            else if (a.flags & CAME_F_WD_ADD2) pv = round_any(pv - a.h.wd_lr * pv, a.p_dtype);
            else pv = pv - a.h.wd_lr * pv;
        }
        store_any(a.p, a.p_dtype, idx, pv - a.h.lr * m);
    }
    if (a.quant) {
        const float vmax = fix_absmax(block_max(valid ? v : 0.0f, red));
        const float mmax = fix_absmax(block_max(valid ? fabsf(m) : 0.0f, red));
        if (threadIdx.x == 0) { a.v_absmax[b] = vmax; a.m_absmax[b] = mmax; }
        if (valid) {
            reinterpret_cast<uint8_t*>(a.v)[idx] = (uint8_t)quant_u8_div(v, vmax);
            reinterpret_cast<int8_t*>(a.m)[idx] = (int8_t)quant_i8_div(m, mmax);
        }
    } else if (valid) {
        reinterpret_cast<float*>(a.v)[idx] = v;
        reinterpret_cast<float*>(a.m)[idx] = m;
    }
}

// device address of the static array, looked up once per device
constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_partials_addr[NOALLOC_MAX_DEVICES] = {};
static std::mutex g_noalloc_mutex;

static cudaError_t noalloc_partials_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_partials_addr[dev]) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_partials);   // for the CURRENT device
        if (e != cudaSuccess) return e;
        g_partials_addr[dev] = ptr;
    }
    *out = g_partials_addr[dev];
    return cudaSuccess;
}

}  // namespace came

extern "C" int came_b200_step_vector_noalloc(void* p, const void* g, void* m, float* m_absmax, void* v, float* v_absmax,
                                             int64_t n, int mode, int p_dtype, int g_dtype, uint32_t flags,
                                             const CameHyper* hyper, came_stream_t stream) {
    using namespace came;
    auto fail = [](int code, const char* msg) { set_last_error(msg); return code; };
    if (!p || !g || !m || !v || !hyper) return fail(CAME_E_INVALID, "step_vector_noalloc: p, g, m, v and hyper must be non-null");
    if (mode != CAME_MODE_FP32 && mode != CAME_MODE_FLAT8)
        return fail(CAME_E_INVALID, "step_vector_noalloc: mode must be CAME_MODE_FP32 or CAME_MODE_FLAT8");
    if (mode == CAME_MODE_FLAT8 && (!m_absmax || !v_absmax))
        return fail(CAME_E_INVALID, "step_vector_noalloc: 8-bit states need m_absmax and v_absmax");
    if (p_dtype < CAME_DT_F32 || p_dtype > CAME_DT_BF16 || g_dtype < CAME_DT_F32 || g_dtype > CAME_DT_BF16)
        return fail(CAME_E_INVALID, "step_vector_noalloc: bad dtype");
    if (n <= 0 || !(hyper->clip_threshold > 0.0f)) return fail(CAME_E_INVALID, "step_vector_noalloc: n and clip_threshold must be > 0");
    if (n > CAME_B200_NOALLOC_MAX_ELEMS)      // the static scratch holds 16384 block sums
        return fail(CAME_E_UNSUPPORTED, "step_vector_noalloc: more than CAME_B200_NOALLOC_MAX_ELEMS (4194304) elements; "
                                        "use came_b200_step with a caller-provided workspace");
    NoallocArgs a{};
    a.p = p; a.g = g; a.m = m; a.m_absmax = m_absmax; a.v = v; a.v_absmax = v_absmax;
    a.n = n; a.quant = mode == CAME_MODE_FLAT8; a.p_dtype = p_dtype; a.g_dtype = g_dtype; a.flags = flags; a.h = *hyper;
    if (a.h.grad_scale == 0.0f) a.h.grad_scale = 1.0f;      // a zero-initialised record means "no scaling"
    if (noalloc_partials_address(&a.partials) != cudaSuccess)
        return fail(CAME_E_CUDA, "step_vector_noalloc: cudaGetSymbolAddress failed");
    const int nblocks = (int)((n + QBLOCK - 1) / QBLOCK);
    cudaStream_t st = (cudaStream_t)stream;
    k_noalloc_partial<<<nblocks, THREADS, 0, st>>>(a);
    k_noalloc_reduce<<<1, THREADS, 0, st>>>(a, nblocks);
    k_noalloc_apply<<<nblocks, THREADS, 0, st>>>(a, nblocks);
    return cudaGetLastError() == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "step_vector_noalloc: kernel launch failed");
}
