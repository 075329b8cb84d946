// Internal interface between the C-ABI layer (plan / step) and the kernel translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "came_b200.h"
#include "common.cuh"

namespace came {

struct StepArgs {
    const CameTensorDesc* descs;   // device copy of the descriptor table
    const Scratch* scr;            // device, one per tensor
    const CameHyper* hyp;          // device, one per param_group
    int* status;                   // device, one word: 0, or the STATUS_* code of a kernel that gave up a wait
    // Push mode of the weight exchange: the apply items of the fused kernel also store every updated parameter at the
    // same offset of n_push peer buffers (byte distances from the local buffer to each mapped peer buffer).
    int n_push;
    int pad;
    long long push_delta[7];
};
constexpr int MAX_PUSH_PEERS = 7;

// which template instance a work list is launched with
struct KernelKey {
    int g_dtype;
    int p_dtype;
    int mode;
    int variant;   // 0: scalar loads, any shape; 1: 16-byte vector loads; 2: shared-memory staged fast path
};

enum KernelId {
    KID_SQ_PARTIALS = 0,
    KID_SQ_FINALIZE,
    KID_SUMSQ,
    KID_S_FINALIZE,
    KID_MOMENT,
    KID_RES_FINALIZE,
    KID_APPLY,
    KID_FACTORS,
    KID_APPLY_FLAT,
    KID_NF_PARTIAL,
    KID_NF_APPLY,
    KID_NF_REDUCE,
    KID_ND_SQ,             // tensors of more than two dimensions (nd.cu)
    KID_ND_MEAN,
    KID_ND_SUMSQ,
    KID_ND_S,
    KID_ND_RES,
    KID_ND_RESMEAN,
    KID_ND_APPLY,
    KID_MOMENT_APPLY,      // momentum + residual finalize + apply of the tile layout as one kernel (fused_ma.cu)
    KID_COUNT
};

// kinds of work item of the fused momentum / apply kernel, carried in the top four bits of Work::tile
enum { MA_KIND_M = 0, MA_KIND_F = 1, MA_KIND_A = 2, MA_KIND_END = 3 };

cudaError_t launch_factored(int kernel, const KernelKey& key, const StepArgs& a, const Work* work, int n,
                            cudaStream_t st);
// fp32-state layout, staged momentum / apply passes (fp_wide.cu)
cudaError_t launch_fp32_wide(int kernel, const KernelKey& key, const StepArgs& a, const Work* work, int n,
                             cudaStream_t st);
cudaError_t launch_fast_tile8(int kernel, const KernelKey& key, const StepArgs& a, const Work* work, int n,
                              cudaStream_t st);
// work: the M and A items in taking order; fwork: the F items in tensor order; next_item: two cursors (zeroed)
cudaError_t launch_fused_ma(const KernelKey& key, const StepArgs& a, const Work* work, int n, const Work* fwork, int nf,
                            int* mcount, int* fcount, int* next_item, cudaStream_t st);
cudaError_t launch_fused_sq(const KernelKey& key, const StepArgs& a, const Work* work, int n, cudaStream_t st);
// CTAs a persistent kernel launches: the SM count of the current device minus CAME_B200_RESERVED_SMS (environment,
// read once; default 0).  Leaving a few SMs free lets small kernels of other streams (a collective's flag
// exchange, say) start while a persistent pass occupies the rest for milliseconds.
int persistent_grid_limit();
constexpr int S_FIN_CHUNK = 2048;      // factor-vector entries one CTA of the clip finalize writes
void fused_sq_geometry(int64_t cols, int elem_bytes, int* groups, int* ng, int* rb, int* slot_kb);
bool fused_sq_eligible(int64_t cols, int elem_bytes);
cudaError_t launch_nonfactored(int kernel, const KernelKey& key, const StepArgs& a, const Work* work, int n,
                               cudaStream_t st);

cudaError_t launch_nd(int kernel, const StepArgs& a, const Work* work, int n, cudaStream_t st);
cudaError_t launch_selftest_bounded_wait(int* status, int* observed, cudaStream_t st);

cudaError_t launch_quantize_blockwise(const float* src, void* q, float* absmax, int64_t n, bool is_signed,
                                      cudaStream_t st);
cudaError_t launch_dequantize_blockwise(const void* q, const float* absmax, float* dst, int64_t n, bool is_signed,
                                        cudaStream_t st);
cudaError_t launch_quantize_tile16(const float* src, int8_t* q, float* absmax, int64_t rows, int64_t cols,
                                   cudaStream_t st);
cudaError_t launch_dequantize_tile16(const int8_t* q, const float* absmax, float* dst, int64_t rows, int64_t cols,
                                     cudaStream_t st);

}  // namespace came
