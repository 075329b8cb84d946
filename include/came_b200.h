/*
 * came_b200 -- C ABI of the B200 (sm_100a) CAME optimizer-step library.
 *
 * This is the operator boundary that replaces the pybind11 module `came_pytorch.came_cuda_ext` of
 * tukisuwa/CAME (came_pytorch/came_cuda/csrc/came_bindings.cpp:2026-2051).  Where the reference makes
 * one pybind call per tensor per kernel group (came2d_step, came_fp_factored_step,
 * came_full_factored_{sq_step,expavg_res_prepare,res_step,param_update}, came_full_nonfactored_step,
 * came_full_nonfactored_step_fp16_update), this library takes a table describing every tensor once
 * (a "plan") and steps all of them with one call.
 *
 * Conventions (same as the reference boundary, came_bindings.cpp / came_kernels.cu:3634-3652):
 *   - the caller owns every buffer, including the workspace; nothing here calls cudaMalloc;
 *   - all work is enqueued on the stream passed in, asynchronously, with no host synchronisation;
 *   - all tensors are contiguous row-major; state tensors are updated in place;
 *   - functions return 0 on success, a negative CAME_E_* code otherwise; came_b200_last_error()
 *     gives a message for the calling thread.  No exceptions cross the boundary.
 */
#ifndef CAME_B200_H
#define CAME_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CAME_B200_VERSION 1

typedef void* came_stream_t; /* a cudaStream_t (e.g. torch.cuda.current_stream().cuda_stream) */

/* element types of parameters / gradients */
enum { CAME_DT_F32 = 0, CAME_DT_F16 = 1, CAME_DT_BF16 = 2 };

/* state layout of a tensor */
enum {
    CAME_MODE_FP32 = 0,  /* CAMECUDA: fp32 exp_avg and fp32 row/col vectors (CAMECUDA.py:83-100)              */
    CAME_MODE_TILE8 = 1, /* CAME8bit / CAME8bit2D 2-D: int8 exp_avg, one absmax per 16x16 tile, uint8 vectors  */
                         /* with one absmax per 256 (came8bit2d_state.py:33-55)                                */
    CAME_MODE_FLAT8 = 2  /* CAME8bitFull / CAME8bitMemory, and every 1-D 8-bit tensor: int8 exp_avg with one   */
                         /* absmax per 256 flat elements, uint8 vectors (blockwise_quantization.py:17-27)      */
};

/* per-tensor arithmetic variants; each reproduces one of the reference's code paths */
#define CAME_F_SQ_FIX        (1u << 0) /* mean(v_row) <= 0 -> 1            (came_kernels.cu:319-320)            */
#define CAME_F_SQ_CLAMP      (1u << 1) /* 1e-30 floor on mean, ratio, col  (came_kernels.cu:577,591-592)        */
#define CAME_F_RESROW_FIX    (1u << 2) /* same two guards for the residual row factor                           */
#define CAME_F_RESROW_CLAMP  (1u << 3)
#define CAME_F_RESCOL_CLAMP  (1u << 4) /* 1e-30 floor on the residual col  (came_kernels.cu:1285,1485)          */
#define CAME_F_WD_MUL2       (1u << 5) /* p=T(p*(1-lr*wd)); p=T(p-lr*u)    (came_kernels.cu:2678-2682,3363-3365)*/
#define CAME_F_WD_ADD2       (1u << 6) /* p=T(p-wd_lr*p);   p=T(p-lr*u)    (CAME.py:166-172, CAMECUDA.py:270-273)*/
                                       /* neither: one rounding            (came_kernels.cu:2505-2510)          */
#define CAME_F_UPDATE_F16    (1u << 7) /* 1-D: u rounded to fp16 before use (came_kernels.cu:1069-1122)         */
#define CAME_F_RSQRT_CLAMP   (1u << 8) /* 1-D: rsqrt(max(v,1e-30))         (came_kernels.cu:1041, CAMECUDA.py:267)*/

/*
 * One tensor of the optimizer.  cols == 0 marks a 1-D (non-factored) tensor of `rows` elements, whose
 * second moment lives in sq_row / sq_row_absmax (exp_avg_sq[_q], exp_avg_sq_absmax) and whose other
 * vector fields are NULL.  In CAME_MODE_FP32 the vector fields point at fp32 arrays and every *_absmax
 * is NULL.  Field names follow the reference state keys (came8bit2d_state.py:40-55, CAMECUDA.py:83-100).
 */
typedef struct CameTensorDesc {
    void* p;              /* parameter, p_dtype, [rows, cols] or [rows]           */
    const void* g;        /* gradient, g_dtype, same shape                        */
    void* m;              /* exp_avg (fp32) or exp_avg_q (int8), same shape       */
    float* m_absmax;      /* exp_avg_absmax: [tile_rows*tile_cols] or [ceil(n/256)] */
    void* sq_row;         /* exp_avg_sq_row (fp32|uint8) [rows]; 1-D: exp_avg_sq  */
    float* sq_row_absmax; /* [ceil(rows/256)]                                     */
    void* sq_col;         /* exp_avg_sq_col [cols]                                */
    float* sq_col_absmax;
    void* res_row;        /* exp_avg_res_row [rows]                               */
    float* res_row_absmax;
    void* res_col;        /* exp_avg_res_col [cols]                               */
    float* res_col_absmax;
    int64_t rows;
    int64_t cols;
    int32_t mode;         /* CAME_MODE_*                                          */
    int32_t p_dtype;      /* CAME_DT_*                                            */
    int32_t g_dtype;
    int32_t group;        /* index into the hyper-parameter array given to step   */
    uint32_t flags;       /* CAME_F_*                                             */
    uint32_t batch;       /* 0 or 1: one [rows, cols] matrix.  B > 1: a tensor of more than two dimensions seen as   */
                          /* B contiguous [rows, cols] matrices with one RMS clip over the whole tensor; p, g, m    */
                          /* hold B*rows*cols elements, the row / column vectors B*rows / B*cols entries, quantised */
                          /* in blocks of 256 over those flattened entries (CAME8bitFull.py:1006-1075; modes FP32   */
                          /* and FLAT8 only)                                                                        */
} CameTensorDesc;

/*
 * Hyper-parameters of one param_group, as fp32 (the reference casts double -> float at
 * came_kernels.cu:6224-6231).  Re-read on every step, as LR schedulers mutate group["lr"].
 * The derived fields let the caller choose where the rounding happens: the reference kernels form
 * 1-beta and lr*wd in fp32, its Python paths form them in double and round once.
 */
typedef struct CameHyper {
    float lr;
    float beta1, beta2, beta3;
    float om_beta1, om_beta2, om_beta3; /* 1 - beta                                     */
    float eps0, eps1;                   /* added to g^2 / to the residual               */
    float clip_threshold;
    float weight_decay;                 /* 0 disables decay                             */
    float wd_lr;                        /* weight_decay * lr                            */
    float decay_mul;                    /* 1 - lr * weight_decay (CAME_F_WD_MUL2)       */
    float grad_scale;                   /* every gradient is multiplied by this as it is read (the inverse of a loss  */
                                        /* scale, say: saves the trainer's separate unscale pass over g); 0 means 1   */
    float reserved[2];
} CameHyper;

typedef struct came_plan came_plan_t;

int came_b200_version(void);
const char* came_b200_last_error(void);

/*
 * Blockwise linear absmax codec, block 256, bit-exact with
 * came_pytorch/blockwise_quantization.py:66-82 (quantize_blockwise) and :108-124 (dequantize_blockwise);
 * replaces blockwise_quant / blockwise_dequant (came_bindings.cpp:756-855, came_kernels.cu:849-924).
 * src/dst: n fp32 on the device; q: n int8 (is_signed) or uint8; absmax: max(1, ceil(n/256)) fp32.
 */
int came_b200_quantize_blockwise(const float* src, void* q, float* absmax, int64_t n, int is_signed,
                                 came_stream_t stream);
int came_b200_dequantize_blockwise(const void* q, const float* absmax, float* dst, int64_t n, int is_signed,
                                   came_stream_t stream);

/*
 * Same codec with one absmax per 16x16 tile of a row-major [rows, cols] matrix (tile id =
 * tile_y * ceil(cols/16) + tile_x), the exp_avg layout of came2d_step (came_kernels.cu:2584-2650,
 * 3332-3366: dequantizes to 0 where absmax == 0).
 */
int came_b200_quantize_tile16(const float* src, int8_t* q, float* absmax, int64_t rows, int64_t cols,
                              came_stream_t stream);
int came_b200_dequantize_tile16(const int8_t* q, const float* absmax, float* dst, int64_t rows, int64_t cols,
                                came_stream_t stream);

/*
 * Plan: validates the descriptors (host copies; the pointers inside are device pointers), lays the
 * per-tensor scratch and the per-kernel work lists out in `workspace` (device memory of at least
 * came_b200_workspace_bytes(), 256-byte aligned, owned by the caller, must outlive the plan) and
 * uploads them on `stream`.  Replaces the per-call TORCH_CHECK validation of came_bindings.cpp:617-754
 * and the pointer tables of make_device_ptr_tensor (came_bindings.cpp:443-459).
 */
size_t came_b200_workspace_bytes(const CameTensorDesc* descs, int n_tensors);
int came_b200_plan_create(const CameTensorDesc* descs, int n_tensors, void* workspace, size_t workspace_bytes,
                          came_stream_t stream, came_plan_t** out);
void came_b200_plan_destroy(came_plan_t* plan);

/* Re-point the gradients (and parameters, when non-NULL) of an existing plan: the analogue of
 * fill_device_ptr_tensor (came_bindings.cpp:461-478).  Arrays of n_tensors device pointers, host memory. */
int came_b200_plan_set_pointers(came_plan_t* plan, const void* const* g, void* const* p, int n_tensors,
                                came_stream_t stream);

/*
 * One optimizer step over every tensor of the plan: replaces came2d_step (came_bindings.cpp:617-754),
 * came_fp_factored_step (1692-1769), came_full_factored_sq_step / expavg_res_prepare / res_step /
 * param_update (1406, 1589, 1507, 1675), came_full_nonfactored_step[_fp16_update] (856, 916).
 */
int came_b200_step(came_plan_t* plan, const CameHyper* hypers, int n_groups, came_stream_t stream);

/*
 * CUDA-graph capture.  came_b200_step may be called while `stream` is being captured: nothing in it synchronises
 * or allocates device memory, and the hyper-parameter upload then reads a page-locked copy kept inside the plan
 * instead of `hypers`, so the captured copy node stays valid after the call.  Between replays,
 * came_b200_plan_set_hyper rewrites that copy (learning-rate schedules without re-capturing); it makes no CUDA
 * call that touches a stream.  The copy node reads the buffer when the graph runs, so rewrite it only when no
 * replay that should still see the old values is pending.  The gradient and parameter addresses are those of
 * the plan at capture time.  The reference bakes the learning rate into the captured kernel arguments
 * (came_pytorch/CAME8bit2D.py:52-72 prime_for_cuda_graph, came_pytorch/CAME8bit.py:672-693).
 */
int came_b200_plan_set_hyper(came_plan_t* plan, const CameHyper* hypers, int n_groups);

/*
 * Waits for `stream` and reads the plan's device status word: 0, or 1 when a kernel gave up waiting for a
 * staged copy (every wait inside the kernels is bounded; the step's results are then incomplete).  The
 * reference has no counterpart: it checks no launch or device error at all (no cudaGetLastError in
 * came_kernels.cu).
 */
int came_b200_plan_status(came_plan_t* plan, came_stream_t stream, int* status);

/*
 * Self-test of that bounded wait, without a step: enqueues a one-CTA kernel in which two warps wait, through the wait
 * routine of the step kernels, on a barrier that nothing completes; the first has a limit of 4096 polls, the second the
 * full limit.  device_words: three ints of device memory; after the stream has run they hold {1 (the status a timed-out
 * wait records), 0, 0 (neither wait reported success; the second left through the abort flag the first raised)}.
 * Nothing is left in flight and the context stays usable.  No counterpart in the reference.
 */
int came_b200_selftest_bounded_wait(int* device_words, came_stream_t stream);

/* Number of kernel launches the last came_b200_step on this plan enqueued. */
int came_b200_plan_last_launches(const came_plan_t* plan);

/*
 * Per-kernel device timing with CUDA events recorded on the step's stream around every launch: the
 * device-side counterpart of the reference's opt-in wall-clock dispatch counters
 * (`_benchmark_dispatch_timing`, came_pytorch/CAME8bit.py:695-710, 898-910).  Off by default.
 * read_timing waits for the recorded events, adds their durations into ms[k] / launches[k]
 * (arrays of CAME_KERNEL_COUNT, zeroed by the callee) and forgets them.
 */
#define CAME_KERNEL_COUNT 20
int came_b200_plan_set_timing(came_plan_t* plan, int enable);
int came_b200_plan_read_timing(came_plan_t* plan, float* ms, int* launches);
const char* came_b200_kernel_name(int kernel);

/*
 * One CAME step on a single 1-D tensor WITHOUT any caller-provided workspace.  This entry point has no
 * counterpart in the reference.  It exists for hosts that cannot allocate device memory at the point where they
 * step (the device was handed to the host's own arena at start-up, or the step runs inside a memory plan that
 * forbids new allocations) and so cannot produce the workspace came_b200_plan_create() needs.  The block sums the
 * two kernels exchange live in a fixed device array inside the library instead:
 *   - n <= CAME_B200_NOALLOC_MAX_ELEMS, otherwise CAME_E_UNSUPPORTED;
 *   - mode is CAME_MODE_FLAT8 (m: int8 codes, v: uint8 codes, both with absmax per 256) or CAME_MODE_FP32
 *     (m, v: fp32; the absmax pointers are ignored); flags as for a 1-D CameTensorDesc;
 *   - all calls on a device share that array: calls that overlap on the GPU race, calls on one stream are safe;
 *   - the first call on a device resolves the array's address; make it outside stream capture;
 *   - no cudaMalloc, cudaFree or allocating library call is made.
 * Results are those of came_b200_step() for the same tensor.
 */
#define CAME_B200_NOALLOC_MAX_ELEMS (1 << 22)
int came_b200_step_vector_noalloc(void* p, const void* g, void* m, float* m_absmax, void* v, float* v_absmax,
                                  int64_t n, int mode, int p_dtype, int g_dtype, uint32_t flags,
                                  const CameHyper* hyper, came_stream_t stream);

/*
 * Multi-GPU weight exchange (no counterpart in the reference, which is single-GPU): one plain asynchronous
 * device-to-device copy of `bytes` from `src` (memory of GPU `src_device`, mapped into this process, e.g. through
 * a CUDA IPC handle) to `dst` (memory of the current device) on `stream`, a stream of the current device.  The copy
 * is issued from the destination side, so it runs on the destination GPU's copy engine and never waits for a time
 * slice on the source GPU, which another process keeps busy.  Peer access to `src_device` is enabled on first use;
 * pass -1 when `src` was mapped by came_b200_ipc_open (which enables it itself).
 */
int came_b200_peer_copy_async(void* dst, const void* src, size_t bytes, int src_device, came_stream_t stream);

/*
 * Mapping another process's device buffer for came_b200_peer_copy_async (CUDA IPC, plain cudaMalloc memory only).
 * export: handle of the allocation that contains `ptr` and the offset of `ptr` inside it; send both to the peer
 *         process by any means.  open: maps that allocation into the CURRENT device's address space with peer
 *         access (the current device is the one that will pull) and returns its base; the buffer is at
 *         base + offset.  close: unmaps it.  The exporting process must keep the allocation alive meanwhile.
 */
#define CAME_B200_IPC_HANDLE_BYTES 64
int came_b200_ipc_export(const void* ptr, unsigned char handle[CAME_B200_IPC_HANDLE_BYTES], uint64_t* offset);
int came_b200_ipc_open(const unsigned char handle[CAME_B200_IPC_HANDLE_BYTES], void** base);
int came_b200_ipc_close(void* base);

/*
 * Push mode of the weight exchange (no counterpart in the reference): the step itself delivers the updated weights.
 * `local_base` / `local_bytes` describe the buffer of the current device that holds the parameters of this plan, and
 * `peer_bases[k]` (k < n_peers <= 7) the same buffer of peer k as mapped into this process (came_b200_ipc_open:
 * base + offset).  From the next came_b200_step on, the kernel that applies the update of a tensor also stores every
 * new value at the same offset of every peer buffer, with plain stores over NVLink, for the tensors that
 * came_b200_plan_pushed reports (those the fused momentum / apply kernel steps); the others still have to be copied
 * (came_b200_peer_copy_async).  The stores are complete when the step's kernels are: order a cross-process
 * synchronisation after the step on `stream` before a peer reads them.  Every such tensor must lie inside the local
 * buffer (checked here and by came_b200_plan_set_pointers); n_peers == 0 switches the mode off.
 */
int came_b200_plan_set_push(came_plan_t* plan, const void* local_base, size_t local_bytes, void* const* peer_bases,
                            int n_peers);
/* flags[i] = 1 when tensor i of the plan is delivered by the push mode once it is switched on, else 0 */
int came_b200_plan_pushed(const came_plan_t* plan, int* flags, int n_tensors);

/* error codes */
#define CAME_OK 0
#define CAME_E_INVALID (-1)   /* bad argument / descriptor; see came_b200_last_error() */
#define CAME_E_WORKSPACE (-2) /* workspace too small or misaligned                      */
#define CAME_E_CUDA (-3)      /* a CUDA runtime call failed                             */
#define CAME_E_UNSUPPORTED (-4)

#ifdef __cplusplus
}
#endif
#endif /* CAME_B200_H */
