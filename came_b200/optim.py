"""Drop-in `torch.optim` classes of tukisuwa/CAME backed by libcame_b200 (sm_100a kernels).

Same names, constructor arguments, `param_groups` keys, error behaviour and persistent state keys as
came_pytorch/{CAME,CAMECUDA,CAME8bit,CAME8bitFull,CAME8bitMemory,CAME8bit2D}.py.  Each class maps its
tensors to one of three state layouts and to the arithmetic variant of the reference code path that
class would have taken on a CUDA device:

    class            2-D tensor                              1-D tensor
    CAME             fp32 states, CAME.py:117-172            fp32, CAME.py:132-143
    CAMECUDA         fp32 states, came_kernels.cu:5250-5413  fp32, CAMECUDA.py:247-273
    CAME8bit         tile layout, came_kernels.cu:3598-4040  flat layout, came_kernels.cu:4172-4255
    CAME8bit2D       tile layout (2-D CUDA tensors only)     NotImplementedError
    CAME8bitFull     flat layout, came_kernels.cu:4792-5248  flat layout, came_kernels.cu:4172-4255
    CAME8bitMemory   flat layout                             flat layout, fp16 update (4257-4340)

All tensors of a step are handed to the library in one call; there is no per-tensor launch loop, no
scratch tensor in the optimizer state and no CPU / eager fallback: parameters must live on a CUDA device.
"""
from __future__ import annotations

import copy
import math
import warnings

import torch
import torch.optim

from . import _lib
from .engine import Entry, StepEngine, make_hyper

BLOCK = 256
TILE = 16

_FLAGS_CAME = _lib.F_WD_ADD2
_FLAGS_CUDAFP_2D = _lib.F_SQ_CLAMP | _lib.F_RESROW_CLAMP | _lib.F_RESCOL_CLAMP
_FLAGS_CUDAFP_1D = _lib.F_RSQRT_CLAMP | _lib.F_WD_ADD2
_FLAGS_TILE8 = _lib.F_SQ_FIX | _lib.F_RESROW_FIX | _lib.F_WD_MUL2
_FLAGS_FLAT8_2D = _lib.F_SQ_FIX | _lib.F_RESROW_FIX | _lib.F_RESCOL_CLAMP
_FLAGS_FLAT8_1D = _lib.F_RSQRT_CLAMP
# tensors of more than two dimensions take the classes' generic torch paths in the reference (1e-30 clamps, two roundings
# of p, Python scalars): CAMECUDA.py:275-326, CAME8bitFull.py:1006-1075
_FLAGS_ND_GENERIC = _lib.F_SQ_CLAMP | _lib.F_RESROW_CLAMP | _lib.F_RESCOL_CLAMP | _lib.F_WD_ADD2

_SCRATCH_KEYS = frozenset({
    # keys the reference keeps in its state dicts for kernel scratch; accepted on load, never produced
    "r_factor", "c_factor", "r_res_factor", "c_res_factor", "res_row_sum", "res_col_sum", "res_row_partial",
    "res_col_partial", "sum_sq_row", "sum_update", "sum_update_partial", "sum_res_row", "scratch_fp32",
    "row_factor_fp32", "col_factor_fp32", "row_mean_fp32", "reduce_partial", "sum_row_state", "update_fp32",
    "grad_fp32", "exp_avg_fp32", "row_absmax_scratch", "_cuda_nonfactored_update_fp16", "sum_update_slice",
    "sum_update_equiv", "sum_update_chunk",
})


def _num_blocks(n: int) -> int:
    return max(1, math.ceil(n / BLOCK))


def _check_common(lr, eps, clip_threshold, betas):
    if lr is None or lr <= 0.0:
        raise ValueError(f"lr must be > 0, got {lr}")
    if clip_threshold <= 0.0:
        raise ValueError(f"clip_threshold must be > 0, got {clip_threshold}")
    if len(eps) != 2:
        raise ValueError(f"eps must be a tuple of length 2, got eps={eps}")
    if len(betas) != 3:
        raise ValueError(f"betas must be a tuple of length 3, got betas={betas}")


# ----------------------------------------------------------------------------------------------
# state initialisers (persistent keys of the reference's state dicts; scratch is not stored)
# ----------------------------------------------------------------------------------------------

def _qstate(shape, device, signed):
    """blockwise_quantization.py:17-27: zero codes, absmax of ones."""
    q = torch.zeros(shape, device=device, dtype=torch.int8 if signed else torch.uint8)
    return q, torch.ones((_num_blocks(q.numel()),), device=device, dtype=torch.float32)


def init_state_tile(state: dict, p: torch.Tensor) -> None:
    """came8bit2d_state.py:33-75 without the twelve scratch tensors."""
    rows, cols = p.shape
    dev = p.device
    tile_rows, tile_cols = math.ceil(rows / TILE), math.ceil(cols / TILE)
    state["_mode"] = "8bit2d"
    state["exp_avg_q"] = torch.zeros((rows, cols), device=dev, dtype=torch.int8)
    state["exp_avg_absmax"] = torch.zeros((tile_rows * tile_cols,), device=dev, dtype=torch.float32)
    for key, n in (("exp_avg_sq_row", rows), ("exp_avg_sq_col", cols), ("exp_avg_res_row", rows), ("exp_avg_res_col", cols)):
        state[key + "_q"], state[key + "_absmax"] = _qstate((n,), dev, False)
    state["rows"], state["cols"] = rows, cols
    state["tile_rows"], state["tile_cols"], state["num_tiles"] = tile_rows, tile_cols, tile_rows * tile_cols


def bind_flat_views(state: dict) -> None:
    """CAME8bitFull.py:215-223: index 0 of the stacked vectors is the second moment, 1 the residual."""
    for axis in ("row", "col"):
        state[f"exp_avg_sq_{axis}_q"] = state[f"factored_{axis}_q"][0]
        state[f"exp_avg_res_{axis}_q"] = state[f"factored_{axis}_q"][1]
        state[f"exp_avg_sq_{axis}_absmax"] = state[f"factored_{axis}_absmax"][0]
        state[f"exp_avg_res_{axis}_absmax"] = state[f"factored_{axis}_absmax"][1]


def init_state_flat(state: dict, p: torch.Tensor) -> None:
    """CAME8bitFull.py:748-788, 920-924 / CAME8bitMemory.py:390-447 without scratch."""
    dev = p.device
    state["step"] = 0
    state["_mode"] = "full8bit"
    state["RMS"] = 0
    state["exp_avg_q"], state["exp_avg_absmax"] = _qstate(tuple(p.shape), dev, True)
    factored = p.dim() >= 2
    state["factored"] = factored
    if factored:
        # CAME8bitFull.py:762-783: the vectors of an N-D tensor keep its leading dimensions; one absmax per 256 of their
        # flattened entries
        row_shape, col_shape = tuple(p.shape[:-1]), tuple(p.shape[:-2]) + tuple(p.shape[-1:])
        state["factored_row_q"] = torch.zeros((2, *row_shape), device=dev, dtype=torch.uint8)
        state["factored_row_absmax"] = torch.ones((2, _num_blocks(math.prod(row_shape))), device=dev, dtype=torch.float32)
        state["factored_col_q"] = torch.zeros((2, *col_shape), device=dev, dtype=torch.uint8)
        state["factored_col_absmax"] = torch.ones((2, _num_blocks(math.prod(col_shape))), device=dev, dtype=torch.float32)
        bind_flat_views(state)
        state["_cuda_factored_fastpath"] = True
        state["_cuda_factored_nd_ext_path"] = False
        state["_cuda_factored_nd_chunked_ext_path"] = False
        state["_cuda_factored_ext_path"] = True
    else:
        state["exp_avg_sq_q"], state["exp_avg_sq_absmax"] = _qstate(tuple(p.shape), dev, False)
        state["_cuda_nonfactored_fastpath"] = True


def init_state_fp(state: dict, p: torch.Tensor, *, mode_tag) -> None:
    """CAMECUDA.py:83-118 (mode_tag "cudafp") / CAME.py:97-112 (mode_tag None) without scratch."""
    dev = p.device
    shape = tuple(p.shape)
    state["step"] = 0
    factored = p.dim() >= 2
    if mode_tag is not None:
        state["_mode"] = mode_tag
        state["factored"] = factored
    state["exp_avg"] = torch.zeros(shape, device=dev, dtype=torch.float32)
    if factored:
        row_shape, col_shape = shape[:-1], shape[:-2] + shape[-1:]      # CAMECUDA.py:93-98
        state["exp_avg_sq_row"] = torch.zeros(row_shape, device=dev, dtype=torch.float32)
        state["exp_avg_sq_col"] = torch.zeros(col_shape, device=dev, dtype=torch.float32)
        state["exp_avg_res_row"] = torch.zeros(row_shape, device=dev, dtype=torch.float32)
        state["exp_avg_res_col"] = torch.zeros(col_shape, device=dev, dtype=torch.float32)
    else:
        state["exp_avg_sq"] = torch.zeros(shape, device=dev, dtype=torch.float32)
    if mode_tag is not None:
        state["_cuda_fp_factored_fastpath"] = factored
        state["_cuda_fp_nonfactored_fastpath"] = not factored
    else:
        state["RMS"] = 0


# ----------------------------------------------------------------------------------------------
# base class
# ----------------------------------------------------------------------------------------------

class _CameB200Optimizer(torch.optim.Optimizer):
    """Shared step machinery.  Subclasses implement `_route(p, grad, group)` -> (layout, flags, variant)
    with layout in {"fp", "tile", "flat"} and variant 0 (kernel-style fp32 scalars) or 1 (Python-style)."""

    _fp_mode_tag = None

    def __init__(self, params, defaults):
        super().__init__(params, defaults)
        self._engine = StepEngine()
        self.last_step_launches = 0

    @property
    def supports_memory_efficient_fp16(self):
        return True

    @property
    def supports_flat_params(self):
        return False

    # -- routing ------------------------------------------------------------------------------
    def _route(self, p, grad, group):
        raise NotImplementedError

    def _prepare_state(self, p, state, layout) -> None:
        if layout == "tile":
            if len(state) == 0 or state.get("_mode") != "8bit2d":
                state.clear()
                init_state_tile(state, p)
            if state["rows"] != p.shape[0] or state["cols"] != p.shape[1]:
                raise RuntimeError("Parameter shape changed; this optimizer does not support resizing 8-bit state.")
        elif layout == "flat":
            if len(state) == 0 or state.get("_mode") != "full8bit":
                state.clear()
                init_state_flat(state, p)
            if tuple(state["exp_avg_q"].shape) != tuple(p.shape):
                raise RuntimeError("Parameter shape changed; this optimizer does not support resizing 8-bit state.")
        else:
            tag = self._fp_mode_tag
            if len(state) == 0 or (tag is not None and state.get("_mode") != tag):
                state.clear()
                init_state_fp(state, p, mode_tag=tag)

    def _entry(self, p, grad, state, layout, flags, group_index):
        p_data, g_data, keep = p.data, grad.data, []
        copy_back = None
        if not p_data.is_contiguous():
            # came8bit2d_state.py:25-30: step a contiguous copy, then copy back
            p_data = p_data.contiguous()
            copy_back = (p, p_data)
        if not g_data.is_contiguous():
            g_data = g_data.contiguous()
            keep.append(g_data)
        e = Entry(p=p_data, g=g_data, mode=0, flags=flags, group=group_index, keep=keep)
        factored = p.dim() >= 2
        if layout == "fp":
            e.mode = _lib.MODE_FP32
            e.m = state["exp_avg"]
            if factored:
                e.sq_row, e.sq_col = state["exp_avg_sq_row"], state["exp_avg_sq_col"]
                e.res_row, e.res_col = state["exp_avg_res_row"], state["exp_avg_res_col"]
            else:
                e.sq_row = state["exp_avg_sq"]
        else:
            e.mode = _lib.MODE_TILE8 if layout == "tile" else _lib.MODE_FLAT8
            e.m, e.m_absmax = state["exp_avg_q"], state["exp_avg_absmax"]
            if factored:
                e.sq_row, e.sq_row_absmax = state["exp_avg_sq_row_q"], state["exp_avg_sq_row_absmax"]
                e.sq_col, e.sq_col_absmax = state["exp_avg_sq_col_q"], state["exp_avg_sq_col_absmax"]
                e.res_row, e.res_row_absmax = state["exp_avg_res_row_q"], state["exp_avg_res_row_absmax"]
                e.res_col, e.res_col_absmax = state["exp_avg_res_col_q"], state["exp_avg_res_col_absmax"]
            else:
                e.sq_row, e.sq_row_absmax = state["exp_avg_sq_q"], state["exp_avg_sq_absmax"]
        return e, copy_back

    # -- the step -----------------------------------------------------------------------------
    def _collect(self):
        entries, hypers, copy_backs = [], self._hypers(), []
        for gi, group in enumerate(self.param_groups):
            if gi >= _lib.MAX_GROUPS // 2:
                raise RuntimeError(f"came_b200 supports at most {_lib.MAX_GROUPS // 2} param_groups")
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("CAME does not support sparse gradients.")
                grad = p.grad
                if not p.is_cuda:
                    raise RuntimeError(
                        "came_b200 steps CUDA tensors only (there is no CPU fallback); "
                        f"got a parameter on {p.device}")
                if p.dim() == 0:
                    raise NotImplementedError("came_b200 does not step 0-dimensional parameters")
                layout, flags, variant = self._route(p, grad, group)
                state = self.state[p]
                self._prepare_state(p, state, layout)
                if "step" in state:
                    state["step"] += 1
                e, cb = self._entry(p, grad, state, layout, flags, 2 * gi + variant)
                entries.append(e)
                if cb is not None:
                    copy_backs.append(cb)
        return entries, hypers, copy_backs

    def _hypers(self):
        """Two hyper-parameter records per param_group (kernel-style and Python-style scalars), re-read every step.
        A group may carry `grad_scale` (default 1): its gradients are multiplied by it as the kernels read them, e.g.
        the inverse of a loss scale, which saves the trainer's separate unscale pass over the gradients (the
        reference, like torch's other optimizers, expects unscaled gradients)."""
        hypers = []
        for group in self.param_groups:
            hp = (group["lr"], group["betas"], group["eps"], group["clip_threshold"], group["weight_decay"])
            gs = float(group.get("grad_scale", 1.0))
            hypers.append(make_hyper(*hp, python_scalars=False, grad_scale=gs))
            hypers.append(make_hyper(*hp, python_scalars=True, grad_scale=gs))
        return hypers

    def _signature(self):
        """What decides the tensor table of a step: per parameter its gradient's address, dtype and shape (None for a
        parameter without gradient).  While it stays the same the plans of the previous step are stepped again
        without rebuilding the per-tensor entries (hyper-parameters are re-read every step all the same)."""
        sig = []
        for group in self.param_groups:
            for p in group["params"]:
                g = p.grad
                if g is None:
                    sig.append(None)
                elif g.is_sparse or not (g.is_contiguous() and p.is_contiguous()):
                    return None            # slow path: raises / copies as the reference does
                else:
                    sig.append((p.data_ptr(), g.data_ptr(), g.dtype, p.shape))
        return sig

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        sig = self._signature()
        cached = getattr(self, "_step_cache", None)
        if sig is not None and cached is not None and cached[0] == sig and cached[3] == len(self.param_groups):
            _, plans, stepped_states, _ = cached
            for st in stepped_states:
                st["step"] += 1
            hypers = self._hypers()
            launches = 0
            for plan in plans:
                plan.step(hypers)
                launches += plan.last_launches
            self.last_step_launches = launches
            return loss
        self._step_cache = None
        entries, hypers, copy_backs = self._collect()
        if entries:
            self.last_step_launches = self._engine.step(entries, hypers)
        for p, p_data in copy_backs:
            p.data.copy_(p_data)
        if entries and sig is not None and not copy_backs and not any(e.keep for e in entries):
            stepped = [self.state[p] for g in self.param_groups for p in g["params"]
                       if p.grad is not None and "step" in self.state[p]]
            self._step_cache = (sig, list(self._engine.plans.values()), stepped, len(self.param_groups))
        return loss

    @torch.no_grad()
    def prime_for_cuda_graph(self) -> None:
        """Allocates every state tensor and builds the device tensor table ahead of the first step
        (CAME8bit2D.py:52-72, CAME8bit.py:672-693)."""
        entries, _, _ = self._collect()
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state.get(p)
                if st is not None and "step" in st and p.grad is not None:
                    st["step"] -= 1   # _collect counted a step that did not run
        if entries:
            self._engine.prepare(entries)

    def update_captured_hypers(self) -> None:
        """After `step()` has been captured into a CUDA graph: re-reads lr / betas / eps / clip_threshold /
        weight_decay from `param_groups` and rewrites the records the captured step uploads at each replay, so a
        learning-rate schedule needs no re-capture.  (The reference's captured kernels carry these values as
        launch arguments and have to be captured again, CAME8bit2D.py:52-72.)  Call it before launching the
        replay that should see the new values."""
        self._engine.set_hyper(self._hypers())

    # -- checkpointing --------------------------------------------------------------------------
    def state_dict(self):
        return super().state_dict()

    def load_state_dict(self, state_dict):
        """torch's loader casts every state tensor to the parameter's dtype, which destroys int8/uint8
        codes and fp32 absmax for bf16/fp16 parameters.  Reload, then restore each tensor with the dtype
        it was saved with, drop the reference's scratch keys and rebuild the flat-layout alias views."""
        super().load_state_dict(state_dict)
        saved_groups = state_dict["param_groups"]
        saved_state = state_dict["state"]
        ids = [i for g in saved_groups for i in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        for pid, p in zip(ids, params):
            if pid not in saved_state:
                continue
            st = self.state[p]
            for k, v in saved_state[pid].items():
                if k in _SCRATCH_KEYS:
                    st.pop(k, None)
                elif torch.is_tensor(v):
                    st[k] = v.detach().to(device=p.device).clone()
                else:
                    st[k] = copy.deepcopy(v)   # torch's loader turns str values such as "_mode" into garbage
            if st.get("_mode") == "full8bit" and st.get("factored", False) and "factored_row_q" in st:
                bind_flat_views(st)
        self._engine.invalidate()
        self._step_cache = None

    def add_param_group(self, param_group):
        super().add_param_group(param_group)
        self._step_cache = None


# ----------------------------------------------------------------------------------------------
# the six classes
# ----------------------------------------------------------------------------------------------

class CAME(_CameB200Optimizer):
    """CAME with fp32 states and the arithmetic of came_pytorch/CAME.py:24-172 (no guards; weight decay
    and update applied as two roundings of p).  `state["RMS"]` is kept as a key but not recomputed."""

    def __init__(self, params, lr=None, eps=(1e-30, 1e-16), clip_threshold=1.0, betas=(0.9, 0.999, 0.9999),
                 weight_decay=0.0):
        assert lr > 0.0
        assert all([0.0 <= beta <= 1.0 for beta in betas])
        defaults = dict(lr=lr, eps=eps, clip_threshold=clip_threshold, betas=betas, weight_decay=weight_decay)
        super().__init__(params, defaults)

    def _route(self, p, grad, group):
        return "fp", _FLAGS_CAME, 1


class CAMECUDA(_CameB200Optimizer):
    """came_pytorch/CAMECUDA.py:16-426: fp32 optimizer state."""

    _fp_mode_tag = "cudafp"

    def __init__(self, params, lr: float, eps=(1e-30, 1e-16), clip_threshold: float = 1.0,
                 betas=(0.9, 0.999, 0.9999), weight_decay: float = 0.0):
        _check_common(lr, eps, clip_threshold, betas)
        if not all(0.0 <= beta <= 1.0 for beta in betas):
            raise ValueError(f"betas must be in [0, 1], got betas={betas}")
        defaults = dict(lr=float(lr), eps=(float(eps[0]), float(eps[1])), clip_threshold=float(clip_threshold),
                        betas=(float(betas[0]), float(betas[1]), float(betas[2])), weight_decay=float(weight_decay))
        super().__init__(params, defaults)

    def _route(self, p, grad, group):
        if p.dim() == 2:
            return "fp", _FLAGS_CUDAFP_2D, 0       # came_kernels.cu:5250-5413
        if p.dim() > 2:
            return "fp", _FLAGS_ND_GENERIC, 1      # CAMECUDA.py:275-326 (generic torch branch)
        return "fp", _FLAGS_CUDAFP_1D, 1           # CAMECUDA.py:247-273 (torch ops, Python scalars)


class CAME8bitFull(_CameB200Optimizer):
    """came_pytorch/CAME8bitFull.py:40-1118: every state blockwise 8-bit, flat layout."""

    def __init__(self, params, lr: float, eps=(1e-30, 1e-16), clip_threshold: float = 1.0,
                 betas=(0.9, 0.999, 0.9999), weight_decay: float = 0.0, block_size: int = 256,
                 prefer_factored_cuda_ext_path: bool = True, cuda_factored_nd_chunk_size_override=None,
                 cuda_factored_nd_chunked_direct_row_sum_min_matrix_numel=None,
                 cuda_factored_nd_chunked_direct_row_sum_max_matrix_numel=None,
                 cuda_nonfactored_use_fp16_update: bool = False):
        _check_common(lr, eps, clip_threshold, betas)
        if block_size <= 0:
            raise ValueError(f"block_size must be > 0, got {block_size}")
        if block_size != BLOCK:
            raise ValueError("came_b200 supports block_size=256 only")
        if cuda_factored_nd_chunk_size_override is not None and int(cuda_factored_nd_chunk_size_override) <= 0:
            raise ValueError("cuda_factored_nd_chunk_size_override must be positive when set")
        defaults = dict(lr=float(lr), eps=(float(eps[0]), float(eps[1])), clip_threshold=float(clip_threshold),
                        betas=(float(betas[0]), float(betas[1]), float(betas[2])), weight_decay=float(weight_decay),
                        block_size=int(block_size))
        super().__init__(params, defaults)
        # accepted for signature compatibility; the fused step has a single code path
        self.prefer_factored_cuda_ext_path = bool(prefer_factored_cuda_ext_path)
        self.cuda_factored_nd_chunk_size_override = cuda_factored_nd_chunk_size_override
        self.cuda_factored_nd_chunked_direct_row_sum_min_matrix_numel = cuda_factored_nd_chunked_direct_row_sum_min_matrix_numel
        self.cuda_factored_nd_chunked_direct_row_sum_max_matrix_numel = cuda_factored_nd_chunked_direct_row_sum_max_matrix_numel
        self.cuda_nonfactored_use_fp16_update = bool(cuda_nonfactored_use_fp16_update)
        self.track_cuda_rms_state = False

    def _flat_route(self, p):
        if p.dim() == 2:
            return "flat", _FLAGS_FLAT8_2D, 0
        if p.dim() > 2:
            return "flat", _FLAGS_ND_GENERIC, 1    # CAME8bitFull.py:1006-1075 (dequantise, torch ops, requantise)
        flags = _FLAGS_FLAT8_1D | (_lib.F_UPDATE_F16 if self.cuda_nonfactored_use_fp16_update else 0)
        return "flat", flags, 0

    def _route(self, p, grad, group):
        return self._flat_route(p)


class CAME8bitMemory(CAME8bitFull):
    """came_pytorch/CAME8bitMemory.py:17-635: flat layout; 1-D tensors carry the update through fp16
    (CAME8bitMemory.py:524-557).  The shared scratch buffers of the reference have no counterpart: the
    fused step needs no per-element scratch."""

    def __init__(self, params, lr: float, eps=(1e-30, 1e-16), clip_threshold: float = 1.0,
                 betas=(0.9, 0.999, 0.9999), weight_decay: float = 0.0, block_size: int = 256):
        super().__init__(params, lr=lr, eps=eps, clip_threshold=clip_threshold, betas=betas,
                         weight_decay=weight_decay, block_size=block_size, prefer_factored_cuda_ext_path=False,
                         cuda_nonfactored_use_fp16_update=False)

    def _route(self, p, grad, group):
        if p.dim() >= 2:
            return self._flat_route(p)
        return "flat", _FLAGS_FLAT8_1D | _lib.F_UPDATE_F16, 0


class CAME8bit(CAME8bitFull):
    """came_pytorch/CAME8bit.py:24-912: 2-D tensors whose gradient dtype equals the parameter dtype take
    the tile layout (CAME8bit.py:216-223); everything else the flat layout of CAME8bitFull."""

    CUDA_1D_RUNTIME_MODE_DEFAULT = "default"
    CUDA_1D_RUNTIME_MODE_REPEATED_FP16_PAIRMIN = "repeated_fp16_pairmin"
    CUDA_ND_RUNTIME_MODE_DEFAULT = "default"
    CUDA_ND_RUNTIME_MODE_CHUNK32_LARGE_DIRECT_ROW_SUM = "chunk32_large_direct_row_sum"
    EXPERIMENTAL_CUDA_TUNING_DEFAULTS = {
        "prefer_cuda_1d_batched_fast_path": False,
        "prefer_cuda_1d_multitensor_fast_path": False,
        "cuda_1d_batched_use_fp16_update": False,
        "cuda_1d_batched_chunk_size": 8,
        "cuda_1d_batched_min_bucket_size": 4,
        "cuda_1d_batched_min_numel": 1024,
        "cuda_1d_batched_max_numel": 65536,
        "cuda_factored_nd_chunk_size_override": None,
        "cuda_factored_nd_chunked_direct_row_sum_min_matrix_numel": None,
        "cuda_factored_nd_chunked_direct_row_sum_max_matrix_numel": None,
        "cuda_nonfactored_use_fp16_update": False,
    }

    def __init__(self, params, lr: float, eps=(1e-30, 1e-16), clip_threshold: float = 1.0,
                 betas=(0.9, 0.999, 0.9999), weight_decay: float = 0.0, block_size: int = 256,
                 prefer_cuda_fast_path: bool = True, prefer_cuda_2d_fast_path=None, prefer_cuda_1d_fast_path=None,
                 prefer_cuda_1d_batched_fast_path: bool = False, prefer_cuda_1d_multitensor_fast_path: bool = False,
                 cuda_1d_batched_use_fp16_update: bool = False, cuda_1d_batched_chunk_size: int = 8,
                 cuda_1d_batched_min_bucket_size: int = 4, cuda_1d_batched_min_numel: int = 1024,
                 cuda_1d_batched_max_numel: int = 65536, cuda_1d_runtime_mode: str = "default",
                 prefer_factored_cuda_ext_path: bool = True, cuda_factored_nd_chunk_size_override=None,
                 cuda_factored_nd_chunked_direct_row_sum_min_matrix_numel=None,
                 cuda_factored_nd_chunked_direct_row_sum_max_matrix_numel=None,
                 cuda_nd_runtime_mode: str = "default", cuda_nonfactored_use_fp16_update: bool = False,
                 cuda_graph_compatible: bool = False):
        if cuda_1d_runtime_mode not in {self.CUDA_1D_RUNTIME_MODE_DEFAULT, self.CUDA_1D_RUNTIME_MODE_REPEATED_FP16_PAIRMIN}:
            raise ValueError(
                "cuda_1d_runtime_mode must be one of "
                f"{self.CUDA_1D_RUNTIME_MODE_DEFAULT!r}, {self.CUDA_1D_RUNTIME_MODE_REPEATED_FP16_PAIRMIN!r}; "
                f"got {cuda_1d_runtime_mode!r}")
        if cuda_nd_runtime_mode not in {self.CUDA_ND_RUNTIME_MODE_DEFAULT, self.CUDA_ND_RUNTIME_MODE_CHUNK32_LARGE_DIRECT_ROW_SUM}:
            raise ValueError(
                "cuda_nd_runtime_mode must be one of "
                f"{self.CUDA_ND_RUNTIME_MODE_DEFAULT!r}, {self.CUDA_ND_RUNTIME_MODE_CHUNK32_LARGE_DIRECT_ROW_SUM!r}; "
                f"got {cuda_nd_runtime_mode!r}")
        given = dict(
            prefer_cuda_1d_batched_fast_path=prefer_cuda_1d_batched_fast_path,
            prefer_cuda_1d_multitensor_fast_path=prefer_cuda_1d_multitensor_fast_path,
            cuda_1d_batched_use_fp16_update=cuda_1d_batched_use_fp16_update,
            cuda_1d_batched_chunk_size=cuda_1d_batched_chunk_size,
            cuda_1d_batched_min_bucket_size=cuda_1d_batched_min_bucket_size,
            cuda_1d_batched_min_numel=cuda_1d_batched_min_numel,
            cuda_1d_batched_max_numel=cuda_1d_batched_max_numel,
            cuda_factored_nd_chunk_size_override=cuda_factored_nd_chunk_size_override,
            cuda_factored_nd_chunked_direct_row_sum_min_matrix_numel=cuda_factored_nd_chunked_direct_row_sum_min_matrix_numel,
            cuda_factored_nd_chunked_direct_row_sum_max_matrix_numel=cuda_factored_nd_chunked_direct_row_sum_max_matrix_numel,
            cuda_nonfactored_use_fp16_update=cuda_nonfactored_use_fp16_update,
        )
        overrides = tuple(k for k, dflt in self.EXPERIMENTAL_CUDA_TUNING_DEFAULTS.items() if given[k] != dflt)
        if overrides:
            warnings.warn(
                "CAME8bit low-level CUDA tuning kwargs are experimental and intended for benchmark/diagnostic use: "
                + ", ".join(overrides) + ". came_b200 accepts them for compatibility; its single fused step ignores "
                "the bucketing knobs.", RuntimeWarning, stacklevel=2)
        if int(cuda_1d_batched_chunk_size) <= 0:
            raise ValueError("cuda_1d_batched_chunk_size must be positive")
        if int(cuda_1d_batched_min_bucket_size) <= 0:
            raise ValueError("cuda_1d_batched_min_bucket_size must be positive")
        if int(cuda_1d_batched_min_numel) <= 0 or int(cuda_1d_batched_max_numel) < int(cuda_1d_batched_min_numel):
            raise ValueError("cuda_1d_batched_min_numel/max_numel must define a positive range")
        fp16_update = bool(cuda_nonfactored_use_fp16_update) or cuda_1d_runtime_mode == self.CUDA_1D_RUNTIME_MODE_REPEATED_FP16_PAIRMIN
        super().__init__(params, lr=lr, eps=eps, clip_threshold=clip_threshold, betas=betas, weight_decay=weight_decay,
                         block_size=block_size, prefer_factored_cuda_ext_path=prefer_factored_cuda_ext_path,
                         cuda_factored_nd_chunk_size_override=cuda_factored_nd_chunk_size_override,
                         cuda_factored_nd_chunked_direct_row_sum_min_matrix_numel=cuda_factored_nd_chunked_direct_row_sum_min_matrix_numel,
                         cuda_factored_nd_chunked_direct_row_sum_max_matrix_numel=cuda_factored_nd_chunked_direct_row_sum_max_matrix_numel,
                         cuda_nonfactored_use_fp16_update=fp16_update)
        self.cuda_1d_runtime_mode = cuda_1d_runtime_mode
        self.cuda_nd_runtime_mode = cuda_nd_runtime_mode
        self.prefer_cuda_fast_path = bool(prefer_cuda_fast_path)
        self.prefer_cuda_2d_fast_path = self.prefer_cuda_fast_path if prefer_cuda_2d_fast_path is None else bool(prefer_cuda_2d_fast_path)
        self.prefer_cuda_1d_fast_path = bool(prefer_cuda_1d_fast_path) if prefer_cuda_1d_fast_path is not None else False
        self.cuda_graph_compatible = bool(cuda_graph_compatible)
        self.experimental_cuda_tuning_overrides = overrides

    def _route(self, p, grad, group):
        # CAME8bit.py:216-223: tile layout needs block 256, a 2-D tensor and matching dtypes
        if self.prefer_cuda_2d_fast_path and p.dim() == 2 and grad.dtype == p.dtype and group["block_size"] == BLOCK:
            return "tile", _FLAGS_TILE8, 0
        return self._flat_route(p)


class CAME8bit2D(_CameB200Optimizer):
    """came_pytorch/CAME8bit2D.py:9-131: 2-D CUDA tensors only, tile layout."""

    def __init__(self, params, lr: float, eps=(1e-30, 1e-16), clip_threshold: float = 1.0,
                 betas=(0.9, 0.999, 0.9999), weight_decay: float = 0.0, block_size: int = 256,
                 cuda_graph_compatible: bool = False):
        _check_common(lr, eps, clip_threshold, betas)
        if block_size != BLOCK:
            raise ValueError("Only block_size=256 is supported in this minimal implementation.")
        defaults = dict(lr=float(lr), eps=(float(eps[0]), float(eps[1])), clip_threshold=float(clip_threshold),
                        betas=(float(betas[0]), float(betas[1]), float(betas[2])), weight_decay=float(weight_decay),
                        block_size=int(block_size))
        super().__init__(params, defaults)
        self.cuda_graph_compatible = bool(cuda_graph_compatible)

    def _collect(self):
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.dim() != 2:
                    raise NotImplementedError("CAME8bit2D currently supports 2D parameters only.")
                if not p.is_cuda:
                    raise NotImplementedError("CAME8bit2D requires CUDA parameters.")
                if p.grad.is_sparse:
                    raise RuntimeError("CAME does not support sparse gradients.")
                if p.grad.dtype != p.dtype:
                    raise RuntimeError(f"Expected g.dtype == p.dtype, got {p.grad.dtype} vs {p.dtype}")
                if self.cuda_graph_compatible and not (p.data.is_contiguous() and p.grad.data.is_contiguous()):
                    raise RuntimeError("CUDA graph capture requires contiguous parameter and gradient tensors.")
        return super()._collect()

    def _route(self, p, grad, group):
        return "tile", _FLAGS_TILE8, 0
