"""Drives the reference's compiled CUDA extension (oracle/_ref/came_cuda_ext.so, built by oracle/build_ref.py)
operator by operator -- TEST INFRASTRUCTURE ONLY.

The reference's Python classes do not travel to the GPU machine; its compiled operators do.  This module allocates
the state and scratch tensors exactly as the reference's state initialisers do and issues the operator calls in the
reference's order, so that the kernels of tukisuwa/CAME themselves produce the second-oracle trajectories
(tests/golden/make_golden_gpu.py) and the GPU baseline timing (bench.py --impl reference_ext).  Nothing in the
shipped package imports it.

    layout "tile"  -> came2d_step                      (came8bit2d_state.py:33-75 init, :90-139 call)
    layout "flat"  -> came_full_factored_sq_step, ..._expavg_res_prepare, ..._res_step, ..._param_update
                      (CAME8bitFull.py:748-917 init, :618-746 calls); 1-D: came_full_nonfactored_step[_fp16_update]
                      (CAME8bitFull.py:470-509, 920-937; CAME8bitMemory.py:524-557)
    layout "fp"    -> came_fp_factored_step            (CAMECUDA.py:83-140 init, :142-192 call); 2-D only
"""
from __future__ import annotations

import math

import torch

from oracle import build_ref

BLOCK = 256


def load():
    """The extension module, or None when it has not been built."""
    return build_ref.load()


def _qstate(shape, device, signed):
    """blockwise_quantization.py:17-27: zero codes, absmax of ones."""
    n = math.prod(shape)
    q = torch.zeros(shape, device=device, dtype=torch.int8 if signed else torch.uint8)
    return q, torch.ones((max(1, math.ceil(n / BLOCK)),), device=device, dtype=torch.float32)


def init_state(p: torch.Tensor, layout: str, *, update_f16: bool = False) -> dict:
    dev = p.device
    f32 = dict(device=dev, dtype=torch.float32)
    st: dict = {"layout": layout, "dim": p.dim()}
    if p.dim() == 1:
        # CAME8bitFull.py:920-937 (flat layout; CAME8bit sends its 1-D CUDA tensors here too, CAME8bit.py:812-843)
        assert layout in ("flat", "tile")
        n = p.numel()
        st["exp_avg_q"], st["exp_avg_absmax"] = _qstate((n,), dev, True)
        st["exp_avg_sq_q"], st["exp_avg_sq_absmax"] = _qstate((n,), dev, False)
        st["update"] = torch.empty(n, device=dev, dtype=torch.float16 if update_f16 else torch.float32)
        st["sum_update_partial"] = torch.empty(((n + BLOCK - 1) // BLOCK,), **f32)
        st["sum_update"] = torch.zeros((1,), **f32)
        st["update_f16"] = update_f16
        return st
    rows, cols = p.shape
    if layout == "tile":
        # came8bit2d_state.py:33-75
        tr, tc = math.ceil(rows / 16), math.ceil(cols / 16)
        st["exp_avg_q"] = torch.zeros((rows, cols), device=dev, dtype=torch.int8)
        st["exp_avg_absmax"] = torch.zeros((tr * tc,), **f32)
        for key, n in (("exp_avg_sq_row", rows), ("exp_avg_sq_col", cols), ("exp_avg_res_row", rows), ("exp_avg_res_col", cols)):
            st[key + "_q"], st[key + "_absmax"] = _qstate((n,), dev, False)
        for key, n in (("r_factor", rows), ("c_factor", cols), ("r_res_factor", rows), ("c_res_factor", cols),
                       ("res_row_sum", rows), ("res_col_sum", cols), ("res_row_partial", tc * rows),
                       ("res_col_partial", tr * cols), ("sum_sq_row", 1), ("sum_update", 1),
                       ("sum_update_partial", (rows * cols + 255) // 256), ("sum_res_row", 1)):
            st[key] = torch.empty((n,), **f32)
    elif layout == "flat":
        # CAME8bitFull.py:748-917 (2-D, prefer_factored_cuda_ext_path)
        st["exp_avg_q"], st["exp_avg_absmax"] = _qstate((rows, cols), dev, True)
        for key, n in (("exp_avg_sq_row", rows), ("exp_avg_sq_col", cols), ("exp_avg_res_row", rows), ("exp_avg_res_col", cols)):
            st[key + "_q"], st[key + "_absmax"] = _qstate((n,), dev, False)
        st["exp_avg_fp32"] = torch.empty((rows, cols), **f32)
        st["scratch_fp32"] = torch.empty((rows, cols), **f32)
        st["row_factor_fp32"] = torch.empty((rows,), **f32)
        st["col_factor_fp32"] = torch.empty((cols,), **f32)
        st["row_absmax_scratch"] = torch.empty(((rows + BLOCK - 1) // BLOCK,), **f32)
        st["reduce_partial"] = torch.empty((max((rows + 255) // 256, (rows * cols + 255) // 256),), **f32)
        st["sum_row_state"] = torch.zeros((1,), **f32)
        st["sum_update"] = torch.zeros((1,), **f32)
    elif layout == "fp":
        # CAMECUDA.py:83-140
        st["exp_avg"] = torch.zeros((rows, cols), **f32)
        for key, n in (("exp_avg_sq_row", rows), ("exp_avg_sq_col", cols), ("exp_avg_res_row", rows), ("exp_avg_res_col", cols)):
            st[key] = torch.zeros((n,), **f32)
        st["scratch_fp32"] = torch.empty((rows, cols), **f32)
        st["row_factor_fp32"] = torch.empty((rows,), **f32)
        st["col_factor_fp32"] = torch.empty((cols,), **f32)
        st["sum_update"] = torch.zeros((1,), **f32)
        st["reduce_partial"] = torch.empty((max((rows + 255) // 256, (rows * cols + 255) // 256),), **f32)
        st["sum_row_state"] = torch.zeros((1,), **f32)
    else:
        raise ValueError(layout)
    return st


def step(ext, p: torch.Tensor, g: torch.Tensor, st: dict, h: dict) -> None:
    """One in-place step of tensor `p` with gradient `g`; `h` holds lr, betas, eps, clip_threshold, weight_decay."""
    b1, b2, b3 = (float(x) for x in h["betas"])
    e0, e1 = (float(x) for x in h["eps"])
    lr, clip, wd = float(h["lr"]), float(h["clip_threshold"]), float(h["weight_decay"])
    if st["dim"] == 1:
        g32 = g if g.dtype == torch.float32 else g.float()          # CAME8bitFull.py:138-146
        fn = ext.came_full_nonfactored_step_fp16_update if st["update_f16"] else ext.came_full_nonfactored_step
        fn(p, g32, st["exp_avg_q"], st["exp_avg_absmax"], st["exp_avg_sq_q"], st["exp_avg_sq_absmax"], st["update"],
           st["sum_update_partial"], st["sum_update"], b1, b2, e0, lr, clip, wd, BLOCK)
        return
    if st["layout"] == "tile":
        ext.came2d_step(p, g, st["exp_avg_q"], st["exp_avg_absmax"], st["exp_avg_sq_row_q"], st["exp_avg_sq_row_absmax"],
                        st["exp_avg_sq_col_q"], st["exp_avg_sq_col_absmax"], st["exp_avg_res_row_q"],
                        st["exp_avg_res_row_absmax"], st["exp_avg_res_col_q"], st["exp_avg_res_col_absmax"],
                        st["r_factor"], st["c_factor"], st["r_res_factor"], st["c_res_factor"], st["res_row_sum"],
                        st["res_col_sum"], st["res_row_partial"], st["res_col_partial"], st["sum_sq_row"],
                        st["sum_update"], st["sum_update_partial"], st["sum_res_row"], b1, b2, b3, e0, e1, lr, clip, wd,
                        BLOCK)
        return
    g32 = g if g.dtype == torch.float32 else g.float()
    if st["layout"] == "flat":
        # CAME8bitFull.py:618-746
        ext.came_full_factored_sq_step(g32, st["exp_avg_sq_row_q"], st["exp_avg_sq_row_absmax"], st["exp_avg_sq_col_q"],
                                       st["exp_avg_sq_col_absmax"], st["row_factor_fp32"], st["col_factor_fp32"],
                                       st["row_absmax_scratch"], st["reduce_partial"], st["sum_row_state"],
                                       st["sum_update"], b2, e0, BLOCK)
        ext.came_full_factored_expavg_res_prepare(g32, st["exp_avg_q"], st["exp_avg_absmax"], st["row_factor_fp32"],
                                                  st["col_factor_fp32"], st["exp_avg_fp32"], st["scratch_fp32"],
                                                  st["sum_update"], b1, e1, clip, BLOCK)
        ext.came_full_factored_res_step(st["scratch_fp32"], st["exp_avg_res_row_q"], st["exp_avg_res_row_absmax"],
                                        st["exp_avg_res_col_q"], st["exp_avg_res_col_absmax"], st["row_factor_fp32"],
                                        st["col_factor_fp32"], st["row_absmax_scratch"], st["reduce_partial"],
                                        st["sum_row_state"], b3, BLOCK)
        ext.came_full_factored_param_update(p, st["exp_avg_fp32"], st["row_factor_fp32"], st["col_factor_fp32"], lr, wd)
        return
    # CAMECUDA.py:142-192
    ext.came_fp_factored_step(p, g32, st["exp_avg"], st["exp_avg_sq_row"], st["exp_avg_sq_col"], st["exp_avg_res_row"],
                              st["exp_avg_res_col"], st["row_factor_fp32"], st["col_factor_fp32"], st["scratch_fp32"],
                              st["reduce_partial"], st["sum_row_state"], st["sum_update"], b1, b2, b3, e0, e1, lr, clip,
                              wd, BLOCK)


PERSISTENT_KEYS = ("exp_avg_q", "exp_avg_absmax", "exp_avg", "exp_avg_sq_q", "exp_avg_sq_absmax",
                   "exp_avg_sq_row_q", "exp_avg_sq_row_absmax", "exp_avg_sq_col_q", "exp_avg_sq_col_absmax",
                   "exp_avg_res_row_q", "exp_avg_res_row_absmax", "exp_avg_res_col_q", "exp_avg_res_col_absmax",
                   "exp_avg_sq_row", "exp_avg_sq_col", "exp_avg_res_row", "exp_avg_res_col")
