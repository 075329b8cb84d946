"""Shared helpers of the GPU parity tests: run a came_b200 optimizer and the CPU oracle side by side on
identical seeded inputs and report the differences."""
from __future__ import annotations

import numpy as np
import torch

from oracle import came_oracle as orc


def make_inputs(shapes, dtype, steps, seed, outlier_rows=True, grad_scale=1e-3, per_tensor_scale=False,
                student_t_frac=0.0):
    """Seeded parameters N(0, 0.02^2) and per-step gradients N(0, grad_scale^2).
    outlier_rows: every 7th row x100.  per_tensor_scale: each tensor's gradients are scaled by its own
    10^U(-5, -2) instead of grad_scale (the Llama-7B benchmark configuration).  student_t_frac: that fraction of
    the entries is replaced by grad_scale * StudentT(nu=2) draws (the Llama-1B drift configuration)."""
    rs = np.random.RandomState(seed)
    params = [torch.from_numpy((rs.standard_normal(s) * 0.02).astype(np.float32)).to(dtype) for s in shapes]
    scales = [10.0 ** rs.uniform(-5, -2) if per_tensor_scale else grad_scale for _ in shapes]
    grads = []
    for _ in range(steps):
        gs = []
        for s, sc in zip(shapes, scales):
            g = (rs.standard_normal(s) * sc).astype(np.float32)
            if outlier_rows:
                g[::7] *= 100.0
            if student_t_frac > 0.0:
                mask = rs.random_sample(s) < student_t_frac
                g[mask] = (rs.standard_t(2.0, size=int(mask.sum())) * sc).astype(np.float32)
            gs.append(torch.from_numpy(g).to(dtype))
        grads.append(gs)
    return params, grads


def hyper_of(h):
    return orc.Hyper(lr=h["lr"], beta1=h["betas"][0], beta2=h["betas"][1], beta3=h["betas"][2], eps0=h["eps"][0],
                     eps1=h["eps"][1], clip_threshold=h["clip_threshold"], weight_decay=h["weight_decay"])


STATE_KEYS_Q = ["exp_avg_q", "exp_avg_sq_row_q", "exp_avg_sq_col_q", "exp_avg_res_row_q", "exp_avg_res_col_q",
                "exp_avg_sq_q"]
STATE_KEYS_F = ["exp_avg_absmax", "exp_avg_sq_row_absmax", "exp_avg_sq_col_absmax", "exp_avg_res_row_absmax",
                "exp_avg_res_col_absmax", "exp_avg_sq_absmax", "exp_avg", "exp_avg_sq_row", "exp_avg_sq_col",
                "exp_avg_res_row", "exp_avg_res_col", "exp_avg_sq"]


def relerr(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    return ((a - b).norm() / b.norm().clamp_min(1e-300)).item()


def run_pair(opt_cls, preset_of, shapes, dtype, steps, hyper, seed, device="cuda", opt_kwargs=None, oracle_kw=None,
             **input_kw):
    """Steps `opt_cls` on the GPU and the oracle on the CPU.  `preset_of(dim)` gives the oracle preset of a
    tensor.  Returns a dict of worst-case differences over all steps / tensors."""
    params0, grads = make_inputs(shapes, dtype, steps, seed, **input_kw)
    gp = [torch.nn.Parameter(p.clone().to(device)) for p in params0]
    opt = opt_cls(gp, **hyper, **(opt_kwargs or {}))
    hp = hyper_of(hyper)
    cp = [p.clone() for p in params0]
    sems = [preset_of(p.dim()) for p in cp]
    states = [orc.init_state(p, s) for p, s in zip(cp, sems)]
    out = {"p_rel": 0.0, "p_diff_frac": 0.0, "p_maxspacing": 0.0, "p_far_frac": 0.0, "code_frac": 0.0, "code_frac2": 0.0, "code_max": 0,
           "f_rel": 0.0}
    eps = {torch.float32: 2.0 ** -23, torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}[dtype]
    scale = [p.float().abs() for p in cp]      # running max of |p| per entry: the magnitude a rounding happened at
    for gs in grads:
        for p, g in zip(gp, gs):
            p.grad = g.clone().to(device)
        opt.step()
        for i, g in enumerate(gs):
            kw = (oracle_kw or {}) if cp[i].dim() == 1 else {}
            cp[i] = orc.step(cp[i], g, states[i], hp, sems[i], **kw)
        for i, (p, c) in enumerate(zip(gp, cp)):
            got, ref = p.data.float().cpu(), c.float()
            scale[i] = torch.maximum(scale[i], ref.abs())
            out["p_rel"] = max(out["p_rel"], relerr(got, ref))
            # distance in spacings of `dtype` at the running-max magnitude, with a tenth of a typical update
            # (lr * 1) as floor: an entry that cancels to ~0 has no meaningful spacing of its own
            spacing = (scale[i] * eps).clamp_min(0.1 * hyper["lr"])
            out["p_diff_frac"] = max(out["p_diff_frac"], (got != ref).float().mean().item())
            dist = (got - ref).abs() / spacing
            out["p_maxspacing"] = max(out["p_maxspacing"], dist.max().item())
            out["p_far_frac"] = max(out["p_far_frac"], (dist > 2.0).float().mean().item())
    for p, st in zip(gp, states):
        gst = opt.state[p]
        for k in STATE_KEYS_Q:
            if k in st:
                d = (gst[k].cpu().to(torch.int32) - st[k].to(torch.int32)).abs()
                out["code_frac"] = max(out["code_frac"], (d != 0).float().mean().item())
                out["code_frac2"] = max(out["code_frac2"], (d > 1).float().mean().item())
                out["code_max"] = max(out["code_max"], int(d.max().item()))
        for k in STATE_KEYS_F:
            if k in st:
                out["f_rel"] = max(out["f_rel"], relerr(gst[k].cpu(), st[k]))
    return out, opt, gp
