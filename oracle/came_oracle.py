"""CPU restatement of the CAME optimizer step of tukisuwa/CAME -- TEST INFRASTRUCTURE ONLY.

This module is the parity checker for the CUDA library.  It is imported by the
tests, by the smoke check and by the CPU-baseline leg of the benchmark, and by
nothing else: the shipped optimizers never route through it.

It restates, in plain fp32 torch-on-CPU arithmetic (IEEE division and square
root, round-half-even), what the reference computes on each of its paths.  The
reference keeps several slightly different variants of the same algorithm; each
one is a ``Semantics`` preset below, citing the reference lines it follows.

Pinning: the reference ships no tests or golden vectors, so every preset is pinned
against outputs of the reference itself.  ``CAME``, ``CUDAFP_GENERIC`` and
``FLAT8_CPU`` against trajectories of the reference's own Python classes run on CPU
(``tests/golden/traj_<class>_<case>.npz``, generator ``tests/golden/make_golden.py``);
``TILE8``, ``FLAT8`` and ``CUDAFP``, which restate the reference's CUDA kernels,
against trajectories of those kernels themselves: the reference's extension compiled
for sm_100 by ``oracle/build_ref.py`` and run on a B200
(``tests/golden/traj_gpu_<preset>_<case>.npz``, generator
``tests/golden/make_golden_gpu.py``).  The blockwise codec is pinned bit-exactly
against ``came_pytorch/blockwise_quantization.py``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

F32 = torch.float32
BLOCK = 256      # came_pytorch/came8bit2d_state.py:33-55, CAME8bit2D.py:38-39 (only 256 is supported)
TILE = 16        # came_pytorch/came_cuda/csrc/came_kernels.cu:19
SIGNED_QMAX = 127.0    # came_pytorch/blockwise_quantization.py:7
UNSIGNED_QMAX = 255.0  # came_pytorch/blockwise_quantization.py:8


def _f(x: float) -> torch.Tensor:
    """A Python double rounded once to fp32 (came_kernels.cu:6224-6231 casts double -> float)."""
    return torch.tensor(float(x), dtype=F32)


# ----------------------------------------------------------------------------------------------
# Blockwise linear absmax codec (came_pytorch/blockwise_quantization.py:66-124)
# ----------------------------------------------------------------------------------------------

def num_blocks(numel: int, block: int = BLOCK) -> int:
    """blockwise_quantization.py:11-14."""
    return max(1, math.ceil(numel / block))


def quantize_blockwise(x: torch.Tensor, *, signed: bool, block: int = BLOCK):
    """blockwise_quantization.py:66-82: zero-pad to whole blocks, absmax (signed) or max (unsigned)
    per block with 0 -> 1, q = clamp(rint((x / absmax) * qmax))."""
    flat = x.detach().reshape(-1).to(F32)
    n = flat.numel()
    nb = num_blocks(n, block)
    pad = torch.zeros(nb * block, dtype=F32)
    pad[:n] = flat
    pad = pad.view(nb, block)
    if signed:
        a = pad.abs().amax(dim=1)
        a = torch.where(a > 0, a, torch.ones_like(a))
        q = torch.round((pad / a[:, None]) * SIGNED_QMAX).clamp(-SIGNED_QMAX, SIGNED_QMAX).to(torch.int8)
    else:
        a = pad.amax(dim=1)
        a = torch.where(a > 0, a, torch.ones_like(a))
        q = torch.round((pad / a[:, None]) * UNSIGNED_QMAX).clamp(0, UNSIGNED_QMAX).to(torch.uint8)
    return q.reshape(-1)[:n].view(x.shape), a


def dequantize_blockwise(q: torch.Tensor, absmax: torch.Tensor, *, signed: bool, block: int = BLOCK) -> torch.Tensor:
    """blockwise_quantization.py:108-124: q * (absmax / qmax), one absmax per `block` flat elements."""
    flat = q.reshape(-1).to(F32)
    scales = absmax.reshape(-1).repeat_interleave(block)[: flat.numel()]
    qmax = SIGNED_QMAX if signed else UNSIGNED_QMAX
    return (flat * (scales / qmax)).view(q.shape)


def quantize_tile16(m: torch.Tensor):
    """Tile layout of exp_avg: one absmax per 16x16 tile, tile id = tile_y * tile_cols + tile_x,
    out-of-range elements of edge tiles count as 0 (came_kernels.cu:2584-2650)."""
    R, C = m.shape
    tr, tc = math.ceil(R / TILE), math.ceil(C / TILE)
    pad = torch.zeros(tr * TILE, tc * TILE, dtype=F32)
    pad[:R, :C] = m
    t = pad.view(tr, TILE, tc, TILE).permute(0, 2, 1, 3)          # [tr, tc, 16, 16]
    a = t.abs().amax(dim=(2, 3))
    a = torch.where(a > 0, a, torch.ones_like(a))
    q = torch.round((t / a[:, :, None, None]) * SIGNED_QMAX).clamp(-SIGNED_QMAX, SIGNED_QMAX)
    q = q.permute(0, 2, 1, 3).reshape(tr * TILE, tc * TILE)[:R, :C].to(torch.int8)
    return q.contiguous(), a.reshape(-1).contiguous()


def dequantize_tile16(q: torch.Tensor, absmax: torch.Tensor) -> torch.Tensor:
    """m = absmax > 0 ? q * (absmax / 127) : 0 per 16x16 tile (came_kernels.cu:2625-2626, 3359-3360)."""
    R, C = q.shape
    tr, tc = math.ceil(R / TILE), math.ceil(C / TILE)
    a = absmax.view(tr, tc).repeat_interleave(TILE, 0).repeat_interleave(TILE, 1)[:R, :C]
    scale = torch.where(a > 0, a / SIGNED_QMAX, torch.zeros_like(a))
    return q.to(F32) * scale


# ----------------------------------------------------------------------------------------------
# Semantics presets
# ----------------------------------------------------------------------------------------------

@dataclass(frozen=True)
class Semantics:
    name: str
    m_layout: str            # "fp32" | "tile" | "flat"
    vec_quant: bool          # factored row/col vectors stored as uint8 + absmax per 256
    guard_sq: str            # "none" | "fix" (mean<=0 -> 1) | "clamp" (1e-30 on mean, ratio, col)
    guard_res_row: str       # same vocabulary, for the residual row factor
    guard_res_col: str       # "none" | "clamp"
    wd_form: str             # "sub1" | "mul2" | "add2"
    m_for_update: str        # "fp32" | "requant"
    factor_order: str        # "g_r_c": (g*r)*c  |  "rc_g": (r*c)*g
    clip_form: str           # "kernel": max(1, sqrt(S/n)/thr) | "norm": norm(u)/sqrt(n)/thr clamp
    one_minus_in_double: bool  # 1-beta formed in double by Python (torch alpha=) vs in fp32 by the kernel


# came_pytorch/CAME.py:117-172 (no guards; weight decay and update as two in-place ops on p.data)
CAME = Semantics("came", "fp32", False, "none", "none", "none", "add2", "fp32", "rc_g", "norm", True)
# came_pytorch/CAMECUDA.py:275-326 (generic branch: clamp_min(1e-30) in _approx_sq_grad, CAMECUDA.py:67-71)
CUDAFP_GENERIC = Semantics("cudafp_generic", "fp32", False, "clamp_py", "clamp_py", "clamp", "add2", "fp32",
                           "rc_g", "norm", True)
# came_kernels.cu:5250-5413 with 524-593, 1436-1487, 2307-2342, 2487-2511 (CAMECUDA 2-D CUDA kernel path)
CUDAFP = Semantics("cudafp", "fp32", False, "clamp", "clamp", "clamp", "sub1", "fp32", "g_r_c", "kernel", False)
# came_kernels.cu:3598-4040 with 61-96, 198-243, 298-333, 596-619, 2584-2779, 3332-3366 (CAME8bit / CAME8bit2D)
TILE8 = Semantics("tile8", "tile", True, "fix", "fix", "none", "mul2", "requant", "g_r_c", "kernel", False)
# came_kernels.cu:4792-4876, 2246-2305, 4979-5043 (1285: clamp on res col), 2487-2511 (CAME8bitFull / Memory)
FLAT8 = Semantics("flat8", "flat", True, "fix", "fix", "clamp", "sub1", "fp32", "g_r_c", "kernel", False)
# came_pytorch/CAME8bitFull.py:1006-1075 (pure-PyTorch branch taken for CPU tensors)
FLAT8_CPU = Semantics("flat8_cpu", "flat", True, "clamp_py", "clamp_py", "clamp", "add2", "fp32", "rc_g", "norm", True)

PRESETS = {s.name: s for s in (CAME, CUDAFP_GENERIC, CUDAFP, TILE8, FLAT8, FLAT8_CPU)}


@dataclass
class Hyper:
    lr: float = 2e-4
    beta1: float = 0.9
    beta2: float = 0.999
    beta3: float = 0.9999
    eps0: float = 1e-30
    eps1: float = 1e-16
    clip_threshold: float = 1.0
    weight_decay: float = 0.0


# ----------------------------------------------------------------------------------------------
# State containers (same keys / dtypes / initial values as the reference's state dicts)
# ----------------------------------------------------------------------------------------------

def init_state(p: torch.Tensor, sem: Semantics) -> dict:
    shape = tuple(p.shape)
    st: dict = {}
    factored = p.dim() >= 2
    if sem.m_layout == "fp32":
        # CAME.py:97-112, CAMECUDA.py:83-100
        st["exp_avg"] = torch.zeros(shape, dtype=F32)
        if factored:
            rs, cs = shape[:-1], shape[:-2] + shape[-1:]      # CAMECUDA.py:93-98: row / column state shapes of an N-D tensor
            for k, n in (("exp_avg_sq_row", rs), ("exp_avg_sq_col", cs), ("exp_avg_res_row", rs), ("exp_avg_res_col", cs)):
                st[k] = torch.zeros(n, dtype=F32)
        else:
            st["exp_avg_sq"] = torch.zeros(shape, dtype=F32)
        return st
    if sem.m_layout == "tile" and factored and p.dim() == 2:
        # came8bit2d_state.py:33-55: tile absmax starts at ZERO, vector absmax at ONE
        R, C = shape
        st["exp_avg_q"] = torch.zeros(shape, dtype=torch.int8)
        st["exp_avg_absmax"] = torch.zeros(math.ceil(R / TILE) * math.ceil(C / TILE), dtype=F32)
    else:
        # blockwise_quantization.py:17-27: codes zero, absmax ONE
        st["exp_avg_q"] = torch.zeros(shape, dtype=torch.int8)
        st["exp_avg_absmax"] = torch.ones(num_blocks(p.numel()), dtype=F32)
    if factored:
        # CAME8bitFull.py:762-783: the vectors of an N-D tensor keep the leading dimensions and are quantised in
        # blocks of 256 over their flattened entries (a block may straddle matrices)
        rs, cs = shape[:-1], shape[:-2] + shape[-1:]
        for k, n in (("exp_avg_sq_row", rs), ("exp_avg_sq_col", cs), ("exp_avg_res_row", rs), ("exp_avg_res_col", cs)):
            st[k + "_q"] = torch.zeros(n, dtype=torch.uint8)
            st[k + "_absmax"] = torch.ones(num_blocks(math.prod(n)), dtype=F32)
    else:
        st["exp_avg_sq_q"] = torch.zeros(shape, dtype=torch.uint8)
        st["exp_avg_sq_absmax"] = torch.ones(num_blocks(p.numel()), dtype=F32)
    return st


def _load_vec(st: dict, key: str, sem: Semantics) -> torch.Tensor:
    if sem.vec_quant:
        return dequantize_blockwise(st[key + "_q"], st[key + "_absmax"], signed=False)
    return st[key]


def _store_vec(st: dict, key: str, v: torch.Tensor, sem: Semantics) -> None:
    if sem.vec_quant:
        q, a = quantize_blockwise(v, signed=False)
        st[key + "_q"], st[key + "_absmax"] = q, a
    else:
        st[key] = v


def _ema(old: torch.Tensor, new: torch.Tensor, beta: float, sem: Semantics) -> torch.Tensor:
    """(old * beta) + ((1 - beta) * new), all fp32 (came_kernels.cu:91, 546).  The Python branches
    form 1-beta in double and round the difference once (torch `alpha=1.0 - beta`)."""
    b = _f(beta)
    om = _f(1.0 - beta) if sem.one_minus_in_double else (_f(1.0) - b)
    return old * b + om * new


def _factor_row(v: torch.Tensor, guard: str) -> torch.Tensor:
    """Row factor; the mean runs over the rows of one matrix (the last dimension of the row state)."""
    n = v.shape[-1]
    if guard == "none":        # CAME.py:61-66
        return (v / v.mean(dim=-1, keepdim=True)).rsqrt()
    if guard == "clamp_py":    # CAMECUDA.py:67-69, CAME8bitFull.py:124-126: only the mean is clamped in Python
        return (v / v.mean(dim=-1, keepdim=True).clamp_min(1e-30)).rsqrt()
    mean = v.sum(dim=-1, keepdim=True) / n
    if guard == "fix":         # came_kernels.cu:319-320, 330
        mean = torch.where(mean > 0, mean, torch.ones_like(mean))
        return (v / mean).rsqrt()
    if guard == "clamp":       # came_kernels.cu:591-592
        mean = torch.clamp_min(mean, 1e-30)
        return torch.clamp_min(v / mean, 1e-30).rsqrt()
    raise ValueError(guard)


def _factor_col(v: torch.Tensor, guard: str) -> torch.Tensor:
    if guard == "none":        # came_kernels.cu:241, 2777; CAME.py:67
        return v.rsqrt()
    return torch.clamp_min(v, 1e-30).rsqrt()   # came_kernels.cu:577, 1285; CAMECUDA.py:70


def _apply(p: torch.Tensor, upd: torch.Tensor, hp: Hyper, sem: Semantics) -> torch.Tensor:
    """Parameter write-back in the three forms the reference uses; `upd` is fp32, p keeps its dtype."""
    lr, wd = hp.lr, hp.weight_decay
    if sem.wd_form == "add2":
        # CAME.py:166-172 / CAMECUDA.py:324-326: two in-place ops on p.data, each rounding to p.dtype
        out = p.clone()
        if wd != 0:
            out.add_(out, alpha=-wd * lr)
        if sem.name == "came":
            out.add_(-(upd * lr))          # CAME.py:171-172: update.mul_(lr); p.data.add_(-update)
        else:
            out.add_(upd, alpha=-lr)
        return out
    pv = p.to(F32)
    if sem.wd_form == "sub1":
        # came_kernels.cu:2505-2510: one rounding to T
        if wd != 0:
            pv = pv - (_f(wd) * _f(lr)) * pv
        pv = pv - _f(lr) * upd
        return pv.to(p.dtype)
    if sem.wd_form == "mul2":
        # came_kernels.cu:2678-2682 then 3363-3365: rounded to T after the decay, again after the update
        if wd != 0:
            pv = (pv * (_f(1.0) - _f(lr) * _f(wd))).to(p.dtype).to(F32)
        pv = pv - _f(lr) * upd
        return pv.to(p.dtype)
    raise ValueError(sem.wd_form)


def _clip(u0: torch.Tensor, hp: Hyper, sem: Semantics) -> torch.Tensor:
    n = u0.numel()
    if sem.clip_form == "norm":   # CAME.py:58-59, 139-141
        return (u0.norm(2) / (n ** 0.5) / hp.clip_threshold).clamp_(min=1.0)
    S = (u0 * u0).sum()           # came_kernels.cu:605-612
    return torch.clamp_min(torch.sqrt(S / _f(n)) / _f(hp.clip_threshold), 1.0)   # came_kernels.cu:2619-2620


# ----------------------------------------------------------------------------------------------
# One step, 2-D (factored) tensor
# ----------------------------------------------------------------------------------------------

def step_factored(p: torch.Tensor, g: torch.Tensor, st: dict, hp: Hyper, sem: Semantics) -> torch.Tensor:
    """One CAME step on a factored parameter; mutates `st`, returns the new parameter (dtype of p).  A tensor of more
    than two dimensions is a batch of [shape[-2], shape[-1]] matrices that share one RMS clip (over the whole tensor)
    and whose state vectors are quantised over their flattened entries (CAME.py:117-172, CAME8bitFull.py:1006-1075)."""
    R, C = p.shape[-2], p.shape[-1]
    gf = g.to(F32)

    # factored second moment (CAME.py:117-127; came_kernels.cu:61-96, 198-243, 298-333, 524-593)
    sq = gf * gf + _f(hp.eps0)
    a = sq.sum(dim=-1) / C
    b = sq.sum(dim=-2) / R
    vr = _ema(_load_vec(st, "exp_avg_sq_row", sem), a, hp.beta2, sem)
    vc = _ema(_load_vec(st, "exp_avg_sq_col", sem), b, hp.beta2, sem)
    r = _factor_row(vr, sem.guard_sq)                      # from the fresh fp32 values, not the codes
    c = _factor_col(vc, "none" if sem.guard_sq in ("none", "fix") else "clamp")
    _store_vec(st, "exp_avg_sq_row", vr, sem)
    _store_vec(st, "exp_avg_sq_col", vc, sem)

    # update, RMS clip, momentum (CAME.py:129-145; came_kernels.cu:596-619, 2619-2627, 2246-2342)
    if sem.factor_order == "g_r_c":
        u0 = (gf * r[..., :, None]) * c[..., None, :]
    else:
        u0 = (r[..., :, None] * c[..., None, :]) * gf
    u = u0 / _clip(u0, hp, sem)
    if sem.m_layout == "fp32":
        m_old = st["exp_avg"]
    elif sem.m_layout == "tile":
        m_old = dequantize_tile16(st["exp_avg_q"], st["exp_avg_absmax"])
    else:
        m_old = dequantize_blockwise(st["exp_avg_q"], st["exp_avg_absmax"], signed=True)
    m = _ema(m_old, u, hp.beta1, sem)

    # confidence / instability (CAME.py:147-162; came_kernels.cu:2631-2676, 2685-2779, 1124-1156, 1246-1287)
    diff = u - m
    res = diff * diff + _f(hp.eps1)
    rho = res.sum(dim=-1) / C
    kap = res.sum(dim=-2) / R
    Rr = _ema(_load_vec(st, "exp_avg_res_row", sem), rho, hp.beta3, sem)
    Rc = _ema(_load_vec(st, "exp_avg_res_col", sem), kap, hp.beta3, sem)
    rr = _factor_row(Rr, sem.guard_res_row)
    rc = _factor_col(Rc, sem.guard_res_col)
    _store_vec(st, "exp_avg_res_row", Rr, sem)
    _store_vec(st, "exp_avg_res_col", Rc, sem)

    # store momentum
    if sem.m_layout == "fp32":
        st["exp_avg"] = m
        m_used = m
    elif sem.m_layout == "tile":
        st["exp_avg_q"], st["exp_avg_absmax"] = quantize_tile16(m)
        m_used = dequantize_tile16(st["exp_avg_q"], st["exp_avg_absmax"]) if sem.m_for_update == "requant" else m
    else:
        st["exp_avg_q"], st["exp_avg_absmax"] = quantize_blockwise(m, signed=True)
        m_used = m

    # apply (CAME.py:160-172; came_kernels.cu:3332-3366, 2487-2511)
    if sem.factor_order == "g_r_c":
        upd = (m_used * rr[..., :, None]) * rc[..., None, :]
    else:
        upd = (rr[..., :, None] * rc[..., None, :]) * m_used
    return _apply(p, upd, hp, sem)


# ----------------------------------------------------------------------------------------------
# One step, 1-D (non-factored) tensor
# ----------------------------------------------------------------------------------------------

def step_nonfactored(p: torch.Tensor, g: torch.Tensor, st: dict, hp: Hyper, sem: Semantics,
                     *, update_f16: bool = False) -> torch.Tensor:
    """One CAME step on a 1-D parameter (no confidence term: CAME.py:132-143, 163-172).

    Which reference code a 1-D tensor reaches depends on the class, not only on the preset:
      * tile8 / flat8 -> the flat 8-bit kernels came_kernels.cu:1013-1066, 1489-1544 (CAME8bit.py:812-843
        sends 1-D CUDA tensors there too).  `update_f16`: the scratch carrying u between the two kernels
        is fp16 in CAME8bitMemory (came_kernels.cu:1069-1122, CAME8bitMemory.py:524-557).
      * cudafp -> seven torch ops, CAMECUDA.py:247-273 (Python scalars: 1-beta formed in double, two
        roundings of p, the clamp only inside the rsqrt).
      * came / cudafp_generic / flat8_cpu -> the pure-Python branches."""
    gf = g.to(F32)
    n = gf.numel()
    name = sem.name
    quant = sem.m_layout != "fp32"
    kernel_path = name in ("tile8", "flat8")
    ema_sem = FLAT8 if kernel_path else CAME            # only `one_minus_in_double` is read from it
    v_old = dequantize_blockwise(st["exp_avg_sq_q"], st["exp_avg_sq_absmax"], signed=False) if quant else st["exp_avg_sq"]
    v = _ema(v_old, gf * gf + _f(hp.eps0), hp.beta2, ema_sem)
    if name == "came":
        u0 = v.rsqrt() * gf                               # CAME.py:136-137
    elif name in ("cudafp_generic", "flat8_cpu"):
        v = v.clamp_min(1e-30)                            # CAMECUDA.py:305 / CAME8bitFull.py:1031: in place on the state
        u0 = v.rsqrt() * gf
    else:
        u0 = torch.clamp_min(v, 1e-30).rsqrt() * gf       # came_kernels.cu:1041, CAMECUDA.py:267
    if kernel_path:
        S = (u0 * u0).sum()                               # from the fp32 value, before any fp16 rounding
        clip = torch.clamp_min(torch.sqrt(S / _f(n)) / _f(hp.clip_threshold), 1.0)   # came_kernels.cu:1509-1510
    else:
        clip = (u0.norm(2) / (n ** 0.5) / hp.clip_threshold).clamp_(min=1.0)          # CAMECUDA.py:268
    if update_f16:
        u0 = u0.to(torch.float16).to(F32)
    u = u0 / clip
    m_old = dequantize_blockwise(st["exp_avg_q"], st["exp_avg_absmax"], signed=True) if quant else st["exp_avg"]
    m = _ema(m_old, u, hp.beta1, ema_sem)
    if quant:
        st["exp_avg_sq_q"], st["exp_avg_sq_absmax"] = quantize_blockwise(v, signed=False)
        st["exp_avg_q"], st["exp_avg_absmax"] = quantize_blockwise(m, signed=True)
    else:
        st["exp_avg_sq"], st["exp_avg"] = v, m
    # write-back: single rounding in the flat kernels (came_kernels.cu:1536-1541), two torch ops elsewhere
    if kernel_path:
        return _apply(p, m, hp, FLAT8)
    return _apply(p, m, hp, CAME if name == "came" else CUDAFP_GENERIC)


def step(p: torch.Tensor, g: torch.Tensor, st: dict, hp: Hyper, sem: Semantics, **kw) -> torch.Tensor:
    if p.dim() >= 2:
        if p.dim() > 2 and sem.m_layout == "tile":
            raise NotImplementedError("the tile layout holds 2-D tensors only (CAME8bit.py:216-223)")
        return step_factored(p, g, st, hp, sem)
    if p.dim() == 1:
        return step_nonfactored(p, g, st, hp, sem, **kw)
    raise NotImplementedError("oracle covers tensors of one or more dimensions")
