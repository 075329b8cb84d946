"""Host side of the step: turns optimizer state into the device-resident tensor table ("plan") of
libcame_b200 and issues one C call per step per device.

This is the replacement of the reference's extension shim (came_pytorch/came_cuda/__init__.py:131-1106,
25 keyword wrappers, one pybind call per tensor per kernel group).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import numpy as np
import torch

from . import _lib
from ._lib import CameHyper, CameTensorDesc

_DT = {torch.float32: _lib.DT_F32, torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise RuntimeError(f"came_b200 supports float32/float16/bfloat16 tensors, got {dt}") from None


@dataclass
class Entry:
    """One tensor of a step: the parameter/gradient views handed to the kernels and its state tensors."""
    p: torch.Tensor
    g: torch.Tensor
    mode: int
    flags: int
    group: int                      # index into the hyper array of the step
    m: torch.Tensor = None
    m_absmax: torch.Tensor = None
    sq_row: torch.Tensor = None
    sq_row_absmax: torch.Tensor = None
    sq_col: torch.Tensor = None
    sq_col_absmax: torch.Tensor = None
    res_row: torch.Tensor = None
    res_row_absmax: torch.Tensor = None
    res_col: torch.Tensor = None
    res_col_absmax: torch.Tensor = None
    keep: list = field(default_factory=list)   # temporaries that must outlive the step's kernels

    def structure_key(self):
        """Everything except the p / g addresses: a change here needs a new plan."""
        return (tuple(self.p.shape), self.p.dtype, self.g.dtype, self.mode, self.flags, self.group,
                self.m.data_ptr(), self.sq_row.data_ptr())


def _ptr(t):
    return None if t is None else t.data_ptr()


def make_hyper(lr, betas, eps, clip_threshold, weight_decay, *, python_scalars: bool, grad_scale: float = 1.0) -> CameHyper:
    """fp32 hyper-parameters of one param_group.

    python_scalars=False: 1-beta, lr*wd and 1-lr*wd are formed in fp32 from the fp32-rounded inputs, as the
    reference kernels do after the double->float casts of came_kernels.cu:6224-6231.
    python_scalars=True: formed in double and rounded once, as torch does for `alpha=1.0 - beta` and
    `alpha=-weight_decay * lr` on the reference's Python paths (CAME.py:122-172, CAMECUDA.py:262-273)."""
    f = np.float32
    b = [f(x) for x in betas]
    h = CameHyper()
    h.lr = f(lr)
    h.beta1, h.beta2, h.beta3 = b
    if python_scalars:
        h.om_beta1, h.om_beta2, h.om_beta3 = (f(1.0 - float(x)) for x in betas)
        h.wd_lr = f(float(weight_decay) * float(lr))
        h.decay_mul = f(1.0 - float(lr) * float(weight_decay))
    else:
        h.om_beta1, h.om_beta2, h.om_beta3 = (f(1.0) - x for x in b)
        h.wd_lr = f(weight_decay) * f(lr)
        h.decay_mul = f(1.0) - f(lr) * f(weight_decay)
    h.eps0, h.eps1 = f(eps[0]), f(eps[1])
    h.clip_threshold = f(clip_threshold)
    h.weight_decay = f(weight_decay)
    h.grad_scale = f(grad_scale)      # every gradient is multiplied by it as the kernels read it
    return h


class DevicePlan:
    """A came_plan_t and the workspace it lives in, for the tensors of one device."""

    def __init__(self, device: torch.device, entries: list):
        self.lib = _lib.load()
        self.device = device
        self.n = len(entries)
        self.structure = tuple(e.structure_key() for e in entries)
        self.addresses = tuple((e.p.data_ptr(), e.g.data_ptr()) for e in entries)
        descs = (CameTensorDesc * self.n)()
        for d, e in zip(descs, entries):
            if e.p.dim() < 1:
                raise NotImplementedError("came_b200 does not step 0-dimensional tensors")
            d.p, d.g = e.p.data_ptr(), e.g.data_ptr()
            d.m, d.m_absmax = _ptr(e.m), _ptr(e.m_absmax)
            d.sq_row, d.sq_row_absmax = _ptr(e.sq_row), _ptr(e.sq_row_absmax)
            d.sq_col, d.sq_col_absmax = _ptr(e.sq_col), _ptr(e.sq_col_absmax)
            d.res_row, d.res_row_absmax = _ptr(e.res_row), _ptr(e.res_row_absmax)
            d.res_col, d.res_col_absmax = _ptr(e.res_col), _ptr(e.res_col_absmax)
            if e.p.dim() == 1:
                d.rows, d.cols, d.batch = e.p.shape[0], 0, 0
            else:      # more than two dimensions: a batch of [shape[-2], shape[-1]] matrices
                d.rows, d.cols = e.p.shape[-2], e.p.shape[-1]
                d.batch = math.prod(e.p.shape[:-2]) if e.p.dim() > 2 else 0
            d.mode, d.flags, d.group = e.mode, e.flags, e.group
            d.p_dtype, d.g_dtype = dtype_code(e.p.dtype), dtype_code(e.g.dtype)
        nbytes = self.lib.came_b200_workspace_bytes(descs, self.n)
        if nbytes == 0:
            _lib.check(_lib.E_INVALID)
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.workspace_bytes = nbytes
        handle = C.c_void_p()
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            _lib.check(self.lib.came_b200_plan_create(descs, self.n, self.workspace.data_ptr(), nbytes, stream,
                                                      C.byref(handle)))
        self.handle = handle

    def repoint(self, entries: list) -> bool:
        """Refresh p / g addresses in place; False when the library asks for a new plan instead."""
        addresses = tuple((e.p.data_ptr(), e.g.data_ptr()) for e in entries)
        if addresses == self.addresses:
            return True
        g = (C.c_void_p * self.n)(*[a[1] for a in addresses])
        p = (C.c_void_p * self.n)(*[a[0] for a in addresses])
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            rc = self.lib.came_b200_plan_set_pointers(self.handle, g, p, self.n, stream)
        if rc == _lib.E_INVALID:
            return False
        _lib.check(rc)
        self.addresses = addresses
        return True

    def step(self, hypers: list) -> None:
        arr = (CameHyper * len(hypers))(*hypers)
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            _lib.check(self.lib.came_b200_step(self.handle, arr, len(hypers), stream))

    def set_push(self, local_base: int, local_bytes: int, peer_bases: list) -> None:
        """Push mode of the weight exchange: from the next step on, the kernels that apply the update also store the new
        parameters at the same offset of every peer buffer (addresses as mapped into this process)."""
        arr = (C.c_void_p * max(1, len(peer_bases)))(*peer_bases)
        _lib.check(self.lib.came_b200_plan_set_push(self.handle, local_base, local_bytes, arr, len(peer_bases)))

    def pushed(self) -> list:
        """Per tensor of the plan: True when the push mode delivers it."""
        flags = (C.c_int * self.n)()
        _lib.check(self.lib.came_b200_plan_pushed(self.handle, flags, self.n))
        return [bool(f) for f in flags]

    def set_hyper(self, hypers: list) -> None:
        """Rewrites the hyper-parameter records a captured step uploads at every replay (no stream work)."""
        arr = (CameHyper * len(hypers))(*hypers)
        _lib.check(self.lib.came_b200_plan_set_hyper(self.handle, arr, len(hypers)))

    @property
    def last_launches(self) -> int:
        return self.lib.came_b200_plan_last_launches(self.handle)

    def status(self) -> int:
        """Waits for the current stream and returns the plan's device status word (0 = fine)."""
        out = C.c_int(0)
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            _lib.check(self.lib.came_b200_plan_status(self.handle, stream, C.byref(out)))
        return out.value

    def set_timing(self, enable: bool) -> None:
        _lib.check(self.lib.came_b200_plan_set_timing(self.handle, int(enable)))

    def read_timing(self) -> dict:
        """{kernel name: (total ms, launches)} since the last read; waits for the recorded events."""
        ms = (C.c_float * _lib.KERNEL_COUNT)()
        n = (C.c_int * _lib.KERNEL_COUNT)()
        _lib.check(self.lib.came_b200_plan_read_timing(self.handle, ms, n))
        return {self.lib.came_b200_kernel_name(k).decode(): (float(ms[k]), int(n[k]))
                for k in range(_lib.KERNEL_COUNT) if n[k] > 0}

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.came_b200_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class StepEngine:
    """Keeps one DevicePlan per device alive across steps and rebuilds it only when the set of
    tensors, their state buffers or their alignment class changes."""

    def __init__(self):
        self.plans: dict = {}
        self.push = None      # (local_base, local_bytes, [peer bases]) applied to every plan that is (re)built

    def set_push(self, local_base: int, local_bytes: int, peer_bases: list) -> None:
        """Switches the push mode of the weight exchange on for the plans of this engine, present and future."""
        self.push = (int(local_base), int(local_bytes), [int(b) for b in peer_bases])
        for plan in self.plans.values():
            plan.set_push(*self.push)

    def invalidate(self) -> None:
        for plan in self.plans.values():
            plan.close()
        self.plans.clear()

    def prepare(self, entries: list) -> list:
        by_dev: dict = {}
        for e in entries:
            by_dev.setdefault(e.p.device, []).append(e)
        ready = []
        for dev, es in by_dev.items():
            plan = self.plans.get(dev)
            structure = tuple(e.structure_key() for e in es)
            if plan is None or plan.structure != structure or not plan.repoint(es):
                if plan is not None:
                    plan.close()
                plan = DevicePlan(dev, es)
                if self.push is not None:
                    plan.set_push(*self.push)
                self.plans[dev] = plan
            ready.append(plan)
        for dev in [d for d in self.plans if d not in by_dev]:
            self.plans.pop(dev).close()
        return ready

    def set_hyper(self, hypers: list) -> None:
        for plan in self.plans.values():
            plan.set_hyper(hypers)

    def step(self, entries: list, hypers: list) -> int:
        launches = 0
        for plan in self.prepare(entries):
            plan.step(hypers)
            launches += plan.last_launches
        return launches
