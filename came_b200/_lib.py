"""ctypes binding of libcame_b200.so (the C ABI declared in include/came_b200.h).

The library is the product path: if it is missing the import fails loudly.  There is no eager /
PyTorch / CPU fallback anywhere in this package.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libcame_b200.so")

DT_F32, DT_F16, DT_BF16 = 0, 1, 2
MODE_FP32, MODE_TILE8, MODE_FLAT8 = 0, 1, 2

F_SQ_FIX = 1 << 0
F_SQ_CLAMP = 1 << 1
F_RESROW_FIX = 1 << 2
F_RESROW_CLAMP = 1 << 3
F_RESCOL_CLAMP = 1 << 4
F_WD_MUL2 = 1 << 5
F_WD_ADD2 = 1 << 6
F_UPDATE_F16 = 1 << 7
F_RSQRT_CLAMP = 1 << 8

MAX_GROUPS = 64
KERNEL_COUNT = 20
NOALLOC_MAX_ELEMS = 1 << 22
OK, E_INVALID, E_WORKSPACE, E_CUDA, E_UNSUPPORTED = 0, -1, -2, -3, -4


class CameTensorDesc(C.Structure):
    _fields_ = [
        ("p", C.c_void_p), ("g", C.c_void_p), ("m", C.c_void_p), ("m_absmax", C.c_void_p),
        ("sq_row", C.c_void_p), ("sq_row_absmax", C.c_void_p),
        ("sq_col", C.c_void_p), ("sq_col_absmax", C.c_void_p),
        ("res_row", C.c_void_p), ("res_row_absmax", C.c_void_p),
        ("res_col", C.c_void_p), ("res_col_absmax", C.c_void_p),
        ("rows", C.c_int64), ("cols", C.c_int64),
        ("mode", C.c_int32), ("p_dtype", C.c_int32), ("g_dtype", C.c_int32), ("group", C.c_int32),
        ("flags", C.c_uint32), ("batch", C.c_uint32),
    ]


class CameHyper(C.Structure):
    _fields_ = [
        ("lr", C.c_float),
        ("beta1", C.c_float), ("beta2", C.c_float), ("beta3", C.c_float),
        ("om_beta1", C.c_float), ("om_beta2", C.c_float), ("om_beta3", C.c_float),
        ("eps0", C.c_float), ("eps1", C.c_float),
        ("clip_threshold", C.c_float),
        ("weight_decay", C.c_float), ("wd_lr", C.c_float), ("decay_mul", C.c_float),
        ("grad_scale", C.c_float), ("reserved", C.c_float * 2),
    ]


assert C.sizeof(CameTensorDesc) == 136 and C.sizeof(CameHyper) == 64

# name -> (restype, argtypes); every symbol include/came_b200.h declares
SYMBOLS = {
    "came_b200_version": (C.c_int, []),
    "came_b200_last_error": (C.c_char_p, []),
    "came_b200_quantize_blockwise": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "came_b200_dequantize_blockwise": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "came_b200_quantize_tile16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "came_b200_dequantize_tile16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "came_b200_workspace_bytes": (C.c_size_t, [C.POINTER(CameTensorDesc), C.c_int]),
    "came_b200_plan_create": (C.c_int, [C.POINTER(CameTensorDesc), C.c_int, C.c_void_p, C.c_size_t, C.c_void_p,
                                         C.POINTER(C.c_void_p)]),
    "came_b200_plan_destroy": (None, [C.c_void_p]),
    "came_b200_plan_set_pointers": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int,
                                               C.c_void_p]),
    "came_b200_step": (C.c_int, [C.c_void_p, C.POINTER(CameHyper), C.c_int, C.c_void_p]),
    "came_b200_plan_set_hyper": (C.c_int, [C.c_void_p, C.POINTER(CameHyper), C.c_int]),
    "came_b200_peer_copy_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "came_b200_ipc_export": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64)]),
    "came_b200_ipc_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "came_b200_ipc_close": (C.c_int, [C.c_void_p]),
    "came_b200_plan_set_push": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_int]),
    "came_b200_plan_pushed": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.c_int]),
    "came_b200_plan_last_launches": (C.c_int, [C.c_void_p]),
    "came_b200_plan_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]),
    "came_b200_selftest_bounded_wait": (C.c_int, [C.c_void_p, C.c_void_p]),
    "came_b200_plan_set_timing": (C.c_int, [C.c_void_p, C.c_int]),
    "came_b200_plan_read_timing": (C.c_int, [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "came_b200_kernel_name": (C.c_char_p, [C.c_int]),
    "came_b200_step_vector_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                C.c_int64, C.c_int, C.c_int, C.c_int, C.c_uint32, C.POINTER(CameHyper),
                                                C.c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library (once).  Raises ImportError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python came_b200/_build.py` (needs nvcc, sm_100a). "
            "came_b200 has no fallback path."
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)   # AttributeError if the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    if lib.came_b200_version() != 1:
        raise ImportError(f"{LIB_PATH}: ABI version {lib.came_b200_version()}, this package expects 1")
    _lib = lib
    return lib


class CameError(RuntimeError):
    """A non-zero status from the C ABI (message from came_b200_last_error)."""


def check(rc: int) -> None:
    if rc != OK:
        msg = load().came_b200_last_error()
        raise CameError(f"came_b200 error {rc}: {msg.decode() if msg else ''}")
