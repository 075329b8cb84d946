"""CPU-side checks: the C-ABI library loads and exports every symbol include/came_b200.h declares, its
validation rejects bad descriptors before touching a GPU, and the host-side optimizer logic (constructor
validation, state layouts, hyper-parameter rounding) mirrors the reference."""
import ctypes as C
import math
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from came_b200 import _lib
    lib = _lib.load()
    header = open(os.path.join(ROOT, "include", "came_b200.h")).read()
    declared = set(re.findall(r"\b(came_b200_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.came_b200_version() == 1


def test_struct_layout_matches_header():
    from came_b200 import _lib
    assert C.sizeof(_lib.CameTensorDesc) == 136
    assert _lib.CameTensorDesc.rows.offset == 96 and _lib.CameTensorDesc.flags.offset == 128
    assert C.sizeof(_lib.CameHyper) == 64


def _desc(**kw):
    from came_b200 import _lib
    d = _lib.CameTensorDesc()
    fake = 0x10000
    for f in ("p", "g", "m", "m_absmax", "sq_row", "sq_row_absmax", "sq_col", "sq_col_absmax", "res_row",
              "res_row_absmax", "res_col", "res_col_absmax"):
        setattr(d, f, fake)
        fake += 0x10000
    d.rows, d.cols, d.mode, d.p_dtype, d.g_dtype, d.group = 64, 64, _lib.MODE_TILE8, _lib.DT_BF16, _lib.DT_BF16, 0
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_validation_without_gpu():
    from came_b200 import _lib
    lib = _lib.load()
    arr = (_lib.CameTensorDesc * 1)(_desc())
    assert lib.came_b200_workspace_bytes(arr, 1) > 0
    for bad in (dict(rows=0), dict(p=None), dict(mode=7), dict(g_dtype=9), dict(group=64), dict(m_absmax=None),
                dict(cols=0, mode=_lib.MODE_TILE8), dict(res_col=None), dict(rows=1 << 31)):
        arr = (_lib.CameTensorDesc * 1)(_desc(**bad))
        assert lib.came_b200_workspace_bytes(arr, 1) == 0, bad
        assert lib.came_b200_last_error()
    handle = C.c_void_p()
    arr = (_lib.CameTensorDesc * 1)(_desc())
    rc = lib.came_b200_plan_create(arr, 1, None, 0, None, C.byref(handle))
    assert rc == _lib.E_WORKSPACE and not handle.value
    rc = lib.came_b200_plan_create(arr, 1, 0x1001, 1 << 30, None, C.byref(handle))   # misaligned
    assert rc == _lib.E_WORKSPACE
    rc = lib.came_b200_plan_create(arr, 1, 0x1000, 16, None, C.byref(handle))        # too small
    assert rc == _lib.E_WORKSPACE
    assert lib.came_b200_step(None, None, 1, None) == _lib.E_INVALID
    assert lib.came_b200_quantize_blockwise(None, None, None, 10, 1, None) == _lib.E_INVALID


def test_workspace_is_small_relative_to_the_tensors():
    from came_b200 import _lib
    lib = _lib.load()
    arr = (_lib.CameTensorDesc * 1)(_desc(rows=4096, cols=11008))
    ws = lib.came_b200_workspace_bytes(arr, 1)
    assert ws < 0.02 * 4096 * 11008 * 5      # < 2 % of p + g + m bytes


def test_make_hyper_rounding_variants():
    from came_b200.engine import make_hyper
    k = make_hyper(2e-4, (0.9, 0.999, 0.9999), (1e-30, 1e-16), 1.0, 1e-2, python_scalars=False)
    p = make_hyper(2e-4, (0.9, 0.999, 0.9999), (1e-30, 1e-16), 1.0, 1e-2, python_scalars=True)
    f = np.float32
    assert k.om_beta3 == f(1.0) - f(0.9999) and p.om_beta3 == f(1.0 - 0.9999) and k.om_beta3 != p.om_beta3
    assert k.wd_lr == f(1e-2) * f(2e-4) and p.wd_lr == f(1e-2 * 2e-4)
    assert k.decay_mul == f(1.0) - f(2e-4) * f(1e-2)
    assert k.eps0 == f(1e-30) and k.eps1 == f(1e-16)


def test_constructor_validation_mirrors_reference():
    import came_b200
    w = [torch.nn.Parameter(torch.zeros(4, 4))]
    for cls in (came_b200.CAMECUDA, came_b200.CAME8bit, came_b200.CAME8bitFull, came_b200.CAME8bitMemory,
                came_b200.CAME8bit2D):
        with pytest.raises(ValueError):
            cls(w, lr=0.0)
        with pytest.raises(ValueError):
            cls(w, lr=1e-3, clip_threshold=0.0)
        with pytest.raises(ValueError):
            cls(w, lr=1e-3, eps=(1e-30,))
        with pytest.raises(ValueError):
            cls(w, lr=1e-3, betas=(0.9, 0.99))
        opt = cls(w, lr=1e-3, weight_decay=0.1)
        g = opt.param_groups[0]
        assert g["lr"] == 1e-3 and g["weight_decay"] == 0.1 and g["betas"] == (0.9, 0.999, 0.9999)
        assert g["eps"] == (1e-30, 1e-16) and g["clip_threshold"] == 1.0
        assert opt.supports_memory_efficient_fp16 and not opt.supports_flat_params
    with pytest.raises(AssertionError):
        came_b200.CAME(w, lr=-1.0)
    with pytest.raises(ValueError):
        came_b200.CAMECUDA(w, lr=1e-3, betas=(0.9, 1.5, 0.9))
    with pytest.raises(ValueError):
        came_b200.CAME8bit(w, lr=1e-3, cuda_1d_runtime_mode="nope")
    with pytest.warns(RuntimeWarning):
        came_b200.CAME8bit(w, lr=1e-3, cuda_1d_batched_chunk_size=16)
    assert "block_size" in came_b200.CAME8bit(w, lr=1e-3).param_groups[0]


def test_state_layouts_match_reference_keys():
    from came_b200 import optim
    p = torch.zeros(40, 300)
    st = {}
    optim.init_state_tile(st, p)
    assert st["_mode"] == "8bit2d" and "step" not in st
    assert st["exp_avg_q"].dtype == torch.int8 and st["exp_avg_q"].shape == (40, 300)
    assert st["exp_avg_absmax"].shape == (math.ceil(40 / 16) * math.ceil(300 / 16),) and float(st["exp_avg_absmax"].sum()) == 0
    assert st["exp_avg_sq_col_q"].dtype == torch.uint8 and st["exp_avg_sq_col_absmax"].shape == (2,)
    assert float(st["exp_avg_res_row_absmax"][0]) == 1.0
    assert (st["rows"], st["cols"], st["tile_rows"], st["tile_cols"], st["num_tiles"]) == (40, 300, 3, 19, 57)
    st = {}
    optim.init_state_flat(st, p)
    assert st["_mode"] == "full8bit" and st["step"] == 0 and st["RMS"] == 0 and st["factored"]
    assert st["exp_avg_absmax"].shape == (math.ceil(40 * 300 / 256),) and float(st["exp_avg_absmax"][0]) == 1.0
    assert st["factored_row_q"].shape == (2, 40) and st["factored_col_absmax"].shape == (2, 2)
    assert st["exp_avg_res_col_q"].data_ptr() == st["factored_col_q"][1].data_ptr()
    st = {}
    optim.init_state_flat(st, torch.zeros(700))
    assert not st["factored"] and st["exp_avg_sq_q"].dtype == torch.uint8 and st["exp_avg_sq_absmax"].shape == (3,)
    st = {}
    optim.init_state_fp(st, p, mode_tag="cudafp")
    assert st["_mode"] == "cudafp" and st["exp_avg"].dtype == torch.float32 and st["exp_avg_sq_row"].shape == (40,)
    st = {}
    optim.init_state_fp(st, torch.zeros(9), mode_tag=None)
    assert "_mode" not in st and st["exp_avg_sq"].shape == (9,) and st["RMS"] == 0


def test_cpu_parameters_are_refused_not_silently_stepped():
    import came_b200
    p = torch.nn.Parameter(torch.zeros(8, 8))
    p.grad = torch.ones(8, 8)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        came_b200.CAMECUDA([p], lr=1e-3).step()
    s = torch.nn.Parameter(torch.zeros(8, 8))
    s.grad = torch.sparse_coo_tensor(torch.tensor([[0], [0]]), torch.tensor([1.0]), (8, 8))
    with pytest.raises(RuntimeError, match="sparse"):
        came_b200.CAME8bit([s], lr=1e-3).step()


def test_work_list_never_overflows():
    """plan_create sizes the work lists from the descriptors before it builds them; the two counts must agree for
    every shape class (staged / generic kernels, fused / two-pass first pass, every layout).  With fake pointers
    and no GPU the call gets past the work lists and fails at its first CUDA call."""
    from came_b200 import _lib
    lib = _lib.load()
    shapes = [(4096, 32768), (128, 32000), (64, 20480), (1, 64), (130, 16448), (257, 8192), (100, 100),
              (4096, 11008), (32000, 4096), (300, 72), (16, 65536 + 64), (5, 7), (2048, 256), (1000, 0), (70001, 0)]
    ws = 1 << 40
    for rows, cols in shapes:
        for mode, flags in ((_lib.MODE_TILE8, 0), (_lib.MODE_FLAT8, 0), (_lib.MODE_FP32, _lib.F_SQ_CLAMP),
                            (_lib.MODE_TILE8, _lib.F_SQ_CLAMP)):
            if cols == 0 and mode == _lib.MODE_TILE8:
                continue
            for dt in (_lib.DT_BF16, _lib.DT_F32):
                arr = (_lib.CameTensorDesc * 1)(_desc(rows=rows, cols=cols, mode=mode, flags=flags, p_dtype=dt, g_dtype=dt))
                handle = C.c_void_p()
                rc = lib.came_b200_plan_create(arr, 1, 0x10000000, ws, None, C.byref(handle))
                msg = lib.came_b200_last_error().decode()
                assert "overflow" not in msg, (rows, cols, mode, flags, dt, msg)
                if rc == _lib.OK:
                    lib.came_b200_plan_destroy(handle)
