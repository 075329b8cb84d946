"""The workspace-free 1-D step (`came_b200_step_vector_noalloc`) against the regular entry point.

Some hosts cannot allocate device memory when they step -- the whole device belongs to their own arena, or the
step sits inside a fixed memory plan -- so they cannot supply the workspace `came_b200_plan_create` wants.  For
them the library keeps the 1-D step's block sums in a fixed device array of its own.  This test drives that entry
point through the C ABI next to the regular one (an optimizer class -> `came_b200_step`) on the same inputs, two
steps in a row (the second call meets whatever the first left in the shared array), and expects identical bytes.

The last case runs at the size limit (all 16 384 slots of the array).

It lives in a file that pytest collects last, so that a failure here cannot hide the results of the other tests.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

HYPER = dict(lr=2e-4, betas=(0.9, 0.95, 0.995), eps=(1e-30, 1e-16), clip_threshold=1.0, weight_decay=1e-2)


def _noalloc_step(lib, _lib, p, g, m, m_absmax, v, v_absmax, mode, flags, hyper):
    from came_b200.engine import dtype_code
    rc = lib.came_b200_step_vector_noalloc(
        p.data_ptr(), g.data_ptr(), m.data_ptr(), None if m_absmax is None else m_absmax.data_ptr(), v.data_ptr(),
        None if v_absmax is None else v_absmax.data_ptr(), p.numel(), mode, dtype_code(p.dtype), dtype_code(g.dtype),
        flags, C.byref(hyper), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc)


@pytest.mark.parametrize("cls_name,n,dtype", [("CAME8bitFull", 5000, torch.bfloat16), ("CAME8bitMemory", 70001, torch.float16),
                                              ("CAMECUDA", 300, torch.float32), ("CAME8bitFull", 1 << 22, torch.bfloat16)])
def test_noalloc_matches_regular_entry_point_two_steps_in_a_row(cls_name, n, dtype):
    import came_b200
    from came_b200 import _lib
    from came_b200.engine import make_hyper
    lib = _lib.load()
    torch.manual_seed(n)
    p_ref = torch.nn.Parameter((torch.randn(n, device="cuda") * 0.02).to(dtype))
    opt = getattr(came_b200, cls_name)([p_ref], **HYPER)
    _, flags, variant = opt._route(p_ref, p_ref, opt.param_groups[0])
    quant = cls_name != "CAMECUDA"
    p = p_ref.data.clone()
    if quant:
        m = torch.zeros(n, device="cuda", dtype=torch.int8)
        v = torch.zeros(n, device="cuda", dtype=torch.uint8)
        nb = (n + 255) // 256
        m_absmax, v_absmax = torch.ones(nb, device="cuda"), torch.ones(nb, device="cuda")
        mode = _lib.MODE_FLAT8
    else:
        m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        m_absmax = v_absmax = None
        mode = _lib.MODE_FP32
    hyper = make_hyper(HYPER["lr"], HYPER["betas"], HYPER["eps"], HYPER["clip_threshold"], HYPER["weight_decay"],
                       python_scalars=bool(variant))
    for step in range(2):
        g = (torch.randn(n, device="cuda") * 1e-3).to(dtype)
        p_ref.grad = g.clone()
        opt.step()                                                        # regular entry point (plan + workspace)
        _noalloc_step(lib, _lib, p, g, m, m_absmax, v, v_absmax, mode, flags, hyper)
        st = opt.state[p_ref]
        assert torch.equal(p, p_ref.data), (cls_name, step)
        if quant:
            assert torch.equal(m, st["exp_avg_q"]) and torch.equal(v, st["exp_avg_sq_q"]), (cls_name, step)
            assert torch.equal(m_absmax, st["exp_avg_absmax"]) and torch.equal(v_absmax, st["exp_avg_sq_absmax"])
        else:
            assert torch.equal(m, st["exp_avg"]) and torch.equal(v, st["exp_avg_sq"]), (cls_name, step)


def test_noalloc_rejects_oversized_tensors_without_touching_the_gpu():
    from came_b200 import _lib
    from came_b200.engine import make_hyper
    lib = _lib.load()
    hyper = make_hyper(1e-3, (0.9, 0.999, 0.9999), (1e-30, 1e-16), 1.0, 0.0, python_scalars=False)
    fake = 0x1000
    rc = lib.came_b200_step_vector_noalloc(fake, fake, fake, fake, fake, fake, _lib.NOALLOC_MAX_ELEMS + 1, _lib.MODE_FLAT8,
                                           _lib.DT_BF16, _lib.DT_BF16, 0, C.byref(hyper), None)
    assert rc == _lib.E_UNSUPPORTED
    assert b"CAME_B200_NOALLOC_MAX_ELEMS" in lib.came_b200_last_error()
