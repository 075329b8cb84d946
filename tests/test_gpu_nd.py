"""Tensors of more than two dimensions on the GPU against the CPU oracle (pinned on such tensors by the reference's own
CPU trajectories, tests/golden/traj_*_nd_*.npz): a batch of [shape[-2], shape[-1]] matrices with one RMS clip over
the whole tensor and state vectors quantised in blocks of 256 across the matrices.  In the reference these tensors
take the classes' generic torch paths (came_pytorch/CAME8bitFull.py:1006-1075, CAMECUDA.py:275-326, CAME.py:117-172),
whose arithmetic the presets FLAT8_CPU / CUDAFP_GENERIC / CAME restate.  Tolerances as in tests/test_gpu_parity.py."""
import pytest
import torch

from oracle import came_oracle as orc
from tests.parity_util import run_pair
from tests.test_gpu_parity import H_DEFAULT, H_LLAMA, _check_8bit, _check_fp, _dt

pytestmark = pytest.mark.gpu

# a conv weight as the task's example names it, tiny and ragged batches, stacked larger matrices, plus 2-D / 1-D company
ND_SHAPES = [(64, 32, 3, 3), (12, 5, 3, 3), (3, 40, 24), (2, 3, 17, 9), (5, 300, 20), (2, 130, 272), (96, 64), (300,)]


def _status_ok(opt):
    for plan in opt._engine.plans.values():
        assert plan.status() == 0


@pytest.mark.parametrize("cls_name,f16", [("CAME8bitFull", False), ("CAME8bit", False), ("CAME8bitMemory", True)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
def test_8bit_classes_step_nd_tensors(cls_name, f16, dtype):
    import came_b200
    two_d = orc.TILE8 if cls_name == "CAME8bit" else orc.FLAT8
    preset = lambda dim: orc.FLAT8_CPU if dim > 2 else (two_d if dim == 2 else orc.FLAT8)
    out, opt, gp = run_pair(getattr(came_b200, cls_name), preset, ND_SHAPES, _dt(dtype), 6, H_LLAMA, seed=51,
                            oracle_kw=dict(update_f16=f16))
    _check_8bit(out, _dt(dtype))
    _status_ok(opt)
    st = opt.state[gp[0]]
    assert st["_mode"] == "full8bit" and st["exp_avg_q"].shape == (64, 32, 3, 3)
    assert st["factored_row_q"].shape == (2, 64, 32, 3) and st["factored_col_absmax"].shape == (2, 24)


@pytest.mark.parametrize("cls_name,preset_nd,preset_2d", [("CAMECUDA", "CUDAFP_GENERIC", "CUDAFP"), ("CAME", "CAME", "CAME")])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_fp32_state_classes_step_nd_tensors(cls_name, preset_nd, preset_2d, dtype):
    import came_b200
    preset = lambda dim: getattr(orc, preset_nd) if dim > 2 else getattr(orc, preset_2d)
    out, opt, gp = run_pair(getattr(came_b200, cls_name), preset, ND_SHAPES, _dt(dtype), 6, H_DEFAULT, seed=52)
    _check_fp(out, _dt(dtype))
    _status_ok(opt)
    assert opt.state[gp[0]]["exp_avg_sq_col"].shape == (64, 32, 3)


def test_came8bit2d_still_refuses_nd():
    import came_b200
    p = torch.nn.Parameter(torch.zeros(2, 4, 4, device="cuda"))
    p.grad = torch.zeros(2, 4, 4, device="cuda")
    with pytest.raises(NotImplementedError):
        came_b200.CAME8bit2D([p], lr=1e-3).step()
