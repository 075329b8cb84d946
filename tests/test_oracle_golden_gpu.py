"""Pins the oracle presets that restate the reference's CUDA kernels (TILE8, FLAT8, CUDAFP) to outputs of those
kernels themselves: fixtures tests/golden/traj_gpu_*.npz, produced on a B200 by tests/golden/make_golden_gpu.py from
the reference's extension compiled for sm_100 (oracle/build_ref.py).

Tolerance.  The reference builds with --use_fast_math (approximate division / rsqrt, flush to zero), so agreement is
stated, not bit-exact: fp32 parameters to 1e-6 relative Frobenius error per step, 16-bit parameters equal except
<= 1e-4 of the entries (or two entries of a short vector), each by at most one spacing; 8-bit codes equal except
as many entries, each by one step; fp32 states and absmax to 1e-5.  Measured when the fixtures were made: 1e-7 on fp32 parameters, identical
16-bit parameters and codes on the small cases, 2e-5 of the codes off by one at 4096 / 11008 columns."""
import os

import numpy as np
import pytest
import torch

from oracle import came_oracle as orc
from tests.golden.make_golden import golden_inputs
from tests.golden.make_golden_gpu import PRESETS_GPU, cases_of

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# fixture preset -> (oracle preset of 2-D tensors, of 1-D tensors, fp16 update of 1-D tensors)
ORACLE_OF = {
    "tile8": (orc.TILE8, orc.FLAT8, False),       # came2d_step; CAME8bit's 1-D tensors take the flat kernels
    "flat8": (orc.FLAT8, orc.FLAT8, False),       # came_full_factored_* / came_full_nonfactored_step
    "flat8mem": (orc.FLAT8, orc.FLAT8, True),     # came_full_nonfactored_step_fp16_update
    "cudafp": (orc.CUDAFP, None, False),          # came_fp_factored_step
}
ALL = [(p, c) for p in PRESETS_GPU for c in cases_of(p)]


def _unbits(a: np.ndarray, dtype: str) -> torch.Tensor:
    t = torch.from_numpy(a)
    return t.view(torch.bfloat16) if (dtype == "bfloat16" and a.dtype == np.int16) else t


@pytest.mark.parametrize("preset,case_name", ALL)
def test_cuda_presets_match_reference_kernels(preset, case_name):
    case = cases_of(preset)[case_name]
    sem2, sem1, f16 = ORACLE_OF[preset]
    gold = np.load(os.path.join(GOLD, f"traj_gpu_{preset}_{case_name}.npz"))
    h = case["hyper"]
    hp = orc.Hyper(lr=h["lr"], beta1=h["betas"][0], beta2=h["betas"][1], beta3=h["betas"][2], eps0=h["eps"][0],
                   eps1=h["eps"][1], clip_threshold=h["clip_threshold"], weight_decay=h["weight_decay"])
    params, grads = golden_inputs(case)
    keep = [i for i, p in enumerate(params) if p.dim() == 2 or sem1 is not None]
    sems = {i: (sem2 if params[i].dim() == 2 else sem1) for i in keep}
    states = {i: orc.init_state(params[i], sems[i]) for i in keep}
    compared = 0
    for s, gs in enumerate(grads):
        for i in keep:
            kw = dict(update_f16=f16) if params[i].dim() == 1 else {}
            params[i] = orc.step(params[i], gs[i], states[i], hp, sems[i], **kw)
            key = f"p{i}.step{s}"
            if key not in gold.files:
                continue
            compared += 1
            ref, got = _unbits(gold[key], case["dtype"]).float(), params[i].float()
            if case["dtype"] == "float32":
                err = ((got - ref).norm() / ref.norm().clamp_min(1e-30)).item()
                assert err <= 1e-6, (key, err)
            else:
                # an entry that cancels to ~0 has no meaningful spacing of its own: floor at a tenth of a typical update
                spacing = (ref.abs() * 2.0 ** -7).clamp_min(0.1 * h["lr"])
                assert ((got - ref).abs() <= spacing).all(), key
                assert int((got != ref).sum()) <= max(2, 1e-4 * got.numel()), key
    assert compared > 0
    for i in keep:
        for k, v in states[i].items():
            key = f"state{i}.{k}"
            assert key in gold.files, key
            ref = torch.from_numpy(gold[key])
            if v.dtype in (torch.int8, torch.uint8):
                d = (v.to(torch.int32) - ref.to(torch.int32)).abs()
                assert d.max().item() <= 1 and int((d != 0).sum()) <= max(2, 1e-4 * d.numel()), (key, int((d != 0).sum()))
            else:
                err = ((v - ref).norm() / ref.norm().clamp_min(1e-30)).item()
                assert err <= 1e-5, (key, err)
