"""The fused momentum / apply kernel against the three separate passes: the two schedules run the same arithmetic
item by item, so every parameter and state byte must be identical.  (The separate passes are compared with the CPU
oracle in tests/test_gpu_parity.py and tests/test_gpu_bench_shapes.py; the fused kernel is the default there too.)"""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

H = dict(lr=2e-4, eps=(1e-30, 1e-16), clip_threshold=1.0, betas=(0.9, 0.95, 0.995), weight_decay=1e-2)
# many tensors, more items than CTAs, ragged tile widths and row counts, a vector in between
SHAPES = [(4096, 1024), (130, 11008), (257, 5632), (1024, 4096), (4096,), (2048, 2304), (640, 64), (384, 8192),
          (16, 1024), (1000, 1088), (3000, 1024)]


def _run(fused: bool, dtype, steps=3, wd=1e-2, cls_name="CAME8bit"):
    import came_b200
    os.environ["CAME_B200_FUSED_MA"] = "1" if fused else "0"      # read when the plan is created
    try:
        gen = torch.Generator(device="cuda").manual_seed(3)
        params = [torch.nn.Parameter((torch.randn(s, device="cuda", generator=gen) * 0.02).to(dtype)) for s in SHAPES]
        opt = getattr(came_b200, cls_name)(params, **dict(H, weight_decay=wd))
        for k in range(steps):
            for i, p in enumerate(params):
                p.grad = (torch.randn(p.shape, device="cuda", generator=gen) * 10.0 ** (-2 - (i % 4))).to(dtype)
            opt.step()
        for plan in opt._engine.plans.values():
            assert plan.status() == 0
        out = [p.data.clone() for p in params]
        for p in params:
            out += [v.clone() for k, v in sorted(opt.state[p].items()) if torch.is_tensor(v)]
        return out, opt.last_step_launches
    finally:
        os.environ.pop("CAME_B200_FUSED_MA", None)


@pytest.mark.parametrize("cls_name", ["CAME8bit", "CAME8bitFull"])      # tile layout, flat layout
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("wd", [1e-2, 0.0])
def test_fused_equals_separate_passes(cls_name, dtype, wd):
    a, la = _run(True, dtype, wd=wd, cls_name=cls_name)
    b, lb = _run(False, dtype, wd=wd, cls_name=cls_name)
    assert la < lb                      # one launch instead of three
    assert len(a) == len(b)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
