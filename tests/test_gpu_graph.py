"""CUDA-graph capture of the step (reference: prime_for_cuda_graph / cuda_graph_compatible,
came_pytorch/CAME8bit2D.py:52-72, came_pytorch/CAME8bit.py:672-693): a captured step replayed with fresh
gradients and a changing learning rate must leave exactly the bytes the eager step leaves."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(256, 512), (384, 1024), (128, 192), (4096,), (300,)]


def _make(cls_name, dtype, **kw):
    import came_b200
    torch.manual_seed(5)
    ps = [torch.nn.Parameter((torch.randn(s, device="cuda") * 0.02).to(dtype)) for s in SHAPES]
    for p in ps:
        p.grad = torch.zeros_like(p)
    return ps, getattr(came_b200, cls_name)(ps, lr=1e-3, weight_decay=1e-2, **kw)


@pytest.mark.parametrize("cls_name,dtype,kw", [
    ("CAME8bit", torch.bfloat16, {"cuda_graph_compatible": True}),
    ("CAME8bitMemory", torch.bfloat16, {}),
    ("CAMECUDA", torch.float32, {}),
])
def test_captured_step_equals_eager(cls_name, dtype, kw):
    steps = 5
    gen = torch.Generator(device="cuda").manual_seed(9)
    grads = [[(torch.randn(s, device="cuda", generator=gen) * 1e-2).to(dtype) for s in SHAPES] for _ in range(steps)]
    lrs = [1e-3 * (0.5 ** k) for k in range(steps)]

    # eager
    pe, oe = _make(cls_name, dtype, **kw)
    for k in range(steps):
        for p, g in zip(pe, grads[k]):
            p.grad.copy_(g)
        for grp in oe.param_groups:
            grp["lr"] = lrs[k]
        oe.step()

    # captured once, replayed: gradients go into the static .grad buffers, lr through update_captured_hypers
    pg, og = _make(cls_name, dtype, **kw)
    og.prime_for_cuda_graph()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    for p, g in zip(pg, grads[0]):
        p.grad.copy_(g)
    for grp in og.param_groups:
        grp["lr"] = lrs[0]
    torch.cuda.synchronize()
    with torch.cuda.graph(graph, stream=side):
        og.step()
    # capture records, it does not run: parameters are still the initial ones
    for k in range(steps):
        for p, g in zip(pg, grads[k]):
            p.grad.copy_(g)
        for grp in og.param_groups:
            grp["lr"] = lrs[k]
        og.update_captured_hypers()
        graph.replay()
        torch.cuda.synchronize()
    for a, b in zip(pe, pg):
        assert torch.equal(a.data, b.data)
    for a, b in zip(pe, pg):
        sa, sb = oe.state[a], og.state[b]
        for key, va in sa.items():
            if torch.is_tensor(va):
                assert torch.equal(va, sb[key]), key
    for plan in og._engine.plans.values():
        assert plan.status() == 0


def test_set_hyper_rejects_bad_records():
    import came_b200
    from came_b200 import _lib
    ps, opt = _make("CAME8bit", torch.bfloat16)
    opt.step()
    plan = next(iter(opt._engine.plans.values()))
    bad = _lib.CameHyper()
    with pytest.raises(_lib.CameError):
        plan.set_hyper([bad, bad])      # clip_threshold 0


def test_bounded_wait_runs_out_cleanly():
    """A wait inside the kernels that never completes must end by itself: status word 1, both warps back, and the
    context still usable afterwards (a normal step right after)."""
    import came_b200
    from came_b200 import _lib
    lib = _lib.load()
    words = torch.full((3,), 7, device="cuda", dtype=torch.int32)
    _lib.check(lib.came_b200_selftest_bounded_wait(words.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert words.tolist() == [1, 0, 0]
    p = torch.nn.Parameter(torch.ones(64, 64, device="cuda"))
    p.grad = torch.ones(64, 64, device="cuda")
    opt = came_b200.CAME8bit([p], lr=1e-3)
    opt.step()
    assert all(plan.status() == 0 for plan in opt._engine.plans.values())
    assert bool((p.data < 1.0).all())
