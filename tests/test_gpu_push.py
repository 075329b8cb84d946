"""Push mode of the weight exchange on ONE GPU: the "peer" is a second buffer of the same device, so the stores the
apply kernel adds can be checked without a second process.  After a step the mirror must hold exactly the new values
of every tensor the plan reports as pushed, and nothing else; bad set-ups are refused on the host.  (Two ranks on two
GPUs: tests/test_gpu_peer_gather.py.)  No counterpart in the reference, which is single-GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(256, 1024), (4096,), (130, 2304), (64, 192), (300,), (129, 1088)]


def _setup(cls_name, dtype):
    import came_b200
    dev = torch.device("cuda", 0)
    sizes = [((torch.Size(s).numel() + 127) // 128) * 128 for s in SHAPES]
    flat = torch.zeros(sum(sizes), dtype=dtype, device=dev)
    gen = torch.Generator(device=dev).manual_seed(11)
    flat.copy_((torch.randn(flat.shape, generator=gen, device=dev) * 0.02).to(dtype))
    views, off = [], 0
    for s, n in zip(SHAPES, sizes):
        views.append(flat[off:off + torch.Size(s).numel()].view(s))
        off += n
    params = [torch.nn.Parameter(v) for v in views]
    for i, p in enumerate(params):
        p.grad = (torch.randn(p.shape, generator=gen, device=dev) * 10.0 ** (-2 - i % 3)).to(dtype)
    opt = getattr(came_b200, cls_name)(params, lr=1e-3, weight_decay=1e-2)
    opt.prime_for_cuda_graph()
    return flat, params, opt


@pytest.mark.parametrize("cls_name,dtype", [("CAME8bit", torch.bfloat16), ("CAME8bit", torch.float32),
                                            ("CAME8bitFull", torch.bfloat16)])
def test_mirror_receives_exactly_the_pushed_tensors(cls_name, dtype):
    flat, params, opt = _setup(cls_name, dtype)
    mirrors = [torch.zeros_like(flat) for _ in range(2)]
    nbytes = flat.numel() * flat.element_size()
    opt._engine.set_push(flat.data_ptr(), nbytes, [m.data_ptr() for m in mirrors])
    (plan,) = opt._engine.plans.values()
    pushed = plan.pushed()
    assert any(pushed) and not all(pushed)          # the matrices on the staged path, not the vectors / odd widths
    for _ in range(2):
        opt.step()
    torch.cuda.synchronize()
    assert plan.status() == 0
    base = flat.data_ptr()
    for p, flag in zip(params, pushed):
        lo = (p.data_ptr() - base) // flat.element_size()
        for m in mirrors:
            got = m[lo:lo + p.numel()].view(p.shape)
            if flag:
                assert torch.equal(got, p.data)
            else:
                assert not got.any()
    # switching the mode off stops the stores
    opt._engine.set_push(flat.data_ptr(), nbytes, [])
    before = [m.clone() for m in mirrors]
    opt.step()
    torch.cuda.synchronize()
    for m, b in zip(mirrors, before):
        assert torch.equal(m, b)


def test_bad_push_setups_are_refused():
    flat, params, opt = _setup("CAME8bit", torch.bfloat16)
    (plan,) = opt._engine.plans.values()
    nbytes = flat.numel() * flat.element_size()
    other = torch.zeros_like(flat)
    with pytest.raises(Exception):      # more peers than the kernels serve
        plan.set_push(flat.data_ptr(), nbytes, [other.data_ptr()] * 8)
    with pytest.raises(Exception):      # a pushed tensor outside the local buffer
        plan.set_push(flat.data_ptr(), 1024, [other.data_ptr()])
    with pytest.raises(Exception):      # a peer buffer that overlaps the local one
        plan.set_push(flat.data_ptr(), nbytes, [flat.data_ptr() + 256])
    with pytest.raises(Exception):      # a misaligned peer buffer
        plan.set_push(flat.data_ptr(), nbytes, [other.data_ptr() + 2])
    opt.step()                          # none of the refused calls left the plan in push mode
    torch.cuda.synchronize()
    assert plan.status() == 0 and not other.any()
