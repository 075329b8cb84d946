"""GPU parity: every optimizer class of came_b200, through the C ABI, against the CPU oracle on the same
seeded inputs.  Tolerances (stated per test): codec outputs are bit-exact; fp32-state trajectories agree
to 1e-5 relative Frobenius error on parameters and 1e-4 on states; 8-bit trajectories agree to 1e-3 on
parameters (bf16: never more than 2 ulp apart), 1e-3 on absmax, codes equal except <= 1 % of entries,
each by +-1 (one flipped code is 0.8 % of a block's range; the noise floor is the order of fp32
summation, which differs between any two implementations)."""
import os

import numpy as np
import pytest
import torch

from oracle import came_oracle as orc
from tests.golden.make_golden import codec_inputs
from tests.parity_util import run_pair

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
H_DEFAULT = dict(lr=2e-4, eps=(1e-30, 1e-16), clip_threshold=1.0, betas=(0.9, 0.999, 0.9999), weight_decay=1e-2)
H_LLAMA = dict(lr=2e-4, eps=(1e-30, 1e-16), clip_threshold=1.0, betas=(0.9, 0.95, 0.995), weight_decay=1e-2)
H_NOWD = dict(H_DEFAULT, weight_decay=0.0)

EDGE_SHAPES = [(1, 40), (40, 1), (15, 17), (16, 16), (17, 255), (255, 257), (256, 256), (257, 16), (1,), (255,),
               (256,), (257,), (700,)]
ALIGNED_SHAPES = [(256, 512), (128, 1024), (384, 272), (64, 48), (300, 256), (17, 768), (135, 1280), (4096,), (300,)]


def _dt(name):
    return getattr(torch, name)


# ---------------------------------------------------------------------------------------------
# codec: bit-exact
# ---------------------------------------------------------------------------------------------

def test_codec_bit_exact_vs_reference_fixture():
    from came_b200 import quant
    gold = np.load(os.path.join(GOLD, "codec.npz"))
    for name, x in codec_inputs().items():
        xt = torch.from_numpy(x).cuda()
        for signed in (True, False):
            tag = f"{name}.{'i8' if signed else 'u8'}"
            q, a = quant.quantize_blockwise(xt, signed=signed)
            assert np.array_equal(q.cpu().numpy(), gold[tag + ".q"]), tag
            assert np.array_equal(a.cpu().numpy().view(np.int32), gold[tag + ".absmax"].view(np.int32)), tag
            d = quant.dequantize_blockwise(q, a, signed=signed)
            assert np.array_equal(d.cpu().numpy().view(np.int32), gold[tag + ".deq"].view(np.int32)), tag


@pytest.mark.parametrize("n", [1, 255, 256, 257, 65536 + 3, 1 << 20])
@pytest.mark.parametrize("scale", [1e-3, 1e-20, 1e10])
def test_codec_bit_exact_vs_oracle(n, scale):
    from came_b200 import quant
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=g) * scale
    x[::97] = 0.0
    for signed in (True, False):
        src = x if signed else x.abs()
        q, a = quant.quantize_blockwise(src.cuda(), signed=signed)
        qo, ao = orc.quantize_blockwise(src, signed=signed)
        assert torch.equal(q.cpu(), qo)
        assert torch.equal(a.cpu().view(torch.int32), ao.view(torch.int32))
        d = quant.dequantize_blockwise(q, a, signed=signed)
        assert torch.equal(d.cpu().view(torch.int32), orc.dequantize_blockwise(qo, ao, signed=signed).view(torch.int32))


@pytest.mark.parametrize("shape", [(16, 16), (17, 33), (1, 5), (256, 272), (100, 1)])
def test_tile_codec_bit_exact_vs_oracle(shape):
    from came_b200 import quant
    g = torch.Generator().manual_seed(shape[0] * 1000 + shape[1])
    x = torch.randn(shape, generator=g) * 1e-2
    x[: shape[0] // 2, : min(16, shape[1])] = 0.0     # an all-zero tile when the shape allows
    q, a = quant.quantize_tile16(x.cuda())
    qo, ao = orc.quantize_tile16(x)
    assert torch.equal(q.cpu(), qo)
    assert torch.equal(a.cpu().view(torch.int32), ao.view(torch.int32))
    d = quant.dequantize_tile16(q, a)
    assert torch.equal(d.cpu().view(torch.int32), orc.dequantize_tile16(qo, ao).view(torch.int32))


def test_codec_roundtrip_full_size():
    """Size-independent property at a BASELINE-sized tensor (4096 x 11008): |deq(quant(x)) - x| <= absmax/254
    per element, and quant(deq(q)) == q (idempotence)."""
    from came_b200 import quant
    x = torch.randn(4096, 11008, device="cuda") * 1e-3
    q, a = quant.quantize_blockwise(x, signed=True)
    d = quant.dequantize_blockwise(q, a, signed=True)
    bound = a.repeat_interleave(256)[: x.numel()].view_as(x) / 254.0
    assert bool(((d - x).abs() <= bound * (1 + 1e-3)).all())
    q2, a2 = quant.quantize_blockwise(d, signed=True)
    assert torch.equal(q2, q)


# ---------------------------------------------------------------------------------------------
# trajectories
# ---------------------------------------------------------------------------------------------

def _check_fp(out, dtype):
    """fp32 states: 1e-5 on parameters (fp32) / at most one spacing of the parameter dtype on at most 1 % of
    entries (bf16, fp16); 1e-4 on states."""
    assert out["f_rel"] <= 1e-4, out
    if dtype == torch.float32:
        assert out["p_rel"] <= 1e-5, out
    else:
        assert out["p_rel"] <= 1e-3 and out["p_diff_frac"] <= 0.01 and out["p_maxspacing"] <= 2.0, out


def _check_8bit(out, dtype):
    """8-bit states: codes equal except <= 1 % of entries by one step and <= 0.01 % by more (a flipped code feeds
    back through the EMA); absmax to 1e-3; parameters to 1e-3 in Frobenius norm and, for 16-bit parameters, within
    two spacings of their dtype except on <= 0.1 % of entries (rows whose row-state code sits at 0 or 1 next to an
    outlier row change their factor a lot when that code flips: the reference's quantiser has the same property)."""
    assert out["p_rel"] <= 1e-3, out
    assert out["f_rel"] <= 1e-3, out
    assert out["code_frac"] <= 0.01 and out["code_frac2"] <= 1e-4 and out["code_max"] <= 3, out
    if dtype != torch.float32:
        assert out["p_diff_frac"] <= 0.02 and out["p_far_frac"] <= 1e-3, out


CASES_FP = [("CAME", orc.CAME), ("CAMECUDA", orc.CUDAFP)]


@pytest.mark.parametrize("cls_name,preset", CASES_FP)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("shapes,hyper", [(EDGE_SHAPES, H_DEFAULT), (ALIGNED_SHAPES, H_LLAMA), (ALIGNED_SHAPES, H_NOWD)])
def test_fp32_state_classes(cls_name, preset, dtype, shapes, hyper):
    import came_b200
    out, _, _ = run_pair(getattr(came_b200, cls_name), lambda dim: preset, shapes, _dt(dtype), 6, hyper, seed=11)
    _check_fp(out, _dt(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("shapes,hyper", [(EDGE_SHAPES, H_DEFAULT), (ALIGNED_SHAPES, H_LLAMA), (ALIGNED_SHAPES, H_NOWD)])
def test_came8bit(dtype, shapes, hyper):
    import came_b200
    preset = lambda dim: orc.TILE8 if dim == 2 else orc.FLAT8
    out, opt, gp = run_pair(came_b200.CAME8bit, preset, shapes, _dt(dtype), 6, hyper, seed=12)
    _check_8bit(out, _dt(dtype))
    st = opt.state[gp[0]]
    assert st["_mode"] == "8bit2d" and "step" not in st and st["exp_avg_q"].dtype == torch.int8


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_came8bit2d(dtype):
    import came_b200
    shapes = [s for s in EDGE_SHAPES + ALIGNED_SHAPES if len(s) == 2]
    out, _, _ = run_pair(came_b200.CAME8bit2D, lambda dim: orc.TILE8, shapes, _dt(dtype), 6, H_LLAMA, seed=13)
    _check_8bit(out, _dt(dtype))


@pytest.mark.parametrize("cls_name,f16", [("CAME8bitFull", False), ("CAME8bitMemory", True)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("shapes,hyper", [(EDGE_SHAPES, H_DEFAULT), (ALIGNED_SHAPES, H_LLAMA)])
def test_flat_classes(cls_name, f16, dtype, shapes, hyper):
    import came_b200
    out, opt, gp = run_pair(getattr(came_b200, cls_name), lambda dim: orc.FLAT8, shapes, _dt(dtype), 6, hyper, seed=14,
                            oracle_kw=dict(update_f16=f16))
    _check_8bit(out, _dt(dtype))
    st = opt.state[gp[0]]
    assert st["_mode"] == "full8bit" and st["step"] == 6
    assert st["exp_avg_sq_row_q"].data_ptr() == st["factored_row_q"][0].data_ptr()


# Many work items per persistent CTA: 450 strips / row tiles of 128 rows against 148 CTAs, so every CTA walks
# several items, its double-buffered item records are reused and its copy ring wraps across item boundaries.
MANY_ITEM_SHAPES = [(38400, 64), (12800, 256), (6400, 1280), (4096,)]


@pytest.mark.parametrize("cls_name,preset2d", [("CAME8bit", "TILE8"), ("CAME8bitFull", "FLAT8")])
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_many_items_per_cta(cls_name, preset2d, dtype):
    import came_b200
    preset = lambda dim: getattr(orc, preset2d) if dim == 2 else orc.FLAT8
    out, opt, gp = run_pair(getattr(came_b200, cls_name), preset, MANY_ITEM_SHAPES, _dt(dtype), 2, H_LLAMA, seed=21)
    _check_8bit(out, _dt(dtype))
    for plan in opt._engine.plans.values():
        assert plan.status() == 0


def test_mixed_grad_dtype_takes_flat_layout():
    """CAME8bit.py:216-223: a 2-D tensor whose gradient dtype differs from the parameter dtype does not
    take the tile path."""
    import came_b200
    p = torch.nn.Parameter(torch.randn(64, 64, device="cuda").bfloat16())
    p.grad_dtype = None        # allow a gradient dtype that differs from the parameter's
    p.grad = torch.randn(64, 64, device="cuda") * 1e-3
    opt = came_b200.CAME8bit([p], lr=1e-3)
    opt.step()
    assert opt.state[p]["_mode"] == "full8bit"


def test_bit_reproducible():
    """Two optimizers fed the same inputs end with identical bytes (fixed-order reductions, no float atomics)."""
    import came_b200
    from tests.parity_util import make_inputs
    shapes = [(384, 272), (255, 257), (700,)]
    finals = []
    for _ in range(2):
        params0, grads = make_inputs(shapes, torch.bfloat16, 4, seed=5)
        gp = [torch.nn.Parameter(p.cuda()) for p in params0]
        opt = came_b200.CAME8bit(gp, **H_LLAMA)
        for gs in grads:
            for p, g in zip(gp, gs):
                p.grad = g.cuda()
            opt.step()
        finals.append([p.data.clone() for p in gp] + [opt.state[p]["exp_avg_q"].clone() for p in gp])
    for a, b in zip(*finals):
        assert torch.equal(a, b)


def test_non_contiguous_parameter_and_param_groups():
    import came_b200
    base = torch.randn(64, 96, device="cuda")
    p = torch.nn.Parameter(base.t())          # non-contiguous view
    q = torch.nn.Parameter(torch.randn(32, device="cuda"))
    ref_p, ref_q = p.data.clone().contiguous(), q.data.clone()
    opt = came_b200.CAMECUDA([{"params": [p], "lr": 1e-3}, {"params": [q], "lr": 1e-2, "weight_decay": 0.1}], lr=1e-4)
    gp, gq = torch.randn(96, 64, device="cuda") * 1e-3, torch.randn(32, device="cuda") * 1e-3
    p.grad, q.grad = gp, gq
    opt.step()
    sp, sq = orc.init_state(ref_p.cpu(), orc.CUDAFP), orc.init_state(ref_q.cpu(), orc.CUDAFP)
    op = orc.step(ref_p.cpu(), gp.cpu(), sp, orc.Hyper(lr=1e-3), orc.CUDAFP)
    oq = orc.step(ref_q.cpu(), gq.cpu(), sq, orc.Hyper(lr=1e-2, weight_decay=0.1), orc.CUDAFP)
    assert torch.allclose(p.data.cpu(), op, rtol=1e-5, atol=1e-8)
    assert torch.allclose(q.data.cpu(), oq, rtol=1e-5, atol=1e-8)


def test_lr_is_reread_every_step_and_launch_count():
    import came_b200
    p = torch.nn.Parameter(torch.ones(32, 32, device="cuda"))
    opt = came_b200.CAME8bit([p], lr=1e-3)
    p.grad = torch.ones(32, 32, device="cuda")
    opt.step()
    first = (1.0 - p.data).abs().mean().item()
    opt.param_groups[0]["lr"] = 0.0
    before = p.data.clone()
    opt.step()
    assert first > 0 and torch.equal(before, p.data)
    assert 0 < opt.last_step_launches <= 12


def test_state_dict_roundtrip_preserves_dtypes():
    import came_b200
    def make():
        torch.manual_seed(0)
        ps = [torch.nn.Parameter(torch.randn(64, 48, device="cuda").bfloat16()),
              torch.nn.Parameter(torch.randn(300, device="cuda").bfloat16())]
        return ps
    for cls in (came_b200.CAME8bit, came_b200.CAME8bitFull, came_b200.CAMECUDA):
        a, b = make(), make()
        oa, ob = cls(a, lr=1e-3), cls(b, lr=1e-3)
        gs = [torch.randn_like(p) * 1e-3 for p in a]
        for p, g in zip(a, gs):
            p.grad = g.clone()
        oa.step()
        ob.load_state_dict(oa.state_dict())
        for pa, pb in zip(a, b):
            pb.data.copy_(pa.data)
            for k, v in oa.state[pa].items():
                if torch.is_tensor(v):
                    assert ob.state[pb][k].dtype == v.dtype, (cls.__name__, k)
                    assert torch.equal(ob.state[pb][k], v), (cls.__name__, k)
        for p, q, g in zip(a, b, gs):
            p.grad, q.grad = g.clone(), g.clone()
        oa.step(); ob.step()
        for pa, pb in zip(a, b):
            assert torch.equal(pa.data, pb.data), cls.__name__


def test_errors():
    import came_b200
    with pytest.raises(ValueError):
        came_b200.CAME8bit([torch.nn.Parameter(torch.zeros(2, 2))], lr=-1.0)
    with pytest.raises(ValueError):
        came_b200.CAME8bit2D([torch.nn.Parameter(torch.zeros(2, 2))], lr=1e-3, block_size=128)
    p = torch.nn.Parameter(torch.zeros(4, device="cuda"))
    p.grad = torch.zeros(4, device="cuda")
    with pytest.raises(NotImplementedError):
        came_b200.CAME8bit2D([p], lr=1e-3).step()
    c = torch.nn.Parameter(torch.zeros(4, 4))
    c.grad = torch.zeros(4, 4)
    with pytest.raises(RuntimeError):
        came_b200.CAME8bit([c], lr=1e-3).step()


def test_sharded_stepper_checkpoint_round_trip():
    """A shard saved by ShardedStepper.state_dict() and loaded into a fresh stepper continues bit-identically."""
    import copy
    import came_b200
    from came_b200.partition import ShardedParams, ShardedStepper
    shapes = [(256, 512), (128, 192), (4096,), (300, 256), (64,)]
    dev = torch.device("cuda")

    def build(init):
        sp = ShardedParams(shapes, torch.bfloat16, dev, 1, 0, buckets=2)
        for v, x in zip(sp.views, init):
            v.copy_(x)
        params = {i: torch.nn.Parameter(sp.views[i]) for i in sp.owned}
        return sp, params, ShardedStepper(sp, params, lambda ps: came_b200.CAME8bit(ps, lr=1e-3, weight_decay=1e-2))

    gen = torch.Generator(device=dev).manual_seed(4)
    init = [(torch.randn(s, device=dev, generator=gen) * 0.02).bfloat16() for s in shapes]
    grads = [[(torch.randn(s, device=dev, generator=gen) * 1e-2).bfloat16() for s in shapes] for _ in range(4)]
    sp, params, st = build(init)
    for k in range(2):
        for i, p in params.items():
            p.grad = grads[k][i].clone()
        st.step()
    saved = copy.deepcopy(st.state_dict())
    weights = [v.clone() for v in sp.views]
    for k in range(2, 4):
        for i, p in params.items():
            p.grad = grads[k][i].clone()
        st.step()
    sp2, params2, st2 = build(weights)
    st2.load_state_dict(saved)
    for k in range(2, 4):
        for i, p in params2.items():
            p.grad = grads[k][i].clone()
        st2.step()
    for a, b in zip(sp.views, sp2.views):
        assert torch.equal(a, b)
    bad = dict(saved, owners=[1] * len(shapes))
    with pytest.raises(ValueError):
        st2.load_state_dict(bad)


def test_grad_scale_is_applied_on_load():
    """`grad_scale` of a param_group multiplies every gradient as the kernels read it.  A power of two commutes with
    every rounding, so stepping 1024 * g with grad_scale = 1 / 1024 must leave exactly the bytes of stepping g; a
    general scale is compared with the oracle fed the scaled gradients."""
    import came_b200
    from tests.parity_util import make_inputs, hyper_of, relerr
    shapes = [(256, 512), (130, 4096), (300, 72), (33, 17), (2, 40, 24), (700,)]
    for cls in (came_b200.CAME8bit, came_b200.CAME8bitFull, came_b200.CAMECUDA):
        finals = []
        for scaled in (False, True):
            params0, grads = make_inputs(shapes, torch.bfloat16, 3, seed=61)
            gp = [torch.nn.Parameter(p.cuda()) for p in params0]
            opt = cls(gp, **H_LLAMA)
            if scaled:
                opt.param_groups[0]["grad_scale"] = 1.0 / 1024.0
            for gs in grads:
                for p, g in zip(gp, gs):
                    p.grad = (g.float() * (1024.0 if scaled else 1.0)).bfloat16().cuda()
                opt.step()
            finals.append([p.data.clone() for p in gp] +
                          [v.clone() for p in gp for k, v in sorted(opt.state[p].items()) if torch.is_tensor(v)])
        for x, y in zip(*finals):
            assert torch.equal(x, y), cls.__name__
    # a scale that is not a power of two, against the oracle
    s = 0.37
    params0, grads = make_inputs(shapes[:4], torch.bfloat16, 3, seed=62)
    gp = [torch.nn.Parameter(p.cuda()) for p in params0]
    opt = came_b200.CAME8bit(gp, **H_LLAMA)
    opt.param_groups[0]["grad_scale"] = s
    cp = [p.clone() for p in params0]
    sts = [orc.init_state(p, orc.TILE8) for p in cp]
    for gs in grads:
        for i, (p, g) in enumerate(zip(gp, gs)):
            p.grad = g.cuda()
            cp[i] = orc.step(cp[i], g.float() * s, sts[i], hyper_of(H_LLAMA), orc.TILE8)
        opt.step()
    for p, c in zip(gp, cp):
        assert relerr(p.data.float().cpu(), c.float()) <= 1e-3
