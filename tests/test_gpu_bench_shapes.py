"""GPU parity at the column counts of the benchmark configurations.

The staged first pass picks its template instance and batch geometry from the column count and the element size
(column groups per thread 1..4, one or two row sets, 1..16 rows per staged batch); the momentum / apply passes pick
their tile widths from it too.  These cases step matrices whose column counts are those of the GPT-2-medium,
Llama-1B, Llama-7B and Llama-3-8B parameter sets (1024 ... 14336; 32000 for a [hidden, vocab] matrix), with few rows
so that the CPU oracle stays fast, in every class and dtype, with the per-tensor gradient scales 10^U(-5,-2) of the
Llama-7B configuration.  Two full-size matrices (4096 x 11008, 32000 x 4096) follow.  Tolerances are those of
tests/test_gpu_parity.py.  Reference: came_kernels.cu:61-96, 198-243, 596-619 (first pass), 2584-2683, 3332-3366."""
import pytest
import torch

from oracle import came_oracle as orc
from tests.parity_util import run_pair
from tests.test_gpu_parity import H_DEFAULT, H_LLAMA, _check_8bit, _check_fp, _dt

pytestmark = pytest.mark.gpu

BENCH_COLS = [1024, 2048, 2304, 3072, 4096, 5632, 8192, 11008, 14336]
BENCH_SHAPES = [(rows, cols) for cols in BENCH_COLS for rows in (130, 257)] + [(4096,)]
VOCAB_SHAPES = [(130, 32000), (64, 20480), (130, 16448)]      # beyond the widest staged row of the first pass


def _status_ok(opt):
    for plan in opt._engine.plans.values():
        assert plan.status() == 0


@pytest.mark.parametrize("cls_name,preset2d,f16", [("CAME8bit", "TILE8", False), ("CAME8bit2D", "TILE8", False),
                                                   ("CAME8bitFull", "FLAT8", False), ("CAME8bitMemory", "FLAT8", True)])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
def test_8bit_classes_at_bench_columns(cls_name, preset2d, f16, dtype):
    import came_b200
    shapes = [s for s in BENCH_SHAPES if len(s) == 2 or cls_name != "CAME8bit2D"]
    preset = lambda dim: getattr(orc, preset2d) if dim == 2 else orc.FLAT8
    out, opt, _ = run_pair(getattr(came_b200, cls_name), preset, shapes, _dt(dtype), 6, H_LLAMA, seed=31,
                           oracle_kw=dict(update_f16=f16), per_tensor_scale=True)
    _check_8bit(out, _dt(dtype))
    _status_ok(opt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_camecuda_at_bench_columns(dtype):
    import came_b200
    out, opt, _ = run_pair(came_b200.CAMECUDA, lambda dim: orc.CUDAFP, BENCH_SHAPES, _dt(dtype), 6, H_DEFAULT, seed=32,
                           per_tensor_scale=True)
    _check_fp(out, _dt(dtype))
    _status_ok(opt)


@pytest.mark.parametrize("cls_name,preset2d", [("CAME8bit", "TILE8"), ("CAME8bitFull", "FLAT8")])
def test_vocab_wide_rows(cls_name, preset2d):
    """Rows too wide for the staged first pass take the two-pass kernels while the momentum / apply passes stay on
    the staged path (a [hidden, vocab]-shaped matrix)."""
    import came_b200
    preset = lambda dim: getattr(orc, preset2d)
    out, opt, _ = run_pair(getattr(came_b200, cls_name), preset, VOCAB_SHAPES, torch.bfloat16, 3, H_LLAMA, seed=33,
                           per_tensor_scale=True)
    _check_8bit(out, torch.bfloat16)
    _status_ok(opt)


@pytest.mark.parametrize("shape,steps", [((4096, 11008), 2), ((32000, 4096), 1)])
def test_full_size_matrix(shape, steps):
    """One matrix of the Llama-7B set at full size, CAME8bit, bf16."""
    import came_b200
    out, opt, _ = run_pair(came_b200.CAME8bit, lambda dim: orc.TILE8, [shape], torch.bfloat16, steps, H_LLAMA, seed=34,
                           per_tensor_scale=True)
    _check_8bit(out, torch.bfloat16)
    _status_ok(opt)


def test_camecuda_zero_rows_and_columns_take_the_clamped_path():
    """CAMECUDA clamps its factors at 1e-30 (came_kernels.cu:577, 591-592).  The staged first pass derives the clip sum
    from a closed form that holds while no clamp binds; rows and columns whose gradient is identically zero make one
    bind (v = (1 - beta2) * eps0 ~ 1e-33), and the step must then fall back to the explicit sum and still match."""
    import came_b200
    from tests.parity_util import make_inputs, hyper_of, relerr
    shapes = [(256, 1024), (130, 4096)]
    params0, grads = make_inputs(shapes, torch.float32, 3, seed=71)
    for gs in grads:
        for g in gs:
            g[10:20, :] = 0.0
            g[:, 64:96] = 0.0
    gp = [torch.nn.Parameter(p.cuda()) for p in params0]
    opt = came_b200.CAMECUDA(gp, **H_DEFAULT)
    cp = [p.clone() for p in params0]
    sts = [orc.init_state(p, orc.CUDAFP) for p in cp]
    for gs in grads:
        for i, (p, g) in enumerate(zip(gp, gs)):
            p.grad = g.cuda()
            cp[i] = orc.step(cp[i], g, sts[i], hyper_of(H_DEFAULT), orc.CUDAFP)
        opt.step()
    _status_ok(opt)
    for p, c, st in zip(gp, cp, sts):
        assert relerr(p.data.cpu(), c) <= 1e-5
        for k in ("exp_avg", "exp_avg_sq_row", "exp_avg_sq_col", "exp_avg_res_row", "exp_avg_res_col"):
            assert relerr(opt.state[p][k].cpu(), st[k]) <= 1e-4, k
