"""Generates the golden fixtures in this directory by running the REFERENCE's own Python code on CPU.

Run once where the reference checkout is available:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/tukisuwa-CAME

Outputs (committed): codec.npz, traj_<class>_<case>.npz.  The tests regenerate the inputs from the
same seeded numpy RandomState streams (MT19937, stable across numpy versions) through `golden_inputs`,
so the fixtures only hold the reference's outputs.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> (shapes, dtype, steps, hyper-parameters)
HYPER_DEFAULT = dict(lr=2e-4, eps=(1e-30, 1e-16), clip_threshold=1.0, betas=(0.9, 0.999, 0.9999), weight_decay=1e-2)
HYPER_LLAMA = dict(lr=2e-4, eps=(1e-30, 1e-16), clip_threshold=1.0, betas=(0.9, 0.95, 0.995), weight_decay=1e-2)
CASES = {
    "small_f32": dict(shapes=[(48, 40), (33, 17), (700,)], dtype="float32", steps=6, hyper=HYPER_DEFAULT, seed=1),
    "long_f32": dict(shapes=[(300, 20), (20, 300), (5,)], dtype="float32", steps=6, hyper=HYPER_LLAMA, seed=2),
    "small_bf16": dict(shapes=[(64, 48), (1, 40), (40, 1), (300,)], dtype="bfloat16", steps=6, hyper=HYPER_LLAMA, seed=3),
    "nowd_f32": dict(shapes=[(32, 32), (256,)], dtype="float32", steps=4,
                     hyper=dict(HYPER_DEFAULT, weight_decay=0.0), seed=4),
    # tensors of more than two dimensions: a conv-like weight with tiny matrices, a few larger ones (state-vector
    # blocks of 256 straddle the matrices in both)
    "nd_f32": dict(shapes=[(12, 5, 3, 3), (3, 40, 24)], dtype="float32", steps=5, hyper=HYPER_LLAMA, seed=8),
    "nd_bf16": dict(shapes=[(4, 6, 3, 3), (2, 3, 17, 9)], dtype="bfloat16", steps=5, hyper=HYPER_LLAMA, seed=9),
}
CLASSES = ["CAME", "CAMECUDA", "CAME8bitFull", "CAME8bit", "CAME8bitMemory"]


def golden_inputs(case: dict):
    """Seeded inputs of one case: initial parameters ~N(0, 0.02^2); per-step grads ~N(0, 1e-3^2) with
    every 7th row (or element, 1-D) scaled x100.  Returns (params, grads[step][tensor]) as torch CPU tensors."""
    rs = np.random.RandomState(case["seed"])
    dt = getattr(torch, case["dtype"])
    params = [torch.from_numpy((rs.standard_normal(s) * 0.02).astype(np.float32)).to(dt) for s in case["shapes"]]
    grads = []
    for _ in range(case["steps"]):
        gs = []
        for s in case["shapes"]:
            g = (rs.standard_normal(s) * 1e-3).astype(np.float32)
            g[::7] *= 100.0
            gs.append(torch.from_numpy(g).to(dt))
        grads.append(gs)
    return params, grads


def codec_inputs():
    """Known-answer inputs for the blockwise codec: gaussian blocks, an all-zero block, a single
    outlier, a negative-only block (unsigned codec), a ragged tail, and exact .5 ties."""
    rs = np.random.RandomState(7)
    out = {}
    out["gauss"] = (rs.standard_normal(1000) * 1e-3).astype(np.float32)
    z = (rs.standard_normal(768) * 1e-3).astype(np.float32)
    z[256:512] = 0.0
    out["zero_block"] = z
    o = (rs.standard_normal(512) * 1e-3).astype(np.float32)
    o[300] = 5.0
    out["outlier"] = o
    out["negative"] = -np.abs(rs.standard_normal(300)).astype(np.float32)
    out["ragged"] = rs.standard_normal(257).astype(np.float32)
    out["single"] = np.array([0.3], dtype=np.float32)
    k = np.arange(-127, 128, dtype=np.float32)
    t = np.concatenate([(k + 0.5) / 127.0, [1.0]]).astype(np.float32)      # absmax = 1 -> x*127 lands on .5 ties
    out["ties_signed"] = t
    ku = np.arange(0, 255, dtype=np.float32)
    out["ties_unsigned"] = np.concatenate([(ku + 0.5) / 255.0, [1.0]]).astype(np.float32)
    out["positive"] = np.abs(rs.standard_normal(600) * 1e-6).astype(np.float32)
    return out


def _bits(t: torch.Tensor) -> np.ndarray:
    """Lossless numpy view of a tensor (bf16 -> int16 bit pattern)."""
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().copy()
    return t.detach().numpy().copy()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of tukisuwa/CAME (the directory that holds came_pytorch/)")
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    import came_pytorch
    from came_pytorch import blockwise_quantization as bq

    torch.set_num_threads(1)

    # --- codec known answers ---
    blob = {}
    for name, x in codec_inputs().items():
        xt = torch.from_numpy(x)
        for signed in (True, False):
            q, a = bq.quantize_blockwise(xt, signed=signed, block_size=256)
            d = bq.dequantize_blockwise(q, a, signed=signed, block_size=256)
            tag = f"{name}.{'i8' if signed else 'u8'}"
            blob[tag + ".q"] = q.numpy().copy()
            blob[tag + ".absmax"] = a.numpy().copy()
            blob[tag + ".deq"] = d.numpy().copy()
    np.savez_compressed(os.path.join(HERE, "codec.npz"), **blob)

    # --- trajectories of the reference optimizers on CPU tensors ---
    for cls_name in CLASSES:
        cls = getattr(came_pytorch, cls_name)
        for case_name, case in CASES.items():
            params0, grads = golden_inputs(case)
            params = [torch.nn.Parameter(p.clone()) for p in params0]
            opt = cls(params, **case["hyper"])
            blob = {}
            for s, gs in enumerate(grads):
                for p, g in zip(params, gs):
                    p.grad = g.clone()
                opt.step()
                for i, p in enumerate(params):
                    blob[f"p{i}.step{s}"] = _bits(p.data)
            for i, p in enumerate(params):
                for k, v in opt.state[p].items():
                    if torch.is_tensor(v) and v.dim() > 0 and not k.startswith("factored_"):
                        blob[f"state{i}.{k}"] = _bits(v)
            np.savez_compressed(os.path.join(HERE, f"traj_{cls_name}_{case_name}.npz"), **blob)
            print("wrote", cls_name, case_name, len(blob), "arrays")


if __name__ == "__main__":
    main()
