"""Blockwise linear absmax codec on CUDA tensors: the counterpart of
came_pytorch/blockwise_quantization.py (quantize_blockwise :66-82, dequantize_blockwise :108-124) and of
the tile layout of came2d_step, computed by libcame_b200 and bit-exact with the reference's fp32 formulas.
"""
from __future__ import annotations

import math

import torch

from . import _lib

BLOCK = 256


def num_blocks(numel: int, block_size: int = BLOCK) -> int:
    if block_size <= 0:
        raise ValueError(f"block_size must be > 0, got {block_size}")
    return max(1, math.ceil(numel / block_size))


def _require(t: torch.Tensor, block_size: int) -> None:
    if block_size != BLOCK:
        raise ValueError("came_b200 supports block_size=256 only")
    if not t.is_cuda:
        raise RuntimeError("came_b200.quant works on CUDA tensors only (there is no CPU fallback)")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def quantize_blockwise(tensor: torch.Tensor, *, signed: bool, block_size: int = BLOCK):
    """-> (q, absmax): int8 (signed) or uint8 codes shaped like `tensor`, fp32 absmax per 256 flat elements."""
    _require(tensor, block_size)
    lib = _lib.load()
    flat = tensor.detach().reshape(-1).to(torch.float32).contiguous()
    n = flat.numel()
    q = torch.empty(n, device=tensor.device, dtype=torch.int8 if signed else torch.uint8)
    absmax = torch.empty(num_blocks(n), device=tensor.device, dtype=torch.float32)
    with torch.cuda.device(tensor.device):
        _lib.check(lib.came_b200_quantize_blockwise(flat.data_ptr(), q.data_ptr(), absmax.data_ptr(), n, int(signed),
                                                    _stream(tensor)))
    return q.view(tensor.shape), absmax


def dequantize_blockwise(q: torch.Tensor, absmax: torch.Tensor, *, signed: bool, block_size: int = BLOCK,
                         dtype: torch.dtype = torch.float32) -> torch.Tensor:
    _require(q, block_size)
    want = torch.int8 if signed else torch.uint8
    if q.dtype != want:
        raise RuntimeError(f"expected {want} codes, got {q.dtype}")
    lib = _lib.load()
    qc = q.reshape(-1).contiguous()
    n = qc.numel()
    a = absmax.reshape(-1).to(torch.float32).contiguous()
    if a.numel() < num_blocks(n):
        raise RuntimeError(f"absmax has {a.numel()} entries, {num_blocks(n)} needed")
    out = torch.empty(n, device=q.device, dtype=torch.float32)
    with torch.cuda.device(q.device):
        _lib.check(lib.came_b200_dequantize_blockwise(qc.data_ptr(), a.data_ptr(), out.data_ptr(), n, int(signed),
                                                      _stream(q)))
    return out.view(q.shape).to(dtype)


def quantize_tile16(matrix: torch.Tensor):
    """-> (q int8 [R, C], absmax fp32 [ceil(R/16)*ceil(C/16)]): the exp_avg layout of CAME8bit / CAME8bit2D."""
    _require(matrix, BLOCK)
    if matrix.dim() != 2:
        raise RuntimeError("quantize_tile16 expects a 2-D tensor")
    lib = _lib.load()
    src = matrix.detach().to(torch.float32).contiguous()
    rows, cols = src.shape
    q = torch.empty((rows, cols), device=matrix.device, dtype=torch.int8)
    absmax = torch.empty(math.ceil(rows / 16) * math.ceil(cols / 16), device=matrix.device, dtype=torch.float32)
    with torch.cuda.device(matrix.device):
        _lib.check(lib.came_b200_quantize_tile16(src.data_ptr(), q.data_ptr(), absmax.data_ptr(), rows, cols,
                                                 _stream(matrix)))
    return q, absmax


def dequantize_tile16(q: torch.Tensor, absmax: torch.Tensor) -> torch.Tensor:
    _require(q, BLOCK)
    if q.dim() != 2 or q.dtype != torch.int8:
        raise RuntimeError("dequantize_tile16 expects a 2-D int8 tensor")
    lib = _lib.load()
    qc = q.contiguous()
    rows, cols = qc.shape
    a = absmax.reshape(-1).to(torch.float32).contiguous()
    need = math.ceil(rows / 16) * math.ceil(cols / 16)
    if a.device != q.device:
        raise RuntimeError(f"absmax is on {a.device}, the codes on {q.device}")
    if a.numel() < need:
        raise RuntimeError(f"absmax has {a.numel()} entries, {need} needed")
    out = torch.empty((rows, cols), device=q.device, dtype=torch.float32)
    with torch.cuda.device(q.device):
        _lib.check(lib.came_b200_dequantize_tile16(qc.data_ptr(), a.data_ptr(), out.data_ptr(), rows, cols, _stream(q)))
    return out
