"""The quantisation step in front of the GEMM: bf16 matrix -> ``ScaledOperand`` whose scale
factors are already in the interleaved ``Swizzle32x4x4`` layout (contract:
operators/cutlass/operators/arguments/operand.py:353-367 of the reference).

    A = quantize_blockscaled(x_bf16, ScaleMode.Blockwise1x16)          # NVFP4: e2m1 + ue4m3 per 16
    A = quantize_blockscaled(x_bf16, ScaleMode.Blockwise1x32)          # MXFP8: e4m3 + ue8m0 per 32

The arithmetic is the reference's block-scale computation (tools/util/include/cutlass/util/reference/
host/gett.hpp:436-478); the work is one launch of a hand-written CUDA kernel behind ``bsg_quantize``.
"""
from __future__ import annotations

import ctypes as C

from .arguments import ScaledOperand, ScaleMode, ScaleSwizzleMode
from .formats import numel_scale


def quantize_blockscaled(x, mode=ScaleMode.Blockwise1x16, *, norm_constant=None, out=None, scale_out=None, stream=None,
                         use_pdl: bool = False) -> ScaledOperand:
    """Quantise ``x`` (rows, K) bf16, row-major (last stride 1), on its CUDA device.

    ``norm_constant``: fp32 device tensor with one element (the ``st`` of the reference; NVFP4 callers
    usually pass 448 * 6 / amax(x)), or None for 1.  ``out`` / ``scale_out`` may be given to reuse
    buffers (uint8; ``scale_out`` must hold exactly ``numel_scale`` bytes).  The returned operand's
    logical value is ``scale * quantized / norm_constant``.  Asynchronous on ``stream``.  ``use_pdl``: launch as a
    programmatic dependent launch (its set-up overlaps the kernel before it, the next kernel's set-up overlaps its tail)."""
    import torch
    from . import lib as L
    from .operator import to_cuda_stream
    if ScaleMode.compare(mode, ScaleMode.Blockwise1x16):
        kind, vec = L.KIND_NVFP4, 16
    elif ScaleMode.compare(mode, ScaleMode.Blockwise1x32):
        kind, vec = L.KIND_MXFP8, 32
    else:
        raise ValueError(f"unsupported scale mode {mode}: Blockwise1x16 (NVFP4) or Blockwise1x32 (MXFP8)")
    if x.dim() != 2 or x.dtype != torch.bfloat16 or not x.is_cuda or x.stride(1) != 1:
        raise ValueError("x must be a 2-D bf16 CUDA tensor with unit stride along K")
    rows, K = x.shape
    q_shape = (rows, K // 2) if kind == L.KIND_NVFP4 else (rows, K)
    n_sf = numel_scale(rows, K, vec)
    if out is None:
        out = torch.empty(q_shape, dtype=torch.uint8, device=x.device)
    if scale_out is None:
        scale_out = torch.empty(n_sf, dtype=torch.uint8, device=x.device)
    if tuple(out.shape) != q_shape or out.element_size() != 1 or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous 1-byte tensor of shape {q_shape}")
    if scale_out.numel() != n_sf or scale_out.element_size() != 1 or not scale_out.is_contiguous():
        raise ValueError(f"scale_out must be a contiguous 1-byte tensor of {n_sf} elements")
    if norm_constant is not None and (norm_constant.dtype != torch.float32 or norm_constant.numel() != 1 or not norm_constant.is_cuda):
        raise ValueError("norm_constant must be a one-element fp32 CUDA tensor")
    a = L.QuantArgs()
    a.kind, a.rows, a.K, a.use_pdl = kind, rows, K, int(use_pdl)
    a.X, a.ldx = x.data_ptr(), x.stride(0) if rows > 1 else max(K, x.stride(0))
    a.Q, a.SF = out.data_ptr(), scale_out.data_ptr()
    a.norm_constant = norm_constant.data_ptr() if norm_constant is not None else None
    L.check(L.load().bsg_quantize(C.byref(a), to_cuda_stream(stream)))
    return ScaledOperand(out, scale_out, mode, ScaleSwizzleMode.Swizzle32x4x4)
