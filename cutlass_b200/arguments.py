"""Runtime arguments of the block-scaled GEMM operators.

Same names and meaning as the reference's Python Operator API
(``operators/cutlass/operators/arguments/``): ``GemmArguments`` (``gemm.py:91``),
``GroupedGemmArguments`` (``grouped_gemm.py:40``), ``ScaledOperand`` /
``ScaleMode`` / ``ScaleSwizzleMode`` (``operand.py:60,234,326``).  The reference's
traced ``EpilogueArguments`` is replaced by a fixed-function
``EpilogueDescriptor`` (alpha, beta, C, optional NVFP4 output quantisation),
because the block-scaled operator of the reference accepts no custom epilogue
(``providers/cutedsl/gemm/sm100_dense_blockscaled_static_persistent.py:298-300``).

Tensors are ``torch.Tensor`` (CPU tensors are accepted for validation; running
needs CUDA tensors).  Shapes follow the reference: ``A`` is (L, M, K) or (M, K),
``B`` is (L, K, N) or (K, N) with K contiguous (build it as an (N, K) tensor and
transpose), ``out`` is (L, M, N) or (M, N).  Packed fp4 tensors
(``torch.float4_e2m1fn_x2`` or ``uint8`` with ``ScaleMode.Blockwise1x16``) have a
physical K extent of K/2.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Any

import torch

_FP4X2 = getattr(torch, "float4_e2m1fn_x2", None)
_E8M0 = getattr(torch, "float8_e8m0fnu", None)


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def round_up(a: int, b: int) -> int:
    return ceil_div(a, b) * b


class ScaleMode(enum.Enum):
    """Block of quantized elements (batch, row, col) sharing one scale factor."""

    Blockwise1x16 = (1, 1, 16)   # NVFP4: ue4m3 scale per 16 K-elements
    Blockwise1x32 = (1, 1, 32)   # MXFP8: ue8m0 scale per 32 K-elements

    @staticmethod
    def as_tuple(mode: "ScaleMode | tuple[int, ...]") -> tuple[int, ...]:
        return tuple(mode.value) if isinstance(mode, ScaleMode) else tuple(mode)

    @staticmethod
    def numel(mode: "ScaleMode | tuple[int, ...]") -> int:
        n = 1
        for v in ScaleMode.as_tuple(mode):
            n *= int(v)
        return n

    @staticmethod
    def compare(a: "ScaleMode | tuple[int, ...]", b: "ScaleMode | tuple[int, ...]") -> bool:
        return ScaleMode.as_tuple(a) == ScaleMode.as_tuple(b)


class ScaleSwizzleMode(enum.Enum):
    """In-memory layout of the scale tensor."""

    SwizzleNone = 0
    Swizzle32x4x4 = 1    # 512-byte atoms of (32 x 4 rows) x 4 K-blocks; what tcgen05 block-scaled MMA consumes


def _is_packed_fp4(t: torch.Tensor, mode) -> bool:
    if _FP4X2 is not None and t.dtype == _FP4X2:
        return True
    return t.dtype == torch.uint8 and mode is not None and ScaleMode.compare(mode, ScaleMode.Blockwise1x16)


class DenseTensor:
    """A plain strided tensor operand."""

    def __init__(self, tensor: torch.Tensor):
        if isinstance(tensor, DenseTensor):
            tensor = tensor.tensor
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"expected a torch.Tensor, got {type(tensor).__name__}")
        self.tensor = tensor

    def copy(self) -> "DenseTensor":
        return DenseTensor(self.tensor)

    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(self.tensor.shape)

    @property
    def stride(self) -> tuple[int, ...]:
        return tuple(self.tensor.stride())

    @property
    def dtype(self):
        return self.tensor.dtype

    def data_ptr(self) -> int:
        return self.tensor.data_ptr()

    def numel(self) -> int:
        return self.tensor.numel()


def _operand_or_dense(x: Any):
    if isinstance(x, (DenseTensor, ScaledOperand)):
        return x
    return DenseTensor(x)


class ScaledOperand:
    """Logical value ``scale * quantized``: every entry of ``scale`` multiplies one
    ``mode``-shaped block of ``quantized``; ``swizzle`` names the memory layout of
    ``scale``, which must be contiguous and hold exactly ``numel_scale`` elements."""

    def __init__(self, quantized, scale, mode: ScaleMode | tuple[int, ...], swizzle: ScaleSwizzleMode):
        self.quantized = DenseTensor(quantized)
        self.scale = DenseTensor(scale)
        self.mode = mode
        self.swizzle = swizzle

    def copy(self) -> "ScaledOperand":
        return ScaledOperand(self.quantized, self.scale, self.mode, self.swizzle)

    def __getattr__(self, attr: str):
        q = self.__dict__.get("quantized")
        if q is not None and hasattr(q, attr):
            return getattr(q, attr)
        raise AttributeError(f"'{type(self).__name__}' object has no attribute '{attr}'")

    @property
    def is_packed_fp4(self) -> bool:
        return _is_packed_fp4(self.quantized.tensor, self.mode)

    @staticmethod
    def numel_scale(quantized_shape: tuple[int, ...], mode, swizzle: ScaleSwizzleMode) -> int:
        """Number of scale factors that belong to an operand of logical shape (L, rows, K) or (rows, K): one per
        ``mode`` block along K, and for the Swizzle32x4x4 layout whole 128-row x 4-block atoms (padding included).
        Same contract as the reference's ``ScaledOperand.numel_scale`` (operand.py:212-231)."""
        dims = tuple(int(d) for d in quantized_shape)
        if len(dims) not in (2, 3):
            raise ValueError(f"the operand shape must be (rows, K) or (L, rows, K); got {dims}")
        batch = dims[0] if len(dims) == 3 else 1
        rows, k_blocks = dims[-2], ceil_div(dims[-1], ScaleMode.numel(mode))
        layouts = {ScaleSwizzleMode.SwizzleNone: (1, 1), ScaleSwizzleMode.Swizzle32x4x4: (128, 4)}
        if swizzle not in layouts:
            raise ValueError(f"{swizzle!r} is not a scale layout of this library")
        row_unit, block_unit = layouts[swizzle]
        return batch * round_up(rows, row_unit) * round_up(k_blocks, block_unit)


@dataclass
class Nvfp4Quant:
    """Fused NVFP4 re-quantisation of the output: per row and per 16 columns,
    ``SF = ue4m3(amax * norm_constant / 6)`` and ``D = e2m1(x * norm_constant / SF)``.
    ``scale`` receives the scale factors in the Swizzle32x4x4 layout over (M, N/16);
    ``norm_constant`` is a one-element fp32 CUDA tensor."""

    scale: torch.Tensor
    norm_constant: torch.Tensor


@dataclass
class Mxfp8Quant:
    """Fused MXFP8 re-quantisation of the output: per row and per 32 columns,
    ``SF = ue8m0(amax * norm_constant / 448)`` (the conversion rounds up) and
    ``D = e4m3(x * norm_constant / SF)``.  ``scale`` receives the scale factors in the
    Swizzle32x4x4 layout over (M, N/32); ``norm_constant`` is a one-element fp32 CUDA tensor or None (1)."""

    scale: torch.Tensor
    norm_constant: torch.Tensor | None = None


@dataclass
class EpilogueDescriptor:
    """``out = activation(alpha * acc + bias + beta * C)`` followed by the output conversion (the order of the
    reference's host epilogue, tools/util/include/cutlass/util/reference/host/gett.hpp:714-761).
    ``alpha`` / ``beta`` are Python floats or one-element fp32 CUDA tensors (grouped GEMM: floats, or fp32
    tensors with one entry per group).  ``bias`` is an fp32 vector with one
    entry per output column (N; grouped GEMM: (groups, N)) or, with ``bias_per_row``, per output row (M; dense only).
    ``activation``: "identity", "relu", "gelu" (erf form) or "silu"."""

    alpha: float | torch.Tensor = 1.0
    beta: float | torch.Tensor = 0.0
    C: torch.Tensor | None = None
    out_quant: Nvfp4Quant | Mxfp8Quant | None = None
    bias: torch.Tensor | None = None
    bias_per_row: bool = False
    activation: str = "identity"


ACTIVATIONS = {"identity": 0, "relu": 1, "gelu": 2, "silu": 3}


def _logical_k(op, axis: int) -> int:
    """Logical contraction extent of an operand along ``axis`` (x2 for packed fp4)."""
    k = op.shape[axis]
    if isinstance(op, ScaledOperand) and op.is_packed_fp4:
        return k * 2
    return k


@dataclass
class GemmProblemSize:
    M: int
    N: int
    K: int
    L: int


class GemmArguments:
    """``out = A @ B`` with block-scaled operands; all tensors rank 3 or all rank 2."""

    def __init__(self, A, B, out, accumulator_type=torch.float32, epilogue: EpilogueDescriptor | None = None):
        self.A = _operand_or_dense(A).copy()
        self.B = _operand_or_dense(B).copy()
        self.out = _operand_or_dense(out).copy()
        self.accumulator_type = accumulator_type
        self.epilogue = epilogue
        self._validate()

    @property
    def out_is_packed_fp4(self) -> bool:
        return self.epilogue is not None and isinstance(self.epilogue.out_quant, Nvfp4Quant)

    @property
    def problem_size(self) -> GemmProblemSize:
        M = self.A.shape[-2]
        N = self.B.shape[-1]
        K = _logical_k(self.A, -1)
        L = self.A.shape[0] if len(self.A.shape) == 3 else 1
        return GemmProblemSize(M=M, N=N, K=K, L=L)

    def _validate(self) -> None:
        """Shape agreement of A (.., M, K), B (.., K, N) and out (.., M, N); raises ValueError naming the mismatch.
        Same checks as the reference's ``GemmArguments`` (gemm.py:163-199)."""
        shapes = {"A": self.A.shape, "B": self.B.shape, "out": self.out.shape}
        for name, shp in shapes.items():
            if len(shp) not in (2, 3):
                raise ValueError(f"{name} has rank {len(shp)} ({shp}); operands are matrices (rank 2) or batches of matrices (rank 3)")
        batch = {name: tuple(shp[:-2]) for name, shp in shapes.items()}
        if batch["B"] != batch["A"] or batch["out"] != batch["A"]:
            raise ValueError(f"A, B and out must agree in rank and batch count: A {shapes['A']}, B {shapes['B']}, out {shapes['out']}")
        M, k_of_a = self.A.shape[-2], _logical_k(self.A, -1)
        k_of_b, N = _logical_k(self.B, -2), self.B.shape[-1]
        if k_of_a != k_of_b:
            raise ValueError(f"contraction extents differ: A (.., M, K) has K = {k_of_a}, B (.., K, N) has K = {k_of_b} "
                             f"(shapes {shapes['A']} and {shapes['B']}; packed fp4 counts two elements per byte)")
        out_m, out_n = self.out.shape[-2], self.out.shape[-1] * (2 if self.out_is_packed_fp4 else 1)
        if (out_m, out_n) != (M, N):
            raise ValueError(f"out is {out_m} x {out_n} but A @ B is {M} x {N}")


class GroupedGemmArguments:
    """Contiguous-offset grouped GEMM (``operators/cutlass/operators/arguments/grouped_gemm.py:40``):
    ``A`` is (TotalM, K), ``B`` is (groups, K, N) with K contiguous, ``out`` is (TotalM, N),
    ``offsets`` is int32[groups] with the END row of each group::

        start = 0
        for g in range(groups):
            out[start:offsets[g]] = A[start:offsets[g]] @ B[g]
            start = offsets[g]

    The scale tensor of ``A`` holds one Swizzle32x4x4 layout per group, back to back, each
    padded to a multiple of 128 rows.
    """

    def __init__(self, A, B, out, accumulator_type=torch.float32, offsets=None, epilogue: EpilogueDescriptor | None = None):
        if offsets is None:
            raise ValueError("offsets is required")
        self.A = _operand_or_dense(A).copy()
        self.B = _operand_or_dense(B).copy()
        self.out = _operand_or_dense(out).copy()
        self.accumulator_type = accumulator_type
        self.offsets = DenseTensor(offsets)
        self.epilogue = epilogue
        self._validate()

    @property
    def problem_size(self) -> GemmProblemSize:
        a_shape = self.A.shape[-2:]
        return GemmProblemSize(M=a_shape[0], N=self.B.shape[-1], K=_logical_k(self.A, -1), L=self.B.shape[0])

    def _validate(self) -> None:
        if len(self.A.shape) == 3 and self.A.shape[0] != 1:
            raise ValueError(f"A must be (TotalM, K) or (1, TotalM, K), got {self.A.shape}")
        if len(self.A.shape) not in (2, 3):
            raise ValueError(f"A must be a tensor of rank 2 or 3, got {self.A.shape}")
        if len(self.B.shape) != 3:
            raise ValueError(f"B must be (problems_in_group, K, N), got {self.B.shape}")
        if len(self.out.shape) not in (2, 3) or (len(self.out.shape) == 3 and self.out.shape[0] != 1):
            raise ValueError(f"out must be (TotalM, N) or (1, TotalM, N), got {self.out.shape}")
        if len(self.offsets.shape) != 1:
            raise ValueError(f"offsets must be rank 1, got {self.offsets.shape}")
        if self.offsets.shape[0] != self.B.shape[0]:
            raise ValueError(f"offsets has {self.offsets.shape[0]} entries but B has {self.B.shape[0]} problems")
        if self.offsets.dtype != torch.int32:
            raise ValueError(f"offsets must be int32, got {self.offsets.dtype}")
        a_k = _logical_k(self.A, -1)
        b_k = _logical_k(self.B, -2)
        if a_k != b_k:
            raise ValueError(f"A's K dimension ({a_k}) must be equal to B's K dimension ({b_k})")
        if self.out.shape[-2] != self.A.shape[-2]:
            raise ValueError(f"out's M dimension ({self.out.shape[-2]}) must be equal to A's TotalM ({self.A.shape[-2]})")
        if self.out.shape[-1] != self.B.shape[-1]:
            raise ValueError(f"out's N dimension ({self.out.shape[-1]}) must be equal to B's N dimension ({self.B.shape[-1]})")
