"""Operators over the native library: discovery, support checks, run.

Mirrors the shape of the reference's Operator API
(``operators/cutlass/operators/base.py:49`` ``Operator``, ``__init__.py:72``
``get_operators``): ``get_operators(args)`` returns the operators that can run the
arguments, best first; ``Operator.supports(args)`` returns a ``Status``;
``Operator.run(args, compiled_artifact=None, stream=None, workspace=None,
assume_supported_args=False)`` enqueues the kernel on ``stream`` (``None`` = the
null stream, as in ``base.py:191-192``) and raises ``ValueError`` for unsupported
arguments.  There is one provider: the sm_100a shared library.  ``compile`` has
nothing to build at run time; it resolves the library and returns a handle.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Callable

import torch

from . import lib as L
from .arguments import (ACTIVATIONS, DenseTensor, EpilogueDescriptor, GemmArguments, GroupedGemmArguments, Mxfp8Quant, ScaledOperand,
                        ScaleMode, ScaleSwizzleMode, _E8M0, _FP4X2, _logical_k)
from .status import Status


@dataclass(frozen=True)
class OperatorMetadata:
    """Everything that distinguishes one operator instance from another."""

    operator_name: str
    kind: int                 # lib.KIND_NVFP4 / lib.KIND_MXFP8
    tile_n: int               # MMA tile N (128 or 256)
    cta_group: int            # CTAs per MMA (1 or 2); tile M = 128 * cta_group
    grouped: bool = False
    supported_targets: tuple[str, ...] = ("100a",)

    @property
    def tile_shape(self) -> tuple[int, int, int]:
        return (128 * self.cta_group, self.tile_n, 256 if self.kind in (L.KIND_NVFP4, L.KIND_MXFP4) else 128)


@dataclass
class AllocationRequirement:
    size_bytes: int
    alignment_bytes: int = 16


@dataclass
class Workspace:
    """A caller-provided device buffer (``torch.uint8`` tensor) used as kernel workspace."""

    tensor: torch.Tensor

    def data_ptr(self) -> int:
        return self.tensor.data_ptr()

    def nbytes(self) -> int:
        return self.tensor.numel() * self.tensor.element_size()


@dataclass
class CompiledArtifact:
    """Handle of the loaded native library for one operator configuration."""

    library: C.CDLL
    metadata: OperatorMetadata
    extra: dict = field(default_factory=dict)


_WORKSPACE_BYTES = 16
_default_workspaces: dict[int, torch.Tensor] = {}


def _default_workspace(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _default_workspaces.get(idx)
    if ws is None:
        ws = torch.zeros(_WORKSPACE_BYTES, dtype=torch.uint8, device=torch.device("cuda", idx))
        _default_workspaces[idx] = ws
    return ws


def to_cuda_stream(stream) -> int:
    """Stream-like object -> raw CUstream handle (0 = null stream)."""
    if stream is None:
        return 0
    if isinstance(stream, int):
        return stream
    if hasattr(stream, "cuda_stream"):
        return int(stream.cuda_stream)
    if hasattr(stream, "__cuda_stream__"):
        return int(stream.__cuda_stream__()[1])
    try:
        return int(stream)
    except Exception as exc:  # noqa: BLE001
        raise TypeError(f"cannot interpret {type(stream).__name__} as a CUDA stream") from exc


def _operand_format(op: ScaledOperand) -> str | None:
    """Data / scale format of one operand: "nvfp4" (e2m1, ue4m3 per 16), "mxfp8" (e4m3, ue8m0 per 32) or "mxfp4"
    (e2m1, ue8m0 per 32; needs the packed fp4 dtype, since uint8 with 32-wide blocks means e4m3 codes)."""
    q, s = op.quantized.dtype, op.scale.dtype
    is_fp4 = _FP4X2 is not None and q == _FP4X2
    if ScaleMode.compare(op.mode, ScaleMode.Blockwise1x16):
        if (q == torch.uint8 or is_fp4) and s in (torch.uint8, torch.float8_e4m3fn):
            return "nvfp4"
    if ScaleMode.compare(op.mode, ScaleMode.Blockwise1x32) and (s == torch.uint8 or (_E8M0 is not None and s == _E8M0)):
        if q in (torch.uint8, torch.float8_e4m3fn):
            return "mxfp8"
        if is_fp4:
            return "mxfp4"
    return None


_PAIR_KINDS = {("nvfp4", "nvfp4"): L.KIND_NVFP4, ("mxfp8", "mxfp8"): L.KIND_MXFP8, ("mxfp4", "mxfp4"): L.KIND_MXFP4,
               ("mxfp8", "mxfp4"): L.KIND_MXFP8_MXFP4}


def _pair_kind(A: ScaledOperand, B: ScaledOperand) -> int | None:
    """Library kind of an (A, B) pair, or None when the library has no kernel for the combination."""
    return _PAIR_KINDS.get((_operand_format(A), _operand_format(B)))


def _scalar_ptr(v) -> tuple[float, int | None]:
    if isinstance(v, torch.Tensor):
        if v.numel() != 1 or v.dtype != torch.float32:
            raise ValueError("alpha / beta tensors must be one-element float32 tensors")
        return 0.0, v.data_ptr()
    return float(v), None


class Operator:
    """One runnable kernel configuration behind the uniform supports / compile / run interface."""

    supported_args_type: type = object
    designed_for_min_cc: int = 100

    def __init__(self, metadata: OperatorMetadata):
        self._metadata = metadata

    @property
    def metadata(self) -> OperatorMetadata:
        return self._metadata

    # -- interface ---------------------------------------------------------
    def supports(self, args, target_sm: str | None = None) -> Status:
        if not isinstance(args, self.supported_args_type):
            return Status.fail(f"{type(self).__name__} takes {self.supported_args_type.__name__}, got {type(args).__name__}")
        if target_sm is not None and str(target_sm).replace("sm_", "") not in self._metadata.supported_targets:
            return Status.fail(f"target {target_sm} is not supported (only {self._metadata.supported_targets})")
        return self._supports(args)

    def compile(self, args=None, target_sm: str | None = None) -> CompiledArtifact:
        return CompiledArtifact(library=L.load(), metadata=self._metadata)

    def run(self, args, compiled_artifact: CompiledArtifact | None = None, stream=None,
            workspace: Workspace | torch.Tensor | None = None, assume_supported_args: bool = False) -> None:
        if not assume_supported_args and not (status := self.supports(args)):
            raise ValueError(f"Operator does not support the provided arguments: {status.error}")
        compiled_artifact = compiled_artifact or self.compile(args)
        return self._run(args, compiled_artifact, to_cuda_stream(stream), workspace)

    def get_workspace_size(self, args) -> AllocationRequirement:
        return AllocationRequirement(_WORKSPACE_BYTES, 16)

    def initialize_workspace(self, args, workspace, stream=None) -> None:
        """Zero a caller-provided workspace once, before its first run."""
        t = workspace.tensor if isinstance(workspace, Workspace) else workspace
        L.check(L.load().bsg_workspace_init(t.data_ptr(), t.numel() * t.element_size(), to_cuda_stream(stream)))

    def check_device_status(self, workspace: Workspace | torch.Tensor | None = None, stream=None,
                            device: torch.device | None = None) -> None:
        """Synchronise ``stream`` and raise if a bounded device-side wait ran out in the last run."""
        ws = self._resolve_workspace(workspace, device or torch.device("cuda", torch.cuda.current_device()))
        L.check(L.load().bsg_read_device_status(ws.data_ptr(), to_cuda_stream(stream)))

    # -- helpers -----------------------------------------------------------
    @staticmethod
    def _resolve_workspace(workspace, device) -> torch.Tensor:
        if workspace is None:
            return _default_workspace(device)
        t = workspace.tensor if isinstance(workspace, Workspace) else workspace
        if t.numel() * t.element_size() < _WORKSPACE_BYTES:
            raise ValueError(f"workspace must hold at least {_WORKSPACE_BYTES} bytes")
        return t

    def _check_scaled_pair(self, A, B, a_rows_shape, b_rows_shape, K) -> Status:
        md = self._metadata
        if not isinstance(A, ScaledOperand) or not isinstance(B, ScaledOperand):
            return Status.fail("A and B must be ScaledOperand (block-scaled GEMM)")
        for name, op in (("A", A), ("B", B)):
            if op.swizzle != ScaleSwizzleMode.Swizzle32x4x4:
                return Status.fail(f"{name}: scale swizzle {op.swizzle} is not supported (need Swizzle32x4x4)")
            if _operand_format(op) is None:
                return Status.fail(f"{name}: unsupported combination of dtype {op.quantized.dtype}, scale dtype "
                                   f"{op.scale.dtype} and scale mode {op.mode}")
        if not ScaleMode.compare(A.mode, B.mode):
            return Status.fail("A and B must use the same scale format and scale mode")
        if _pair_kind(A, B) is None:
            return Status.fail(f"no kernel for A {_operand_format(A)} with B {_operand_format(B)} (same format on both sides, or "
                               "MXFP8 A with MXFP4 B)")
        if _pair_kind(A, B) != md.kind:
            return Status.fail("operand format does not match this operator")
        k_align = {L.KIND_NVFP4: 32, L.KIND_MXFP8: 16, L.KIND_MXFP4: 32, L.KIND_MXFP8_MXFP4: 128}[md.kind]
        if K % k_align != 0:
            return Status.fail(f"K={K} must be a multiple of {k_align}")
        for name, op, shp in (("A", A, a_rows_shape), ("B", B, b_rows_shape)):
            want = ScaledOperand.numel_scale(shp, op.mode, op.swizzle)
            if op.scale.numel() != want:
                return Status.fail(f"{name}: scale tensor has {op.scale.numel()} elements, expected {want} for shape {shp}")
            if not op.scale.tensor.is_contiguous():
                return Status.fail(f"{name}: scale tensor must be contiguous")
            if op.scale.data_ptr() % 16 != 0 or op.quantized.data_ptr() % 16 != 0:
                return Status.fail(f"{name}: tensors must be 16-byte aligned")
        return Status.success()

    def _supports(self, args) -> Status:  # pragma: no cover - abstract
        raise NotImplementedError

    def _run(self, args, artifact, stream, workspace) -> None:  # pragma: no cover - abstract
        raise NotImplementedError


# Unquantised output types (the reference's operator lists Float32 / Float16 / BFloat16 / Float8E4M3FN / Float8E5M2,
# providers/cutedsl/gemm/sm100_dense_blockscaled_static_persistent.py:454-460).
_PLAIN_OUT_KINDS = {torch.bfloat16: L.OUT_BF16, torch.float16: L.OUT_F16, torch.float32: L.OUT_F32,
                    torch.float8_e4m3fn: L.OUT_E4M3, torch.float8_e5m2: L.OUT_E5M2}
_PLAIN_OUT_N_MULTIPLE = {torch.bfloat16: 8, torch.float16: 8, torch.float32: 4, torch.float8_e4m3fn: 16, torch.float8_e5m2: 16}


def _plain_out_kind(t: torch.Tensor) -> int:
    return _PLAIN_OUT_KINDS[t.dtype]


def _k_major_rows(t: torch.Tensor, rows_axis: int, k_axis: int) -> bool:
    """True when ``t`` has K contiguous and rows / batch entries that start on 16-byte boundaries: a row pitch
    larger than K and a batch stride larger than one matrix are fine (a slice of a larger buffer)."""
    shape, stride = t.shape, t.stride()
    esz = t.element_size()
    if stride[k_axis] != 1:
        return False
    if shape[rows_axis] > 1 and (stride[rows_axis] < shape[k_axis] or (stride[rows_axis] * esz) % 16 != 0):
        return False
    if t.dim() == 3 and shape[0] > 1 and (stride[0] <= 0 or (stride[0] * esz) % 16 != 0):
        return False
    return True


def _pitches(t: torch.Tensor, rows_axis: int, k_axis: int, elems_per_item: int) -> tuple[int, int]:
    """(row pitch, batch stride) of ``t`` in logical elements; 0 where the extent is 1 (the library's dense default)."""
    shape, stride = t.shape, t.stride()
    row = stride[rows_axis] * elems_per_item if shape[rows_axis] > 1 else 0
    batch = stride[0] * elems_per_item if (t.dim() == 3 and shape[0] > 1) else 0
    return row, batch


class BlockScaledGemmOperator(Operator):
    """Dense (optionally batched) NVFP4 / MXFP8 GEMM, fp32 accumulation, bf16 or NVFP4 output.
    Takes the place of ``PersistentDenseBlockScaledGemmOperator``
    (``operators/cutlass/operators/providers/cutedsl/gemm/sm100_dense_blockscaled_static_persistent.py:80``)."""

    supported_args_type = GemmArguments

    def _supports(self, args: GemmArguments) -> Status:
        md = self._metadata
        ps = args.problem_size
        if args.accumulator_type not in (torch.float32, float, "float32"):
            return Status.fail(f"accumulator type {args.accumulator_type} is not supported (fp32 only)")
        st = self._check_scaled_pair(args.A, args.B, (ps.L, ps.M, ps.K), (ps.L, ps.N, ps.K), ps.K)
        if not st:
            return st
        if not _k_major_rows(args.A.quantized.tensor, -2, -1):
            return Status.fail("A must be K-major (row-major (L, M, K)) with 16-byte aligned rows and batch entries")
        if not _k_major_rows(args.B.quantized.tensor, -1, -2):
            return Status.fail("B must be K-major: build it as (L, N, K) and transpose the last two dimensions")
        epi = args.epilogue or EpilogueDescriptor()
        out = args.out.tensor
        if not _k_major_rows(out, -2, -1):
            return Status.fail("out must be row-major with 16-byte aligned rows")
        if epi.out_quant is None:
            if out.dtype not in _PLAIN_OUT_KINDS:
                return Status.fail(f"out dtype {out.dtype} is not supported (bf16, fp16, fp32, e4m3, e5m2, or a quantised output with out_quant)")
            if out.dtype != torch.bfloat16 and (md.tile_n in (64, 192) or md.cta_group != 2 or md.kind > L.KIND_MXFP8):
                return Status.fail(f"{out.dtype} output is available with the 2-CTA tiles of 128 / 256 columns, NVFP4 or MXFP8 operands")
            if ps.N % _PLAIN_OUT_N_MULTIPLE[out.dtype] != 0:
                return Status.fail(f"N must be a multiple of {_PLAIN_OUT_N_MULTIPLE[out.dtype]} for {out.dtype} output (16-byte rows)")
        elif isinstance(epi.out_quant, Mxfp8Quant):
            if out.dtype not in (torch.uint8, torch.float8_e4m3fn):
                return Status.fail("MXFP8 output needs a uint8 / float8_e4m3fn out tensor")
            if ps.L != 1:
                return Status.fail("MXFP8 output is not batched")
            if ps.N % 32 != 0:
                return Status.fail("N must be a multiple of 32 for MXFP8 output")
            want = ScaledOperand.numel_scale((ps.L, ps.M, ps.N), ScaleMode.Blockwise1x32, ScaleSwizzleMode.Swizzle32x4x4)
            if epi.out_quant.scale.numel() != want or not epi.out_quant.scale.is_contiguous():
                return Status.fail(f"out_quant.scale must be contiguous with {want} elements")
            nc = epi.out_quant.norm_constant
            if nc is not None and (nc.numel() != 1 or nc.dtype != torch.float32):
                return Status.fail("out_quant.norm_constant must be a one-element float32 tensor")
        else:
            if not (out.dtype == torch.uint8 or (_FP4X2 is not None and out.dtype == _FP4X2)):
                return Status.fail("NVFP4 output needs a packed fp4 (uint8 / float4_e2m1fn_x2) out tensor")
            if ps.N % 32 != 0:
                return Status.fail("N must be a multiple of 32 for NVFP4 output")
            want = ScaledOperand.numel_scale((ps.L, ps.M, ps.N), ScaleMode.Blockwise1x16, ScaleSwizzleMode.Swizzle32x4x4)
            if epi.out_quant.scale.numel() != want or not epi.out_quant.scale.is_contiguous():
                return Status.fail(f"out_quant.scale must be contiguous with {want} elements")
            nc = epi.out_quant.norm_constant
            if nc.numel() != 1 or nc.dtype != torch.float32:
                return Status.fail("out_quant.norm_constant must be a one-element float32 tensor")
        if epi.C is not None:
            if epi.C.dtype != torch.bfloat16 or tuple(epi.C.shape) != (tuple(out.shape[:-1]) + (ps.N,)) or not _k_major_rows(epi.C, -2, -1):
                return Status.fail("C must be a row-major bf16 tensor of the logical output shape (16-byte aligned rows)")
        else:
            beta = epi.beta
            if not isinstance(beta, torch.Tensor) and float(beta) != 0.0:
                return Status.fail("beta != 0 needs C")
        if epi.activation not in ACTIVATIONS:
            return Status.fail(f"unknown activation {epi.activation!r}: one of {sorted(ACTIVATIONS)}")
        if epi.bias is not None:
            want = ps.M if epi.bias_per_row else ps.N
            if epi.bias.dtype != torch.float32 or epi.bias.numel() != want or not epi.bias.is_contiguous():
                return Status.fail(f"bias must be a contiguous fp32 vector of {want} entries")
        if md.tile_n not in (64, 128, 192, 256) or md.cta_group not in (1, 2):
            return Status.fail("invalid tile configuration")
        return Status.success()

    def build_args(self, args: GemmArguments) -> L.GemmArgs:
        md = self._metadata
        ps = args.problem_size
        epi = args.epilogue or EpilogueDescriptor()
        a = L.GemmArgs()
        a.kind = md.kind
        a.out_kind = _plain_out_kind(args.out.tensor) if epi.out_quant is None else (L.OUT_MXFP8 if isinstance(epi.out_quant, Mxfp8Quant) else L.OUT_NVFP4)
        a.batch = ps.L
        a.M, a.N, a.K = ps.M, ps.N, ps.K
        a.A = args.A.quantized.data_ptr()
        a.B = args.B.quantized.data_ptr()
        a.SFA = args.A.scale.data_ptr()
        a.SFB = args.B.scale.data_ptr()
        a.C = epi.C.data_ptr() if epi.C is not None else None
        a.D = args.out.data_ptr()
        # Row pitches and batch strides, in logical elements (a packed fp4 byte holds two)
        a_fp4 = 2 if args.A.is_packed_fp4 else 1
        b_fp4 = 2 if args.B.is_packed_fp4 else 1
        d_fp4 = 2 if (epi.out_quant is not None and not isinstance(epi.out_quant, Mxfp8Quant)) else 1
        a.lda, a.batch_stride_A = _pitches(args.A.quantized.tensor, -2, -1, a_fp4)
        a.ldb, a.batch_stride_B = _pitches(args.B.quantized.tensor, -1, -2, b_fp4)
        a.ldd, a.batch_stride_D = _pitches(args.out.tensor, -2, -1, d_fp4)
        if epi.C is not None:
            a.ldc, a.batch_stride_C = _pitches(epi.C, -2, -1, 1)
        a.alpha, alpha_ptr = _scalar_ptr(epi.alpha)
        a.beta, beta_ptr = _scalar_ptr(epi.beta)
        a.alpha_ptr = alpha_ptr
        a.beta_ptr = beta_ptr
        if epi.out_quant is not None:
            a.SFD = epi.out_quant.scale.data_ptr()
            nc = epi.out_quant.norm_constant
            a.norm_constant = nc.data_ptr() if nc is not None else None
        if epi.bias is not None:
            a.bias = epi.bias.data_ptr()
            a.bias_mode = L.BIAS_PER_ROW if epi.bias_per_row else L.BIAS_PER_COLUMN
        a.activation = ACTIVATIONS[epi.activation]
        a.tile_n = md.tile_n
        a.cta_group = md.cta_group
        return a

    def _run(self, args: GemmArguments, artifact: CompiledArtifact, stream: int, workspace) -> None:
        ws = self._resolve_workspace(workspace, args.out.tensor.device)
        a = self.build_args(args)
        L.check(artifact.library.bsg_gemm_run(C.byref(a), ws.data_ptr(), ws.numel() * ws.element_size(), stream))


class GroupedBlockScaledGemmOperator(Operator):
    """Grouped (MoE) block-scaled GEMM with ragged per-group M over contiguous rows.
    API shape of the reference's contiguous-offset grouped operator
    (``operators/cutlass/operators/providers/cutedsl/gemm/sm100_contiguous_offset_2d3d_dense_gemm.py``),
    arithmetic of its block-scaled grouped kernels
    (``include/cutlass/gemm/collective/sm100_blockscaled_mma_array_warpspecialized.hpp``)."""

    supported_args_type = GroupedGemmArguments

    def _supports(self, args: GroupedGemmArguments) -> Status:
        ps = args.problem_size
        if args.accumulator_type not in (torch.float32, float, "float32"):
            return Status.fail(f"accumulator type {args.accumulator_type} is not supported (fp32 only)")
        if ps.L > L.MAX_GROUPS:
            return Status.fail(f"at most {L.MAX_GROUPS} groups are supported, got {ps.L}")
        if not isinstance(args.A, ScaledOperand) or not isinstance(args.B, ScaledOperand):
            return Status.fail("A and B must be ScaledOperand (block-scaled GEMM)")
        # The A-side scale tensor is per group and padded: its exact size depends on the offsets
        # (device data), so only a lower / upper bound can be checked here.
        vec = ScaleMode.numel(args.A.mode)
        k_blocks4 = -(-(-(-ps.K // vec)) // 4) * 4
        lo = -(-ps.M // 128) * 128 * k_blocks4
        hi = (ps.M // 128 + ps.L) * 128 * k_blocks4
        if not (lo <= args.A.scale.numel() <= hi):
            return Status.fail(f"A: scale tensor has {args.A.scale.numel()} elements, expected between {lo} and {hi} "
                               "(one 128-row-padded layout per group)")
        fake_a_rows = args.A.scale.numel() // k_blocks4
        st = self._check_scaled_pair(args.A, args.B, (1, fake_a_rows, ps.K), (ps.L, ps.N, ps.K), ps.K)
        if not st:
            return st
        if not _k_major_rows(args.A.quantized.tensor, -2, -1):
            return Status.fail("A must be K-major (row-major (TotalM, K)) and densely packed")
        if not _k_major_rows(args.B.quantized.tensor, -1, -2):
            return Status.fail("B must be K-major: build it as (groups, N, K) and transpose the last two dimensions")
        out = args.out.tensor
        epi = args.epilogue or EpilogueDescriptor()
        if not out.is_contiguous():
            return Status.fail("out must be contiguous")
        if epi.out_quant is None:
            if out.dtype not in _PLAIN_OUT_KINDS:
                return Status.fail("out must be a bf16, fp16, fp32, e4m3 or e5m2 tensor (or a quantised output with out_quant)")
            if out.dtype != torch.bfloat16 and (self._metadata.tile_n in (64, 192) or self._metadata.cta_group != 2 or self._metadata.kind > L.KIND_MXFP8):
                return Status.fail(f"{out.dtype} output is available with the 2-CTA tiles of 128 / 256 columns, NVFP4 or MXFP8 operands")
            if ps.N % _PLAIN_OUT_N_MULTIPLE[out.dtype] != 0:
                return Status.fail(f"N must be a multiple of {_PLAIN_OUT_N_MULTIPLE[out.dtype]} for {out.dtype} output")
        else:
            # one interleaved scale layout per group, each padded to 128 rows: the form the next grouped GEMM takes as SFA
            mx = isinstance(epi.out_quant, Mxfp8Quant)
            vec_out = 32 if mx else 16
            if ps.N % 32 != 0:
                return Status.fail("N must be a multiple of 32 for a quantised output")
            n_blocks4 = -(-(ps.N // vec_out) // 4) * 4
            lo_sfd, hi_sfd = -(-ps.M // 128) * 128 * n_blocks4, (ps.M // 128 + ps.L) * 128 * n_blocks4
            if not (lo_sfd <= epi.out_quant.scale.numel() <= hi_sfd) or not epi.out_quant.scale.is_contiguous():
                return Status.fail(f"out_quant.scale must be contiguous with between {lo_sfd} and {hi_sfd} elements "
                                   "(one 128-row-padded layout per group)")
            nc = epi.out_quant.norm_constant
            if (nc is None and not mx) or (nc is not None and (nc.numel() != 1 or nc.dtype != torch.float32)):
                return Status.fail("out_quant.norm_constant must be a one-element float32 tensor")
        for name, v in (("alpha", epi.alpha), ("beta", epi.beta)):
            if isinstance(v, torch.Tensor) and (v.dtype != torch.float32 or v.numel() != ps.L or not v.is_contiguous()):
                return Status.fail(f"grouped GEMM takes a scalar {name} or a contiguous fp32 tensor with one entry per group ({ps.L})")
        if epi.C is None and (isinstance(epi.beta, torch.Tensor) or float(epi.beta) != 0.0):
            return Status.fail("beta != 0 needs C")
        if not args.offsets.tensor.is_contiguous():
            return Status.fail("offsets must be contiguous")
        if epi.activation not in ACTIVATIONS:
            return Status.fail(f"unknown activation {epi.activation!r}: one of {sorted(ACTIVATIONS)}")
        if epi.bias is not None:
            if epi.bias_per_row:
                return Status.fail("grouped GEMM takes a per-column bias only")
            if epi.bias.dtype != torch.float32 or epi.bias.numel() != ps.L * ps.N or not epi.bias.is_contiguous():
                return Status.fail(f"bias must be a contiguous fp32 tensor of shape ({ps.L}, {ps.N})")
        return Status.success()

    def build_args(self, args: GroupedGemmArguments) -> L.GroupedArgs:
        md = self._metadata
        ps = args.problem_size
        epi = args.epilogue or EpilogueDescriptor()
        a = L.GroupedArgs()
        a.kind = md.kind
        a.out_kind = _plain_out_kind(args.out.tensor) if epi.out_quant is None else (L.OUT_MXFP8 if isinstance(epi.out_quant, Mxfp8Quant) else L.OUT_NVFP4)
        if epi.out_quant is not None:
            a.SFD = epi.out_quant.scale.data_ptr()
            a.norm_constant = epi.out_quant.norm_constant.data_ptr() if epi.out_quant.norm_constant is not None else None
        a.num_groups = ps.L
        a.total_M, a.N, a.K = ps.M, ps.N, ps.K
        a.A = args.A.quantized.data_ptr()
        a.B = args.B.quantized.data_ptr()
        a.SFA = args.A.scale.data_ptr()
        a.SFB = args.B.scale.data_ptr()
        a.C = epi.C.data_ptr() if epi.C is not None else None
        a.D = args.out.data_ptr()
        a.offsets = args.offsets.data_ptr()
        a.ldc = ps.N
        a.ldd = ps.N
        if isinstance(epi.alpha, torch.Tensor):
            a.alpha, a.alpha_array = 1.0, epi.alpha.data_ptr()
        else:
            a.alpha = float(epi.alpha)
        if isinstance(epi.beta, torch.Tensor):
            a.beta, a.beta_array = 0.0, epi.beta.data_ptr()
        else:
            a.beta = float(epi.beta)
        a.bias = epi.bias.data_ptr() if epi.bias is not None else None
        a.activation = ACTIVATIONS[epi.activation]
        a.tile_n = md.tile_n
        a.cta_group = md.cta_group
        return a

    def _run(self, args: GroupedGemmArguments, artifact: CompiledArtifact, stream: int, workspace) -> None:
        ws = self._resolve_workspace(workspace, args.out.tensor.device)
        a = self.build_args(args)
        L.check(artifact.library.bsg_grouped_run(C.byref(a), ws.data_ptr(), ws.numel() * ws.element_size(), stream))


_TILE_CHOICES = ((2, 256), (2, 128), (1, 256), (1, 128), (2, 192), (2, 64))   # (cta_group, tile_n), best first; the last two
# (the reference's mma_tiler_n also takes 64 and 192) exist for the two main kinds and unquantised-type-bf16 / re-quantised outputs


def _name(kind: int, grouped: bool, cg: int, tn: int) -> str:
    fmt = {L.KIND_NVFP4: "nvfp4_ue4m3x16", L.KIND_MXFP8: "mxfp8_ue8m0x32", L.KIND_MXFP4: "mxfp4_ue8m0x32",
           L.KIND_MXFP8_MXFP4: "mxfp8_mxfp4_ue8m0x32"}[kind]
    fam = "GroupedBlockScaledGemm" if grouped else "BlockScaledGemm"
    return f"native.{fam}_sm100_tn_{fmt}_acc_f32_{cg}cta_tile{128 * cg}x{tn}"


def all_operators() -> list[Operator]:
    """Every operator configuration the library offers."""
    ops: list[Operator] = []
    for kind in (L.KIND_NVFP4, L.KIND_MXFP8, L.KIND_MXFP4, L.KIND_MXFP8_MXFP4):
        for cg, tn in _TILE_CHOICES:
            if kind >= L.KIND_MXFP4 and (cg != 2 or tn in (64, 192)):
                continue          # the two newer kinds are built for the 2-CTA tiles of 128 / 256 columns only
            ops.append(BlockScaledGemmOperator(OperatorMetadata(_name(kind, False, cg, tn), kind, tn, cg, False)))
            ops.append(GroupedBlockScaledGemmOperator(OperatorMetadata(_name(kind, True, cg, tn), kind, tn, cg, True)))
    return ops


class NativeProvider:
    """The one source of operators here: the hand-written sm_100a library.  Takes the place of the reference's
    provider classes (operators/cutlass/operators/providers/provider.py:43) in ``get_operators(providers=...)``."""

    name = "native"

    @staticmethod
    def operators() -> list["Operator"]:
        return all_operators()


def get_operators(args=None, metadata_filter: Callable[[OperatorMetadata], bool] | None = None,
                  target_sm: str | None = None, providers: list | None = None) -> list[Operator]:
    """Operators that can run ``args`` (all operators when ``args`` is None), best first.  Same parameters as the
    reference's ``get_operators`` (operators/cutlass/operators/__init__.py:72); ``providers`` restricts discovery to the
    listed providers, of which this package has one (``NativeProvider``)."""
    if providers is not None and NativeProvider not in providers and not any(isinstance(p, NativeProvider) for p in providers):
        return []
    out = []
    for op in all_operators():
        if metadata_filter is not None and not metadata_filter(op.metadata):
            continue
        if args is not None and not op.supports(args, target_sm=target_sm):
            continue
        out.append(op)
    return out
