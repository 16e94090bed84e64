"""Grouped block-scaled GEMM in the pointer-array form: a list of independent problems, each with its own
(M, N, K) and tensors, run by one kernel launch.

Host-side counterpart of ``bsg_ptr_array_*`` in ``include/bsgemm.h``; takes the role of the reference's grouped GEMM
with ``GroupProblemShape`` (``include/cutlass/gemm/group_array_problem_shape.hpp:55``; device side in
``include/cutlass/gemm/collective/sm100_blockscaled_mma_array_warpspecialized.hpp``), whose arguments are arrays of
per-group pointers, pitches and problem sizes (``tools/library/include/cutlass/library/library.h:558-605``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence


@dataclass
class GroupProblem:
    """One group: ``A`` (M, K) and ``B`` (N, K) K-major packed tensors with their interleaved scale factors, ``D`` the
    (M, N) output (bf16, or packed e2m1 / e4m3 with ``SFD``), ``C`` an optional bf16 addend.  Row pitches are taken
    from the tensors' strides."""
    A: "object"
    SFA: "object"
    B: "object"
    SFB: "object"
    D: "object"
    C: Optional["object"] = None
    SFD: Optional["object"] = None


class PtrArrayGemm:
    """Encodes the per-group table once (``bsg_ptr_array_initialize``) and launches it any number of times."""

    def __init__(self, kind: int, groups: Sequence[GroupProblem], out_kind: int = 0, norm_constant=None, tile_n: int = 0,
                 stream=None):
        import torch
        from . import lib as L
        from .operator import to_cuda_stream
        if not groups:
            raise ValueError("at least one group is needed")
        self._L, self._lib = L, L.load()
        self.kind, self.out_kind, self.groups = kind, out_kind, list(groups)
        n = len(self.groups)
        per_byte = 2 if kind == L.KIND_NVFP4 else 1
        out_per_byte = 2 if out_kind == L.OUT_NVFP4 else 1
        sizes, lda, ldb, ldc, ldd = [], [], [], [], []
        for g in self.groups:
            M, N, K = g.A.shape[0], g.B.shape[0], g.A.shape[1] * per_byte
            if g.B.shape[1] * per_byte != K:
                raise ValueError(f"A and B of a group disagree on K ({K} against {g.B.shape[1] * per_byte})")
            for t in (g.A, g.B, g.D) + ((g.C,) if g.C is not None else ()):
                if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
                    raise ValueError("group tensors must be two-dimensional with a contiguous last dimension")
            sizes += [M, N, K]
            lda.append(g.A.stride(0) * per_byte if M > 1 else K)
            ldb.append(g.B.stride(0) * per_byte if N > 1 else K)
            ldd.append(g.D.stride(0) * out_per_byte if M > 1 else N)
            ldc.append((g.C.stride(0) if M > 1 else N) if g.C is not None else N)
        self.sizes = sizes
        ptrs = lambda ts: (C.c_void_p * n)(*[(t.data_ptr() if t is not None else None) for t in ts])  # noqa: E731
        i64 = lambda v: (C.c_int64 * n)(*v)  # noqa: E731
        self._host = {
            "sizes": (C.c_int32 * (3 * n))(*sizes),
            "A": ptrs([g.A for g in self.groups]), "B": ptrs([g.B for g in self.groups]),
            "SFA": ptrs([g.SFA for g in self.groups]), "SFB": ptrs([g.SFB for g in self.groups]),
            "D": ptrs([g.D for g in self.groups]),
            "C": ptrs([g.C for g in self.groups]) if any(g.C is not None for g in self.groups) else None,
            "SFD": ptrs([g.SFD for g in self.groups]) if out_kind != L.OUT_BF16 else None,
            "lda": i64(lda), "ldb": i64(ldb), "ldc": i64(ldc), "ldd": i64(ldd),
        }
        a = L.PtrArrayArgs()
        a.kind, a.out_kind, a.num_groups = kind, out_kind, n
        a.problem_sizes = C.cast(self._host["sizes"], C.c_void_p)
        for name in ("A", "B", "SFA", "SFB", "D", "C", "SFD", "lda", "ldb", "ldc", "ldd"):
            arr = self._host[name]
            setattr(a, name, C.cast(arr, C.c_void_p) if arr is not None else None)
        a.alpha, a.beta = 1.0, 0.0
        a.norm_constant = norm_constant.data_ptr() if norm_constant is not None else None
        a.tile_n = tile_n
        self._norm = norm_constant
        self.args = a
        need = C.c_size_t()
        L.check(self._lib.bsg_ptr_array_workspace_size(C.byref(a), C.byref(need)))
        dev = self.groups[0].A.device
        self.workspace = torch.zeros(need.value + 128, dtype=torch.uint8, device=dev)
        self._ws_ptr = (self.workspace.data_ptr() + 127) & ~127
        self._ws_bytes = need.value
        L.check(self._lib.bsg_ptr_array_initialize(C.byref(a), self._ws_ptr, self._ws_bytes, to_cuda_stream(stream)))

    def run(self, alpha: float = 1.0, beta: float = 0.0, alpha_array=None, beta_array=None, activation: int = 0,
            use_pdl: bool = False, stream=None) -> None:
        from .operator import to_cuda_stream
        a = self.args
        a.alpha, a.beta = alpha, beta
        a.alpha_array = alpha_array.data_ptr() if alpha_array is not None else None
        a.beta_array = beta_array.data_ptr() if beta_array is not None else None
        a.activation, a.use_pdl = activation, int(use_pdl)
        self._L.check(self._lib.bsg_ptr_array_run(C.byref(a), self._ws_ptr, self._ws_bytes, to_cuda_stream(stream)))

    def check_device_status(self, stream=None) -> None:
        from .operator import to_cuda_stream
        self._L.check(self._lib.bsg_read_device_status(self._ws_ptr, to_cuda_stream(stream)))
