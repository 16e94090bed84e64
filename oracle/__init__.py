"""TEST INFRASTRUCTURE -- CPU oracles for the block-scaled GEMM path.

* ``ref_numpy``           numpy restatement (BLAS summation order).
* ``libbsg_oracle.so``    plain-C restatement with the reference's sequential-k order
                          (``bsg_oracle.c``), built by ``make -C oracle``.
* ``_ref/libbsg_ref.so``  the reference's own host GEMM compiled from its headers
                          (``ref_driver.cpp``); present only where it was built.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline leg of ``bench.py``
import this package.  The GPU library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "libbsg_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libbsg_ref.so")

_oracle = None
_ref = None


def build(reference_root: str | None = None) -> None:
    """Compile the C oracle and, when the reference tree is present, the reference driver."""
    cmd = ["make", "-C", _HERE, "--no-print-directory"]
    if reference_root:
        cmd.append(f"REF={reference_root}")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + proc.stdout + proc.stderr)


def load_oracle() -> C.CDLL:
    global _oracle
    if _oracle is not None:
        return _oracle
    if not os.path.exists(ORACLE_SO):
        build()
    lib = C.CDLL(ORACLE_SO)
    lib.bsg_oracle_decode.restype = C.c_float
    lib.bsg_oracle_decode.argtypes = [C.c_int, C.c_uint32]
    lib.bsg_oracle_encode.restype = C.c_uint32
    lib.bsg_oracle_encode.argtypes = [C.c_int, C.c_float]
    lib.bsg_oracle_sf_offset.restype = C.c_int64
    lib.bsg_oracle_sf_offset.argtypes = [C.c_int64] * 3
    lib.bsg_oracle_gemm_rows.restype = C.c_int
    lib.bsg_oracle_gemm_rows.argtypes = [C.c_int, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 5 + \
        [C.c_int64, C.c_float, C.c_float, C.c_int64, C.c_int64, C.c_void_p]
    lib.bsg_oracle_gemm_rows_epi.restype = C.c_int
    lib.bsg_oracle_gemm_rows_epi.argtypes = [C.c_int, C.c_int64, C.c_int64, C.c_int64] + [C.c_void_p] * 5 + \
        [C.c_int64, C.c_float, C.c_float, C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_void_p]
    lib.bsg_oracle_activation.restype = C.c_float
    lib.bsg_oracle_activation.argtypes = [C.c_int, C.c_float]
    lib.bsg_oracle_quant_nvfp4.restype = None
    lib.bsg_oracle_quant_nvfp4.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p, C.c_void_p]
    lib.bsg_oracle_quant.restype = None
    lib.bsg_oracle_quant.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p, C.c_void_p]
    lib.bsg_oracle_to_bf16.restype = None
    lib.bsg_oracle_to_bf16.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
    lib.bsg_oracle_threads.restype = C.c_int
    _oracle = lib
    return lib


def load_ref() -> C.CDLL | None:
    """The compiled reference driver, or None where it has not been built."""
    global _ref
    if _ref is not None:
        return _ref
    if not os.path.exists(REF_SO):
        return None
    lib = C.CDLL(REF_SO)
    lib.bsg_ref_decode.restype = C.c_float
    lib.bsg_ref_decode.argtypes = [C.c_int, C.c_uint32]
    lib.bsg_ref_encode.restype = C.c_uint32
    lib.bsg_ref_encode.argtypes = [C.c_int, C.c_float]
    if hasattr(lib, "bsg_ref_gemm_epi"):
        lib.bsg_ref_gemm_epi.restype = C.c_int
        lib.bsg_ref_gemm_epi.argtypes = [C.c_int] * 4 + [C.c_void_p] * 5 + [C.c_float, C.c_float, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.bsg_ref_sf_offset.restype = C.c_int64
    lib.bsg_ref_sf_offset.argtypes = [C.c_int] * 5
    lib.bsg_ref_sf_size.restype = C.c_int64
    lib.bsg_ref_sf_size.argtypes = [C.c_int] * 3
    lib.bsg_ref_gemm.restype = C.c_int
    lib.bsg_ref_gemm.argtypes = [C.c_int] * 5 + [C.c_void_p] * 5 + [C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_float]
    _ref = lib
    return lib


def _ptr(a: np.ndarray | None):
    return None if a is None else a.ctypes.data


def gemm_fp32(kind: int, A, SFA, B, SFB, M: int, N: int, K: int, C_bits=None, alpha: float = 1.0, beta: float = 0.0,
              m_begin: int = 0, m_count: int | None = None, bias=None, bias_per_row: bool = False, activation: int = 0) -> np.ndarray:
    """C oracle: act(alpha * (A.SFA)(B.SFB)^T + bias + beta * C) in fp32 for rows [m_begin, m_begin + m_count).
    activation: 0 identity, 1 ReLU, 2 GELU, 3 SiLU; bias: fp32 vector of N (per column) or M (per row) entries."""
    lib = load_oracle()
    m_count = M - m_begin if m_count is None else m_count
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.uint8)
    SFA = np.ascontiguousarray(SFA, dtype=np.uint8)
    SFB = np.ascontiguousarray(SFB, dtype=np.uint8)
    Cb = None if C_bits is None else np.ascontiguousarray(C_bits, dtype=np.uint16)
    out = np.empty((m_count, N), dtype=np.float32)
    bv = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    if bv is not None and bv.size != (M if bias_per_row else N):
        raise ValueError("bias has the wrong number of entries")
    rc = lib.bsg_oracle_gemm_rows_epi(kind, M, N, K, _ptr(A), _ptr(B), _ptr(SFA), _ptr(SFB), _ptr(Cb), N, alpha, beta,
                                      _ptr(bv), 0 if bv is None else (2 if bias_per_row else 1), int(activation),
                                      m_begin, m_count, _ptr(out))
    if rc != 0:
        raise MemoryError("oracle GEMM could not allocate its scratch buffers")
    return out


def quant_nvfp4(x: np.ndarray, st: float):
    """C oracle: NVFP4 re-quantisation of an fp32 matrix -> (packed e2m1, interleaved ue4m3 SFD)."""
    lib = load_oracle()
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, N = x.shape
    nb = N // 16
    D = np.zeros((M, N // 2), dtype=np.uint8)
    SFD = np.zeros(-(-M // 128) * 128 * (-(-nb // 4)) * 4, dtype=np.uint8)
    lib.bsg_oracle_quant_nvfp4(_ptr(x), M, N, float(st), _ptr(D), _ptr(SFD))
    return D, SFD


def quant(kind: int, x: np.ndarray, st: float = 1.0):
    """C oracle: block-scaled quantisation of an fp32 matrix along its rows -> (values, interleaved scale factors).
    kind 0: packed e2m1 + ue4m3 per 16; kind 1: e4m3 + ue8m0 per 32."""
    lib = load_oracle()
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, N = x.shape
    vec = 16 if kind == 0 else 32
    nb = N // vec
    D = np.zeros((M, N // 2 if kind == 0 else N), dtype=np.uint8)
    SFD = np.zeros(-(-M // 128) * 128 * (-(-nb // 4)) * 4, dtype=np.uint8)
    lib.bsg_oracle_quant(int(kind), _ptr(x), M, N, float(st), _ptr(D), _ptr(SFD))
    return D, SFD


def set_threads(n: int) -> None:
    """Use ``n`` OpenMP threads in the oracle and the compiled reference from now on (launchers such as torchrun
    export OMP_NUM_THREADS=1, which the runtime has already read by the time this module loads)."""
    lib = load_oracle()
    lib.bsg_oracle_set_threads.restype = None
    lib.bsg_oracle_set_threads.argtypes = [C.c_int]
    lib.bsg_oracle_set_threads(int(n))


def to_bf16(x: np.ndarray) -> np.ndarray:
    lib = load_oracle()
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib.bsg_oracle_to_bf16(_ptr(x), x.size, _ptr(out))
    return out


def ref_gemm(kind: int, out_mode: int, A, SFA, B, SFB, M: int, N: int, K: int, C_bits=None, alpha=1.0, beta=0.0, st=0.0):
    """Compiled reference: out_mode 0 fp32, 1 bf16 bits, 2 (packed e2m1, ue4m3 SFD per 16), 3 (e4m3, ue8m0 SFD per 32),
    4 / 5 (NVFP4 operands only): as 2 / 3 with D column-major and the scale factors along M -- returned as the
    transposed matrix (N x M values) and its K-major scale-factor buffer."""
    lib = load_ref()
    if lib is None:
        raise FileNotFoundError("oracle/_ref/libbsg_ref.so has not been built")
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.uint8)
    SFA = np.ascontiguousarray(SFA, dtype=np.uint8)
    SFB = np.ascontiguousarray(SFB, dtype=np.uint8)
    Cb = np.zeros((M, N), dtype=np.uint16) if C_bits is None else np.ascontiguousarray(C_bits, dtype=np.uint16)
    sfd = None
    if out_mode == 0:
        D = np.zeros((M, N), dtype=np.float32)
    elif out_mode == 1:
        D = np.zeros((M, N), dtype=np.uint16)
    elif out_mode == 2:
        D = np.zeros((M, N // 2), dtype=np.uint8)
        nb = N // 16
        sfd = np.zeros(-(-M // 128) * 128 * (-(-nb // 4)) * 4, dtype=np.uint8)
    elif out_mode == 3:
        D = np.zeros((M, N), dtype=np.uint8)
        nb = N // 32
        sfd = np.zeros(-(-M // 128) * 128 * (-(-nb // 4)) * 4, dtype=np.uint8)
    else:
        # column-major D (returned as its transpose: N rows of M values) with scale factors along M
        vec = 16 if out_mode == 4 else 32
        D = np.zeros((N, M // 2 if out_mode == 4 else M), dtype=np.uint8)
        mb = M // vec
        sfd = np.zeros(-(-N // 128) * 128 * (-(-mb // 4)) * 4, dtype=np.uint8)
    rc = lib.bsg_ref_gemm(kind, out_mode, M, N, K, _ptr(A), _ptr(B), _ptr(SFA), _ptr(SFB), _ptr(Cb), alpha, beta, _ptr(D),
                          _ptr(sfd), float(st))
    if rc != 0:
        raise ValueError("reference driver rejected the arguments")
    return D if sfd is None else (D, sfd)


def ref_gemm_epi(kind: int, A, SFA, B, SFB, M: int, N: int, K: int, C_bits=None, alpha=1.0, beta=0.0, bias=None,
                 bias_per_row: bool = False, activation: int = 0) -> np.ndarray:
    """Compiled reference with its general epilogue: fp32 act(alpha * acc + bias + beta * C)."""
    lib = load_ref()
    if lib is None:
        raise FileNotFoundError("oracle/_ref/libbsg_ref.so has not been built")
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.uint8)
    SFA = np.ascontiguousarray(SFA, dtype=np.uint8)
    SFB = np.ascontiguousarray(SFB, dtype=np.uint8)
    Cb = np.zeros((M, N), dtype=np.uint16) if C_bits is None else np.ascontiguousarray(C_bits, dtype=np.uint16)
    bv = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    D = np.zeros((M, N), dtype=np.float32)
    rc = lib.bsg_ref_gemm_epi(kind, M, N, K, _ptr(A), _ptr(B), _ptr(SFA), _ptr(SFB), _ptr(Cb), alpha, beta, _ptr(bv),
                              0 if bv is None else (2 if bias_per_row else 1), int(activation), _ptr(D))
    if rc != 0:
        raise ValueError("reference driver rejected the arguments")
    return D
