"""ctypes binding of the C ABI in ``include/bsgemm.h``.

The shared library is built in-tree by ``cutlass_b200/build.py`` (nvcc, sm_100a)
as ``cutlass_b200/lib/libbsgemm.so``.  There is no CPU fallback: if the library
is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# BSG_PROFILE=1 selects the instrumented build (python -m cutlass_b200.build with the same variable set).
LIB_PATH = os.path.join(_HERE, "lib", "libbsgemm" + ("_profile" if os.environ.get("BSG_PROFILE") == "1" else "") + ".so")

BSG_OK = 0
STATUS_NAMES = {
    0: "BSG_OK",
    1: "BSG_ERR_MISALIGNED_OPERAND",
    2: "BSG_ERR_INVALID_PROBLEM",
    3: "BSG_ERR_NOT_SUPPORTED",
    4: "BSG_ERR_WORKSPACE_NULL",
    5: "BSG_ERR_INTERNAL",
    6: "BSG_ERR_ARCH_MISMATCH",
    7: "BSG_ERR_TIMEOUT",
    8: "BSG_ERR_CUDA",
}
KIND_NVFP4 = 0
KIND_MXFP8 = 1
KIND_MXFP4 = 2          # e2m1 data, ue8m0 scale per 32
KIND_MXFP8_MXFP4 = 3    # A e4m3, B e2m1, ue8m0 scale per 32
OUT_BF16 = 0
OUT_NVFP4 = 1
OUT_MXFP8 = 2
OUT_F16 = 3
OUT_F32 = 4
OUT_E4M3 = 5
OUT_E5M2 = 6
ACT_IDENTITY, ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2, 3
BIAS_NONE, BIAS_PER_COLUMN, BIAS_PER_ROW = 0, 1, 2
MAX_GROUPS = 256
SCHED_STATIC, SCHED_DYNAMIC = 0, 1
LAYOUT_ROW_MAJOR, LAYOUT_COL_MAJOR = 0, 1
RS_WITH_ALLREDUCE = 1


class GemmArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("out_kind", C.c_int32), ("batch", C.c_int32), ("reserved0", C.c_int32),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("A", C.c_void_p), ("B", C.c_void_p), ("SFA", C.c_void_p), ("SFB", C.c_void_p),
        ("C", C.c_void_p), ("D", C.c_void_p), ("SFD", C.c_void_p),
        ("ldc", C.c_int64), ("ldd", C.c_int64),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("alpha_ptr", C.c_void_p), ("beta_ptr", C.c_void_p), ("norm_constant", C.c_void_p),
        ("tile_n", C.c_int32), ("cta_group", C.c_int32), ("sm_count", C.c_int32), ("raster_band", C.c_int32),
        ("bias", C.c_void_p), ("bias_mode", C.c_int32), ("activation", C.c_int32),
        ("lda", C.c_int64), ("ldb", C.c_int64),
        ("batch_stride_A", C.c_int64), ("batch_stride_B", C.c_int64), ("batch_stride_C", C.c_int64), ("batch_stride_D", C.c_int64),
        ("use_pdl", C.c_int32), ("scheduler", C.c_int32),
        ("cluster_m", C.c_int32), ("cluster_n", C.c_int32), ("cluster_fallback_m", C.c_int32), ("cluster_fallback_n", C.c_int32),
        ("out_layout", C.c_int32), ("reserved1", C.c_int32),
    ]


class GroupedArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("out_kind", C.c_int32), ("num_groups", C.c_int32), ("reserved0", C.c_int32),
        ("total_M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("A", C.c_void_p), ("B", C.c_void_p), ("SFA", C.c_void_p), ("SFB", C.c_void_p),
        ("C", C.c_void_p), ("D", C.c_void_p), ("offsets", C.c_void_p),
        ("ldc", C.c_int64), ("ldd", C.c_int64),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("tile_n", C.c_int32), ("cta_group", C.c_int32), ("sm_count", C.c_int32), ("raster_band", C.c_int32),
        ("bias", C.c_void_p), ("reserved1", C.c_int32), ("activation", C.c_int32),
        ("alpha_array", C.c_void_p), ("beta_array", C.c_void_p),
        ("SFD", C.c_void_p), ("norm_constant", C.c_void_p), ("use_pdl", C.c_int32), ("scheduler", C.c_int32),
    ]


class Caps(C.Structure):
    _fields_ = [
        ("tile_m", C.c_int32), ("tile_n", C.c_int32), ("tile_k", C.c_int32), ("cta_group", C.c_int32),
        ("stages", C.c_int32), ("smem_bytes", C.c_int32), ("num_tiles", C.c_int64),
    ]


class PtrArrayArgs(C.Structure):
    """``bsg_ptr_array_args`` of include/bsgemm.h, field for field (the arrays are HOST arrays)."""
    _fields_ = [
        ("kind", C.c_int32), ("out_kind", C.c_int32), ("num_groups", C.c_int32), ("activation", C.c_int32),
        ("problem_sizes", C.c_void_p),
        ("A", C.c_void_p), ("B", C.c_void_p), ("SFA", C.c_void_p), ("SFB", C.c_void_p), ("C", C.c_void_p), ("D", C.c_void_p), ("SFD", C.c_void_p),
        ("lda", C.c_void_p), ("ldb", C.c_void_p), ("ldc", C.c_void_p), ("ldd", C.c_void_p),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("alpha_array", C.c_void_p), ("beta_array", C.c_void_p), ("norm_constant", C.c_void_p),
        ("tile_n", C.c_int32), ("sm_count", C.c_int32), ("raster_band", C.c_int32), ("use_pdl", C.c_int32),
    ]


# name -> (restype, argtypes); every symbol include/bsgemm.h declares.
class QuantArgs(C.Structure):
    """``bsg_quant_args`` of include/bsgemm.h, field for field."""
    _fields_ = [("kind", C.c_int32), ("use_pdl", C.c_int32), ("rows", C.c_int64), ("K", C.c_int64), ("X", C.c_void_p),
                ("ldx", C.c_int64), ("Q", C.c_void_p), ("SF", C.c_void_p), ("norm_constant", C.c_void_p)]


SYMBOLS = {
    "bsg_version": (C.c_int32, []),
    "bsg_last_error_string": (C.c_char_p, []),
    "bsg_gemm_query": (C.c_int32, [C.POINTER(GemmArgs), C.POINTER(Caps)]),
    "bsg_grouped_query": (C.c_int32, [C.POINTER(GroupedArgs), C.POINTER(Caps)]),
    "bsg_gemm_workspace_size": (C.c_int32, [C.POINTER(GemmArgs), C.POINTER(C.c_size_t)]),
    "bsg_grouped_workspace_size": (C.c_int32, [C.POINTER(GroupedArgs), C.POINTER(C.c_size_t)]),
    "bsg_gemm_run": (C.c_int32, [C.POINTER(GemmArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "bsg_grouped_run": (C.c_int32, [C.POINTER(GroupedArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "bsg_workspace_init": (C.c_int32, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "bsg_read_device_status": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "bsg_gemm_run_static": (C.c_int32, [C.POINTER(GemmArgs), C.c_void_p, C.POINTER(C.c_uint32)]),
    "bsg_ptr_array_workspace_size": (C.c_int32, [C.POINTER(PtrArrayArgs), C.POINTER(C.c_size_t)]),
    "bsg_ptr_array_initialize": (C.c_int32, [C.POINTER(PtrArrayArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "bsg_ptr_array_initialize_from_device": (C.c_int32, [C.POINTER(PtrArrayArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "bsg_ptr_array_run": (C.c_int32, [C.POINTER(PtrArrayArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "bsg_quantize": (C.c_int32, [C.POINTER(QuantArgs), C.c_void_p]),
    "bsg_tp_create": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.POINTER(C.c_void_p), C.c_void_p]),
    "bsg_tp_connect": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "bsg_tp_buffers": (C.c_int32, [C.c_void_p] + [C.POINTER(C.c_void_p)] * 4),
    "bsg_tp_gemm_run": (C.c_int32, [C.c_void_p, C.POINTER(GemmArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "bsg_tp_set_mode": (C.c_int32, [C.c_void_p, C.c_int32]),
    "bsg_tp_destroy": (C.c_int32, [C.c_void_p]),
    "bsg_rs_create": (C.c_int32, [C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.POINTER(C.c_void_p), C.c_void_p]),
    "bsg_rs_connect": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "bsg_rs_gemm_run": (C.c_int32, [C.c_void_p, C.POINTER(GemmArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "bsg_rs_allreduce_run": (C.c_int32, [C.c_void_p, C.POINTER(GemmArgs), C.c_void_p, C.c_size_t, C.c_void_p, C.POINTER(C.c_void_p)]),
    "bsg_rs_destroy": (C.c_int32, [C.c_void_p]),
}

_lib = None


class BsgError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code


def load() -> C.CDLL:
    """Load ``libbsgemm.so`` (once) and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python -m cutlass_b200.build` (needs nvcc); "
            "there is no CPU fallback for the GEMM path")
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().bsg_last_error_string().decode("utf-8", "replace")


def check(code: int) -> None:
    if code != BSG_OK:
        raise BsgError(code, last_error())
