"""Build ``cutlass_b200/lib/libbsgemm.so`` in-tree with nvcc for sm_100a.

Usage: ``python -m cutlass_b200.build [--force]``.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
PROFILE = os.environ.get("BSG_PROFILE") == "1"      # in-kernel timeline capture, separate file


def lib_name(profile: bool) -> str:
    return "libbsgemm" + ("_profile" if profile else "") + ".so"


OUT = os.path.join(_HERE, "lib", lib_name(PROFILE))
SOURCES = ["bsgemm.cu"]
HEADERS = ["gemm_kernel.cuh", "quant_kernel.cuh", "ptx.cuh", os.path.join("..", "..", "include", "bsgemm.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-cudart", "static",
]


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA library if it is missing or older than its sources; return its path."""
    if not force and not _stale():
        return OUT
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    extra = ["-DBSG_PROFILE"] if PROFILE else []
    cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUT] + [os.path.join(CSRC, f) for f in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
