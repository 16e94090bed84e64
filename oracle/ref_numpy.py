"""TEST INFRASTRUCTURE -- numpy restatement of the reference's host block-scaled GEMM.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline leg of ``bench.py`` may
import this module; the library itself never does.

Follows, in the reference tree (NVIDIA CUTLASS):

* ``tools/util/include/cutlass/util/reference/host/gett.hpp:517-604`` (mainloop:
  ``a = float(A) * float(SFA)``, ``b = float(B) * float(SFB)``, fp32 accumulate),
* ``gett.hpp:690-800`` (epilogue: ``out = alpha * acc``, then ``out = beta * C + out``,
  conversion to the output type),
* ``gett.hpp:364-481`` (``compute_1d_scaling_factor_and_quantized_output``),
* ``include/cutlass/detail/sm100_blockscaled_layout.hpp:49-114`` (scale-factor layout),
* ``include/cutlass/float8.h:1083-1259``, ``include/cutlass/float_subbyte.h:81``,
  ``include/cutlass/exmy_base.h:640-845`` (element formats).

It is written independently of ``cutlass_b200.formats`` so that the two can check
each other.  Accumulation uses numpy's fp32 matmul (summation order differs from the
reference's sequential-k loop; the C oracle in ``oracle/bsg_oracle.c`` keeps that
order).  Pinned against the compiled reference (``oracle/_ref``) and the golden
vectors in ``tests/golden`` by ``tests/test_oracle.py``.
"""
from __future__ import annotations

import numpy as np

FLT_MAX = np.float32(3.4028234663852886e38)


# --------------------------------------------------------------------------- decode
def _fp8_e4m3_value(code: int) -> float:
    s = -1.0 if code & 0x80 else 1.0
    e = (code >> 3) & 0xF
    m = code & 7
    if e == 0xF and m == 7:
        return float("nan")
    if e == 0:
        return s * (m / 8.0) * 2.0 ** -6
    return s * (1.0 + m / 8.0) * 2.0 ** (e - 7)


E4M3_TABLE = np.array([_fp8_e4m3_value(c) for c in range(256)], dtype=np.float32)
UE4M3_TABLE = np.array([_fp8_e4m3_value(c & 0x7F) for c in range(256)], dtype=np.float32)
UE8M0_TABLE = np.array([float("nan") if c == 255 else 2.0 ** (c - 127) for c in range(256)], dtype=np.float64).astype(np.float32)
E2M1_TABLE = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


def sf_index(rows: int, kblocks: int) -> np.ndarray:
    """(rows, kblocks) array of byte offsets into the interleaved scale-factor buffer."""
    k_atoms = -(-kblocks // 4)
    r = np.arange(rows, dtype=np.int64)[:, None]
    kb = np.arange(kblocks, dtype=np.int64)[None, :]
    return (r // 128) * (512 * k_atoms) + (kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (kb % 4)


def decode_operand(kind: int, packed: np.ndarray, sf_buf: np.ndarray, rows: int, K: int, is_b: bool = False) -> np.ndarray:
    """Packed operand + interleaved scale factors -> (rows, K) fp32 of value * scale.
    kind 0 NVFP4, 1 MXFP8, 2 MXFP4 (e2m1 with ue8m0 per 32), 3 mixed (A as kind 1, B as kind 2)."""
    packed = np.asarray(packed, dtype=np.uint8).reshape(rows, -1)
    if kind == 0 or kind == 2 or (kind == 3 and is_b):
        vals = np.empty((rows, K), dtype=np.float32)
        vals[:, 0::2] = E2M1_TABLE[packed & 0xF]
        vals[:, 1::2] = E2M1_TABLE[packed >> 4]
    else:
        vals = E4M3_TABLE[packed]
    vec, table = (16, UE4M3_TABLE) if kind == 0 else (32, UE8M0_TABLE)
    kblocks = -(-K // vec)
    sf = table[np.asarray(sf_buf, dtype=np.uint8).reshape(-1)[sf_index(rows, kblocks)]]
    return (vals * np.repeat(sf, vec, axis=1)[:, :K]).astype(np.float32)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    b = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    out = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(np.isnan(x), np.uint16(0x7FC0), out).astype(np.uint16)


# --------------------------------------------------------------------------- GEMM
def gemm_fp32(kind, A, SFA, B, SFB, M, N, K, C_bits=None, alpha=1.0, beta=0.0) -> np.ndarray:
    """alpha * (A.SFA)(B.SFB)^T + beta * C in fp32 (before the output conversion)."""
    a = decode_operand(kind, A, SFA, M, K)
    b = decode_operand(kind, B, SFB, N, K, is_b=True)
    acc = (a @ b.T).astype(np.float32)
    out = np.float32(alpha) * acc
    if C_bits is not None and beta != 0.0:
        c = bf16_bits_to_f32(np.asarray(C_bits).reshape(M, N))
        out = (np.float32(beta) * c).astype(np.float32) + out
    return out.astype(np.float32)


# --------------------------------------------------------------------------- quantisation
_E4M3_POS = E4M3_TABLE[:0x7F].astype(np.float64)
_E2M1_POS = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], dtype=np.float64)


def _nearest_even(mag: np.ndarray, grid: np.ndarray) -> np.ndarray:
    mag = np.asarray(mag, dtype=np.float64)
    out = np.zeros(mag.shape, dtype=np.int64)
    for i in range(1, len(grid)):
        mid = 0.5 * (grid[i - 1] + grid[i])
        up = (mag > mid) | ((mag == mid) & (i % 2 == 0))
        out = np.where(up & (out == i - 1), i, out)
    return out


def to_ue4m3(x: np.ndarray) -> np.ndarray:
    return _nearest_even(np.abs(np.asarray(x, dtype=np.float32)), _E4M3_POS).astype(np.uint8)


def to_e2m1(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    return (_nearest_even(np.abs(x), _E2M1_POS) | (np.signbit(x).astype(np.int64) << 3)).astype(np.uint8)


def quantize_rows_nvfp4(x: np.ndarray, st: float):
    """fp32 (M, N) -> (packed e2m1 (M, N/2), interleaved ue4m3 SFD buffer).

    Operation order of gett.hpp:364-481 (row-major branch), every step in fp32.
    """
    x = np.asarray(x, dtype=np.float32)
    M, N = x.shape
    assert N % 16 == 0
    st = np.float32(st)
    scale_down = np.float32(1.0) / np.float32(6.0)
    st_scaled = st * scale_down
    blocks = x.reshape(M, N // 16, 16)
    amax = np.max(np.abs(blocks), axis=2).astype(np.float32)
    pv = (amax * st_scaled).astype(np.float32)
    q = to_ue4m3(pv)
    qf = UE4M3_TABLE[q]
    with np.errstate(divide="ignore", over="ignore", invalid="ignore"):
        rcp = (np.float32(1.0) / qf).astype(np.float32)
        sc = np.minimum((st * rcp).astype(np.float32), FLT_MAX)
        y = (blocks * sc[:, :, None]).astype(np.float32)
    codes = to_e2m1(y.reshape(M, N))
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    nb = N // 16
    k_atoms = -(-nb // 4)
    sfd = np.zeros(-(-M // 128) * 128 * k_atoms * 4, dtype=np.uint8)
    sfd[sf_index(M, nb)] = q
    return packed, sfd
