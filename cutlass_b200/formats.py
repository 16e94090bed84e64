"""Narrow-precision codecs and the interleaved scale-factor layout (host side, numpy).

Element formats of the block-scaled GEMM path:

* ``e2m1``  4-bit float {0,.5,1,1.5,2,3,4,6} with sign; two per byte, the even
  K index in the low nibble (reference: ``include/cutlass/float_subbyte.h:81``,
  packing as in ``python/CuTeDSL/cutlass/utils/gemm/tensor_utils.py:337-339``).
* ``e4m3``  8-bit float, bias 7, max 448, 0x7F/0xFF NaN, no Inf
  (``include/cutlass/float8.h``; encode is round-to-nearest-even with
  saturation to the largest finite value, ``include/cutlass/exmy_base.h:640-845``).
* ``ue4m3`` the unsigned e4m3 used for NVFP4 scale factors
  (``include/cutlass/float8.h:1083-1140``).
* ``ue8m0`` power-of-two scale 2^(e-127); 0xFF is NaN; encode rounds up
  (``include/cutlass/float8.h:1163-1259``).

Scale factors live in memory in 512-byte atoms of 128 rows x 4 K-blocks
(``include/cutlass/detail/sm100_blockscaled_layout.hpp:49-114``): K-atoms vary
fastest, then row-atoms.  ``sf_offset`` is the byte offset of the scale factor
of (row, k-block).

These helpers prepare operands on the host; the GEMM itself runs only on the
GPU library (``cutlass_b200.lib``).
"""
from __future__ import annotations

import numpy as np

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_LUT = np.concatenate([E2M1_VALUES, -E2M1_VALUES]).astype(np.float32)  # code -> value

SF_ATOM_ROWS = 128
SF_ATOM_KBLOCKS = 4
SF_ATOM_BYTES = 512


def _e4m3_positive_table() -> np.ndarray:
    """Values of the 127 non-NaN non-negative e4m3 codes 0x00..0x7E."""
    codes = np.arange(0x7F, dtype=np.int32)
    e = codes >> 3
    m = codes & 7
    sub = (m / 8.0) * 2.0 ** (-6)
    nor = (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float64))
    return np.where(e == 0, sub, nor).astype(np.float64)


_E4M3_POS = _e4m3_positive_table()
E4M3_MAX = 448.0


def decode_e4m3(codes: np.ndarray) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    mag = codes & 0x7F
    out = np.empty(codes.shape, dtype=np.float32)
    nan = mag == 0x7F
    out[~nan] = _E4M3_POS[mag[~nan]].astype(np.float32)
    out[nan] = np.nan
    return np.where((codes & 0x80) != 0, -out, out).astype(np.float32)


def decode_ue4m3(codes: np.ndarray) -> np.ndarray:
    """Unsigned e4m3 scale factor; bit 7 is not a sign and must be clear."""
    codes = np.asarray(codes, dtype=np.uint8)
    return decode_e4m3(codes & 0x7F)


def decode_ue8m0(codes: np.ndarray) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    out = np.exp2(np.minimum(codes, 254).astype(np.float64) - 127.0).astype(np.float32)
    out = np.where(codes == 0xFF, np.float32(np.nan), out)
    return out.astype(np.float32)


def decode_e2m1_codes(codes: np.ndarray) -> np.ndarray:
    return E2M1_LUT[np.asarray(codes, dtype=np.uint8) & 0xF]


def pack_e2m1(codes: np.ndarray) -> np.ndarray:
    """(..., K) 4-bit codes -> (..., K/2) bytes, even index in the low nibble."""
    codes = np.asarray(codes, dtype=np.uint8)
    assert codes.shape[-1] % 2 == 0
    return (codes[..., 0::2] & 0xF) | ((codes[..., 1::2] & 0xF) << 4)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


def _round_to_grid(mag: np.ndarray, grid: np.ndarray) -> np.ndarray:
    """Index of the nearest grid value, ties to the even index, clamped (satfinite)."""
    mag = np.asarray(mag, dtype=np.float64)
    hi = np.searchsorted(grid, mag, side="left")
    hi = np.clip(hi, 0, len(grid) - 1)
    lo = np.clip(hi - 1, 0, len(grid) - 1)
    dlo = mag - grid[lo]
    dhi = grid[hi] - mag
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((hi & 1) == 0))
    idx = np.where(pick_hi, hi, lo)
    idx = np.where(mag >= grid[-1], len(grid) - 1, idx)
    return idx.astype(np.uint8)


def encode_e4m3(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3, round-to-nearest-even, saturating; NaN of either sign -> 0x7F (as the reference's float_e4m3_t)."""
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x).astype(np.uint8)) << 7
    mag = np.abs(x).astype(np.float64)
    nan = np.isnan(mag)
    idx = _round_to_grid(np.where(nan, 0.0, mag), _E4M3_POS)
    return np.where(nan, 0x7F, idx | sign).astype(np.uint8)


def _e5m2_positive_table() -> np.ndarray:
    """Values of the 124 finite non-negative e5m2 codes 0x00..0x7B (0x7C is infinity, 0x7D..0x7F NaN)."""
    codes = np.arange(0x7C, dtype=np.int32)
    e = codes >> 2
    m = codes & 3
    sub = (m / 4.0) * 2.0 ** (-14)
    nor = (1.0 + m / 4.0) * np.exp2((e - 15).astype(np.float64))
    return np.where(e == 0, sub, nor).astype(np.float64)


_E5M2_POS = _e5m2_positive_table()
E5M2_MAX = 57344.0


def decode_e5m2(codes: np.ndarray) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    mag = (codes & 0x7F).astype(np.int32)
    out = np.full(codes.shape, np.nan, dtype=np.float32)
    fin = mag < 0x7C
    out[fin] = _E5M2_POS[mag[fin]].astype(np.float32)
    out[mag == 0x7C] = np.inf
    return np.where((codes & 0x80) != 0, -out, out).astype(np.float32)


def encode_e5m2(x: np.ndarray) -> np.ndarray:
    """float32 -> e5m2, round-to-nearest-even, saturating to the largest finite value (infinity too); NaN -> 0x7F
    of either sign: the conversion of the reference's float_e5m2_t and of cvt.rn.satfinite.e5m2x2.f32."""
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x).astype(np.uint8)) << 7
    mag = np.abs(x).astype(np.float64)
    nan = np.isnan(mag)
    idx = _round_to_grid(np.where(nan, 0.0, mag), _E5M2_POS)
    return np.where(nan, 0x7F, idx | sign).astype(np.uint8)


def encode_ue4m3(x: np.ndarray) -> np.ndarray:
    """float32 -> unsigned e4m3 scale factor (the sign of the input is dropped)."""
    x = np.asarray(x, dtype=np.float32)
    nan = np.isnan(x)
    mag = np.where(nan, 0.0, np.abs(x)).astype(np.float64)
    idx = _round_to_grid(mag, _E4M3_POS)
    return np.where(nan, 0x7F, idx).astype(np.uint8)


def encode_e2m1(x: np.ndarray) -> np.ndarray:
    """float32 -> 4-bit e2m1 code, round-to-nearest-even, saturating at 6."""
    x = np.asarray(x, dtype=np.float32)
    sign = np.signbit(x).astype(np.uint8) << 3
    mag = np.abs(np.nan_to_num(x, nan=0.0)).astype(np.float64)
    idx = _round_to_grid(mag, E2M1_VALUES.astype(np.float64))
    return (idx | sign).astype(np.uint8)


def encode_ue8m0(x: np.ndarray) -> np.ndarray:
    """float32 -> ue8m0, rounding the magnitude up to the next power of two."""
    x = np.asarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    exp = ((bits >> 23) & 0xFF).astype(np.int32)
    mant = (bits & 0x7FFFFF).astype(np.uint32)
    bump = (mant > 0) & (exp != 0xFE) & ~((exp == 0) & (mant <= 0x00400000))
    out = np.where(bump, exp + 1, exp)
    out = np.where(np.isnan(x) | np.isinf(x), 0xFF, out)
    return out.astype(np.uint8)


# ---------------------------------------------------------------------------
# Interleaved scale-factor layout
# ---------------------------------------------------------------------------

def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def sf_k_atoms(K: int, vec: int) -> int:
    return ceil_div(ceil_div(K, vec), SF_ATOM_KBLOCKS)


def numel_scale(rows: int, K: int, vec: int, batch: int = 1) -> int:
    """Bytes (= elements) of the interleaved scale tensor, padding included
    (``operators/cutlass/operators/arguments/operand.py:225-231``)."""
    return batch * ceil_div(rows, SF_ATOM_ROWS) * SF_ATOM_ROWS * sf_k_atoms(K, vec) * SF_ATOM_KBLOCKS


def sf_offset(row, kblock, k_atoms: int):
    """Byte offset of the scale factor of (row, kblock); numpy-broadcastable."""
    row = np.asarray(row, dtype=np.int64)
    kblock = np.asarray(kblock, dtype=np.int64)
    return ((row // 128) * (SF_ATOM_BYTES * k_atoms) + (kblock // 4) * SF_ATOM_BYTES
            + 16 * (row % 32) + 4 * ((row % 128) // 32) + (kblock % 4))


def swizzle_sf(sf: np.ndarray, pad_value: int = 0) -> np.ndarray:
    """(rows, kblocks) uint8 scale codes -> flat interleaved buffer."""
    sf = np.asarray(sf, dtype=np.uint8)
    rows, kblocks = sf.shape
    k_atoms = ceil_div(kblocks, SF_ATOM_KBLOCKS)
    out = np.full(ceil_div(rows, 128) * 128 * k_atoms * 4, pad_value, dtype=np.uint8)
    r = np.arange(rows)[:, None]
    kb = np.arange(kblocks)[None, :]
    out[sf_offset(r, kb, k_atoms)] = sf
    return out


def unswizzle_sf(buf: np.ndarray, rows: int, kblocks: int) -> np.ndarray:
    """Flat interleaved buffer -> (rows, kblocks) uint8 scale codes."""
    buf = np.asarray(buf, dtype=np.uint8).reshape(-1)
    k_atoms = ceil_div(kblocks, SF_ATOM_KBLOCKS)
    r = np.arange(rows)[:, None]
    kb = np.arange(kblocks)[None, :]
    return buf[sf_offset(r, kb, k_atoms)]


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bf16, returned as uint16 bit patterns."""
    x = np.asarray(x, dtype=np.float32)
    b = x.view(np.uint32).astype(np.uint64)
    rounded = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    return np.where(nan, np.uint16(0x7FC0), rounded).astype(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
