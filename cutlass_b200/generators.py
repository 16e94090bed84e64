"""Seeded synthetic operands for the benchmark configurations and the tests.

Value distributions:

* NVFP4 data: e2m1 codes drawn uniformly from the 15 distinct values
  {0, +-0.5, +-1, +-1.5, +-2, +-3, +-4, +-6} (-0 is never produced);
  ue4m3 scale factors uniform over the exponents 2^-2 .. 2^2 with zero mantissa,
  i.e. codes {0x28, 0x30, 0x38, 0x40, 0x48} = {0.25, 0.5, 1, 2, 4}.
* MXFP8 data: N(0, 1) rounded to e4m3 (nearest even, saturating);
  ue8m0 scale factors with exponents uniform in [-3, 3] (codes 124 .. 130).

All generators return numpy arrays in the memory layout the library consumes:
packed K-major data and the interleaved scale-factor buffer.
"""
from __future__ import annotations

import numpy as np

from . import formats as F

_E2M1_15 = np.array([0, 1, 2, 3, 4, 5, 6, 7, 9, 10, 11, 12, 13, 14, 15], dtype=np.uint8)
_UE4M3_POW2 = np.array([0x28, 0x30, 0x38, 0x40, 0x48], dtype=np.uint8)


def nvfp4_operand(rows: int, K: int, rng: np.random.Generator):
    """-> (packed (rows, K/2) uint8, sf codes (rows, K/16) uint8, interleaved sf buffer)."""
    codes = _E2M1_15[rng.integers(0, 15, size=(rows, K), dtype=np.uint8)]
    packed = F.pack_e2m1(codes)
    sf = _UE4M3_POW2[rng.integers(0, 5, size=(rows, F.ceil_div(K, 16)), dtype=np.uint8)]
    return packed, sf, F.swizzle_sf(sf)


def mxfp8_operand(rows: int, K: int, rng: np.random.Generator):
    """-> (e4m3 codes (rows, K) uint8, sf codes (rows, K/32) uint8, interleaved sf buffer)."""
    x = rng.standard_normal(size=(rows, K), dtype=np.float32)
    codes = F.encode_e4m3(x)
    sf = rng.integers(124, 131, size=(rows, F.ceil_div(K, 32)), dtype=np.uint8)
    return codes, sf, F.swizzle_sf(sf)


def mxfp4_operand(rows: int, K: int, rng: np.random.Generator):
    """MXFP4: the 15 distinct e2m1 values with ue8m0 scale factors per 32 elements, exponents uniform in [-3, 3].
    -> (packed (rows, K/2) uint8, sf codes (rows, K/32) uint8, interleaved sf buffer)."""
    codes = _E2M1_15[rng.integers(0, 15, size=(rows, K), dtype=np.uint8)]
    sf = rng.integers(124, 131, size=(rows, F.ceil_div(K, 32)), dtype=np.uint8)
    return F.pack_e2m1(codes), sf, F.swizzle_sf(sf)


def exact_mxfp4_operand(rows: int, K: int, rng: np.random.Generator):
    """MXFP4 data in {-1, 0, 1} with ue8m0 scales {1, 2, 4}: exact in fp32 in any accumulation order."""
    codes = np.array([0, 2, 10], dtype=np.uint8)[rng.integers(0, 3, size=(rows, K), dtype=np.uint8)]
    sf = np.array([127, 128, 129], dtype=np.uint8)[rng.integers(0, 3, size=(rows, F.ceil_div(K, 32)), dtype=np.uint8)]
    return F.pack_e2m1(codes), sf, F.swizzle_sf(sf)


def operand_generators(kind: int, exact: bool):
    """(generator of A, generator of B) for an operand kind of the library: 0 NVFP4, 1 MXFP8, 2 MXFP4,
    3 mixed (A MXFP8, B MXFP4)."""
    table = {0: (nvfp4_operand, exact_nvfp4_operand), 1: (mxfp8_operand, exact_mxfp8_operand), 2: (mxfp4_operand, exact_mxfp4_operand)}
    if kind == 3:
        return table[1][exact], table[2][exact]
    return table[kind][exact], table[kind][exact]


def exact_nvfp4_operand(rows: int, K: int, rng: np.random.Generator):
    """Data in {-1, 0, 1} with power-of-two scales {1, 2, 4}: fp32 accumulation is exact
    in any order (the trick of operators/test/test_utils/gemm.py:366-403 in the reference)."""
    codes = np.array([0, 2, 10], dtype=np.uint8)[rng.integers(0, 3, size=(rows, K), dtype=np.uint8)]
    packed = F.pack_e2m1(codes)
    sf = np.array([0x38, 0x40, 0x48], dtype=np.uint8)[rng.integers(0, 3, size=(rows, F.ceil_div(K, 16)), dtype=np.uint8)]
    return packed, sf, F.swizzle_sf(sf)


def exact_mxfp8_operand(rows: int, K: int, rng: np.random.Generator):
    """e4m3 data in {-1, 0, 1} (codes 0xB8, 0x00, 0x38) with ue8m0 scales {1, 2, 4}."""
    codes = np.array([0x00, 0x38, 0xB8], dtype=np.uint8)[rng.integers(0, 3, size=(rows, K), dtype=np.uint8)]
    sf = np.array([127, 128, 129], dtype=np.uint8)[rng.integers(0, 3, size=(rows, F.ceil_div(K, 32)), dtype=np.uint8)]
    return codes, sf, F.swizzle_sf(sf)


def bf16_normal(shape, rng: np.random.Generator) -> np.ndarray:
    """N(0,1) rounded to bf16, returned as uint16 bit patterns."""
    return F.bf16_round(rng.standard_normal(size=shape, dtype=np.float32))


def moe_group_sizes(num_experts: int, tokens: int, top_k: int, rng: np.random.Generator, alpha: float = 1.0) -> np.ndarray:
    """Per-expert row counts: expert probabilities ~ Dirichlet(alpha), tokens*top_k
    assignments drawn multinomially.  Sums to tokens*top_k."""
    p = rng.dirichlet(np.full(num_experts, alpha))
    return rng.multinomial(tokens * top_k, p).astype(np.int32)


def grouped_sfa(sf_per_group) -> np.ndarray:
    """Concatenate per-group interleaved scale-factor buffers (each padded to 128 rows)."""
    return np.concatenate([F.swizzle_sf(sf) if sf.shape[0] > 0 else np.zeros(0, np.uint8) for sf in sf_per_group])


# --------------------------------------------------------------------------- generated on the device
def gpu_nvfp4_operand(rows: int, K: int, gen, device):
    """Seeded NVFP4 operand generated on the device (full-size benchmark inputs): the 15 distinct e2m1
    values (no -0), ue4m3 scales in {0.25, 0.5, 1, 2, 4}.  -> (packed (rows, K/2) uint8, interleaved scales)."""
    import torch
    from . import formats as F
    lut = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 9, 10, 11, 12, 13, 14, 15], dtype=torch.uint8, device=device)
    codes = lut[torch.randint(0, 15, (rows, K), device=device, generator=gen)]
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    sfl = torch.tensor([0x28, 0x30, 0x38, 0x40, 0x48], dtype=torch.uint8, device=device)
    sf = sfl[torch.randint(0, 5, (F.numel_scale(rows, K, 16),), device=device, generator=gen)]
    return packed, sf


def gpu_mxfp8_operand(rows: int, K: int, gen, device):
    """Seeded MXFP8 operand generated on the device: N(0,1) rounded to e4m3, ue8m0 scale exponents uniform in [-3, 3]."""
    import torch
    from . import formats as F
    data = torch.randn((rows, K), device=device, generator=gen).to(torch.float8_e4m3fn).view(torch.uint8)
    sf = torch.randint(124, 131, (F.numel_scale(rows, K, 32),), dtype=torch.uint8, device=device, generator=gen)
    return data, sf
