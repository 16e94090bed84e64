"""Host codecs and scale-factor layout against the golden vectors (outputs of the
reference's numeric types and layout functions) and against the C oracle."""
import numpy as np
import pytest

import oracle
from cutlass_b200 import formats as F
from oracle import ref_numpy as R

DECODERS = {0: F.decode_e2m1_codes, 1: F.decode_e4m3, 2: F.decode_ue4m3, 3: F.decode_ue8m0}
ENCODERS = {0: F.encode_e2m1, 1: F.encode_e4m3, 2: F.encode_ue4m3, 3: F.encode_ue8m0}


def _same_float(a, b):
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    return bool(np.all((a == b) | (np.isnan(a) & np.isnan(b))))


@pytest.mark.parametrize("fmt", [0, 1, 2, 3])
def test_decode_every_code_matches_reference(golden, fmt):
    want = golden[f"decode_{fmt}"]
    n = len(want)
    assert _same_float(DECODERS[fmt](np.arange(n, dtype=np.uint8)), want)
    lib = oracle.load_oracle()
    assert _same_float([lib.bsg_oracle_decode(fmt, c) for c in range(n)], want)
    table = {0: R.E2M1_TABLE, 1: R.E4M3_TABLE, 2: R.UE4M3_TABLE, 3: R.UE8M0_TABLE}[fmt]
    assert _same_float(table[:n], want)


@pytest.mark.parametrize("fmt", [0, 1, 2, 3])
def test_encode_matches_reference(golden, fmt):
    x = golden["encode_in"]
    want = golden[f"encode_{fmt}"]
    got = ENCODERS[fmt](x)
    assert np.array_equal(got, want), [(float(x[i]), int(got[i]), int(want[i])) for i in np.nonzero(got != want)[0][:5]]
    lib = oracle.load_oracle()
    got_c = np.array([lib.bsg_oracle_encode(fmt, float(v)) for v in x], dtype=np.uint8)
    assert np.array_equal(got_c, want)


def test_encode_roundtrip_is_identity_on_representable_values():
    codes = np.arange(0x7F, dtype=np.uint8)
    assert np.array_equal(F.encode_e4m3(F.decode_e4m3(codes)), codes)
    assert np.array_equal(F.encode_ue4m3(F.decode_ue4m3(codes)), codes)
    c4 = np.array([0, 1, 2, 3, 4, 5, 6, 7, 9, 10, 11, 12, 13, 14, 15], dtype=np.uint8)
    assert np.array_equal(F.encode_e2m1(F.decode_e2m1_codes(c4)), c4)
    c8 = np.arange(1, 255, dtype=np.uint8)
    assert np.array_equal(F.encode_ue8m0(F.decode_ue8m0(c8)), c8)


def test_saturation_and_specials():
    assert F.encode_e4m3(np.array([1e9, -1e9], np.float32)).tolist() == [0x7E, 0xFE]
    assert F.encode_e2m1(np.array([100.0, -100.0, 0.0], np.float32)).tolist() == [7, 15, 0]
    assert F.encode_ue8m0(np.array([np.inf, np.nan], np.float32)).tolist() == [0xFF, 0xFF]
    assert np.isnan(F.decode_e4m3(np.array([0x7F, 0xFF], np.uint8))).all()


def test_pack_unpack_e2m1():
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 16, size=(7, 64), dtype=np.uint8)
    packed = F.pack_e2m1(codes)
    assert packed.shape == (7, 32)
    assert packed[0, 0] == (codes[0, 0] | (codes[0, 1] << 4))     # even index in the low nibble
    assert np.array_equal(F.unpack_e2m1(packed), codes)


@pytest.mark.parametrize("vec,rows,K", [(16, 300, 448), (32, 130, 1024), (16, 128, 64)])
def test_sf_offset_matches_reference_layout(golden, vec, rows, K):
    want = golden[f"sf_offset_{vec}_{rows}_{K}"]
    kb = F.ceil_div(K, vec)
    got = F.sf_offset(np.arange(rows)[:, None], np.arange(kb)[None, :], F.sf_k_atoms(K, vec))
    assert np.array_equal(got, want)
    assert np.array_equal(R.sf_index(rows, kb), want)
    assert F.numel_scale(rows, K, vec) == int(golden[f"sf_size_{vec}_{rows}_{K}"][0])
    lib = oracle.load_oracle()
    assert all(lib.bsg_oracle_sf_offset(r, k, F.sf_k_atoms(K, vec)) == want[r, k] for r in range(0, rows, 13) for k in range(kb))


def test_swizzle_roundtrip_and_padding():
    rng = np.random.default_rng(1)
    sf = rng.integers(1, 255, size=(200, 7), dtype=np.uint8)
    buf = F.swizzle_sf(sf)
    assert buf.size == 256 * 8
    assert np.array_equal(F.unswizzle_sf(buf, 200, 7), sf)
    # offsets of distinct (row, kblock) never collide
    off = F.sf_offset(np.arange(256)[:, None], np.arange(8)[None, :], 2)
    assert len(np.unique(off)) == off.size and off.max() == buf.size - 1


def test_bf16_round_matches_oracle():
    rng = np.random.default_rng(2)
    x = np.concatenate([rng.standard_normal(5000).astype(np.float32) * 100, np.array([0.0, -0.0, 1.00390625, 1.01171875, 3.4e38], np.float32)])
    assert np.array_equal(F.bf16_round(x), oracle.to_bf16(x))
    assert np.array_equal(R.f32_to_bf16_bits(x), oracle.to_bf16(x))


def test_e5m2_codec_matches_reference(golden):
    """e5m2 is an output type of the GEMM: decode of every code, and the encode sweep (every midpoint between
    neighbouring values, their float32 neighbours, infinities, NaN, overflow) against the reference's float_e5m2_t."""
    assert _same_float(F.decode_e5m2(np.arange(256, dtype=np.uint8)), golden["decode_4"])
    x, want = golden["encode5_in"], golden["encode_4"]
    got = F.encode_e5m2(x)
    assert np.array_equal(got, want), [(float(x[i]), int(got[i]), int(want[i])) for i in np.nonzero(got != want)[0][:5]]
    codes = np.arange(0x7C, dtype=np.uint8)
    assert np.array_equal(F.encode_e5m2(F.decode_e5m2(codes)), codes)


def test_nan_of_either_sign_encodes_as_the_positive_nan_code():
    neg_nan = np.array([0xFFC00000, 0x7FC00000], dtype=np.uint32).view(np.float32)
    assert F.encode_e4m3(neg_nan).tolist() == [0x7F, 0x7F]
    assert F.encode_e5m2(neg_nan).tolist() == [0x7F, 0x7F]
