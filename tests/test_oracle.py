"""Pins the oracles (plain-C restatement and numpy restatement) to the reference:
against golden vectors produced by the reference's own host GEMM
(tests/golden/make_golden.py) and, where the compiled reference driver is present
(oracle/_ref), against it directly on fresh seeded inputs."""
import numpy as np
import pytest

import oracle
from cutlass_b200 import formats as F
from cutlass_b200 import generators as G
from oracle import ref_numpy as R

GEMM_CASES = ["nvfp4_a", "nvfp4_b", "mxfp8_a", "mxfp8_b", "mxfp4_a", "mixed_a"]


def _case(golden, name):
    kind, M, N, K = (int(v) for v in golden[f"{name}_dims"])
    return kind, M, N, K, golden[f"{name}_A"], golden[f"{name}_SFA"], golden[f"{name}_B"], golden[f"{name}_SFB"], golden[f"{name}_C"]


@pytest.mark.parametrize("name", GEMM_CASES)
def test_c_oracle_bit_exact_on_golden_gemm(golden, name):
    kind, M, N, K, A, sfa, B, sfb, Cb = _case(golden, name)
    alpha, beta = (float(v) for v in golden[f"{name}_ab"])
    got = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, alpha, beta)
    assert np.array_equal(got.view(np.uint32), golden[f"{name}_D32"].view(np.uint32))
    assert np.array_equal(oracle.to_bf16(got), golden[f"{name}_Dbf16"])


@pytest.mark.parametrize("name", GEMM_CASES)
def test_numpy_oracle_close_on_golden_gemm(golden, name):
    kind, M, N, K, A, sfa, B, sfb, Cb = _case(golden, name)
    alpha, beta = (float(v) for v in golden[f"{name}_ab"])
    got = R.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, alpha, beta)
    want = golden[f"{name}_D32"]
    assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want))


def test_row_slab_equals_full(golden):
    kind, M, N, K, A, sfa, B, sfb, Cb = _case(golden, "nvfp4_b")
    alpha, beta = (float(v) for v in golden["nvfp4_b_ab"])
    slab = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, alpha, beta, m_begin=64, m_count=50)
    assert np.array_equal(slab, golden["nvfp4_b_D32"][64:114])


@pytest.mark.parametrize("name", ["nvfp4_a", "mxfp8_a", "mxfp8_b"])
def test_bias_and_activation_epilogue_on_golden(golden, name):
    """act(alpha * acc + bias + beta * C) in the reference's order; ReLU bit for bit, GELU / SiLU up to the
    host math library's erf / exp (the golden values were produced on this image: normally bit for bit too)."""
    kind, M, N, K, A, sfa, B, sfb, Cb = _case(golden, name)
    alpha, beta = (float(v) for v in golden[f"{name}_ab"])
    for tag, per_row, act in (("relu_col", False, 1), ("gelu_col", False, 2), ("silu_row", True, 3)):
        bias = golden[f"{name}_bias_row" if per_row else f"{name}_bias_col"]
        got = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, alpha, beta, bias=bias, bias_per_row=per_row, activation=act)
        want = golden[f"{name}_D32_{tag}"]
        if act == 1:
            assert np.array_equal(got, want)
        else:
            assert np.allclose(got, want, rtol=2e-6, atol=1e-30)


def test_quantisation_bit_exact_on_golden(golden):
    kind, M, N, K, A, sfa, B, sfb, Cb = _case(golden, "quant_a")
    st = float(golden["quant_a_st"][0])
    d32 = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, 1.0, 0.5)
    assert np.array_equal(d32, golden["quant_a_D32"])
    idx = R.sf_index(M, N // 16)
    for D, SFD in (oracle.quant_nvfp4(d32, st), R.quantize_rows_nvfp4(d32, st)):
        assert np.array_equal(D, golden["quant_a_D"])
        assert np.array_equal(SFD[idx], golden["quant_a_SFD"][idx])


def test_mxfp8_quantisation_bit_exact_on_golden(golden):
    """e4m3 values + ue8m0 scale per 32 (round-up conversion), from the reference's own epilogue."""
    kind, M, N, K, A, sfa, B, sfb, Cb = _case(golden, "quant_a")
    d32 = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, 1.0, 0.5)
    idx = R.sf_index(M, N // 32)
    for tag in ("mx1", "mx2"):
        st = float(golden[f"quant_a_st_{tag}"][0])
        D, SFD = oracle.quant(1, d32, st)
        assert np.array_equal(D, golden[f"quant_a_D_{tag}"])
        assert np.array_equal(SFD[idx], golden[f"quant_a_SFD_{tag}"][idx])
    # kind 0 of the general entry point is the NVFP4 routine
    D0, S0 = oracle.quant(0, d32, float(golden["quant_a_st"][0]))
    assert np.array_equal(D0, golden["quant_a_D"])


def test_quantisation_edge_values():
    x = np.zeros((3, 32), np.float32)
    x[1, :16] = 1e-30          # underflows the scale factor to zero
    x[2, 5] = -6.0
    x[2, 20] = 448.0 * 6.0 * 4
    for D, SFD in (oracle.quant_nvfp4(x, 1.0), R.quantize_rows_nvfp4(x, 1.0)):
        sf = SFD[R.sf_index(3, 2)]
        assert sf[0].tolist() == [0, 0] and not D[0].any()
        # scale factor 0 -> reciprocal inf -> clamped to FLT_MAX: tiny values blow up and saturate at 6
        assert sf[1, 0] == 0 and (D[1, :8] == 0x77).all() and not D[1, 8:].any()
        assert sf[2, 0] == F.encode_ue4m3(np.float32(1.0)) and sf[2, 1] == 0x7E        # saturates at 448
        codes = F.unpack_e2m1(D[2])
        assert codes[5] == 15 and codes[20] == 7


ref_missing = oracle.load_ref() is None


@pytest.mark.skipif(ref_missing, reason="compiled reference driver (oracle/_ref) not present")
@pytest.mark.parametrize("kind,M,N,K,alpha,beta", [(0, 200, 264, 416, 1.5, 0.5), (1, 129, 72, 224, 1.0, 0.0), (0, 64, 64, 1024, 1.0, 0.5),
                                                   (2, 150, 200, 320, 1.25, 0.5), (3, 129, 136, 256, 1.0, -0.5)])
def test_c_oracle_equals_compiled_reference(kind, M, N, K, alpha, beta):
    rng = np.random.default_rng(M * 7 + N)
    gen_a, gen_b = G.operand_generators(kind, False)
    A, _, sfa = gen_a(M, K, rng)
    B, _, sfb = gen_b(N, K, rng)
    Cb = G.bf16_normal((M, N), rng)
    o = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, alpha, beta)
    r = oracle.ref_gemm(kind, 0, A, sfa, B, sfb, M, N, K, Cb, alpha, beta)
    assert np.array_equal(o.view(np.uint32), r.view(np.uint32))


@pytest.mark.skipif(ref_missing, reason="compiled reference driver (oracle/_ref) not present")
def test_quantisation_equals_compiled_reference():
    rng = np.random.default_rng(5)
    M, N, K = 130, 160, 256
    A, _, sfa = G.nvfp4_operand(M, K, rng)
    B, _, sfb = G.nvfp4_operand(N, K, rng)
    d32 = oracle.gemm_fp32(0, A, sfa, B, sfb, M, N, K)
    st = np.float32(448 * 6 / np.abs(d32).max())
    D, SFD = oracle.quant_nvfp4(d32, st)
    Dr, SFDr = oracle.ref_gemm(0, 2, A, sfa, B, sfb, M, N, K, None, 1.0, 0.0, st)
    idx = R.sf_index(M, N // 16)
    assert np.array_equal(D, Dr) and np.array_equal(SFD[idx], SFDr[idx])


@pytest.mark.skipif(ref_missing, reason="compiled reference driver (oracle/_ref) not present")
@pytest.mark.parametrize("st", [1.0, 0.37, 1e-3, 300.0])
def test_both_output_quantisations_on_wide_magnitudes_equal_compiled_reference(st):
    """K = 32 with one non-zero per row turns the GEMM into a table of chosen products, so the quantisation of the
    reference's epilogue sees magnitudes more than five decades apart, zero blocks included; both output types, bit for bit."""
    M, N, K = 128, 256, 32
    rng = np.random.default_rng(3)
    codesA = np.zeros((M, K), np.uint8)
    codesB = np.zeros((N, K), np.uint8)
    codesA[np.arange(M), np.arange(M) % K] = rng.integers(1, 8, M)
    codesB[np.arange(N), rng.integers(0, K, N)] = rng.integers(1, 16, N)
    codesB[codesB == 8] = 1
    A, B = F.pack_e2m1(codesA), F.pack_e2m1(codesB)
    sfa = F.swizzle_sf(rng.integers(0x20, 0x60, (M, 2)).astype(np.uint8))
    sfb = F.swizzle_sf(rng.integers(0x20, 0x60, (N, 2)).astype(np.uint8))
    pre = oracle.gemm_fp32(0, A, sfa, B, sfb, M, N, K)
    assert (pre == 0).any() and np.abs(pre).max() / np.abs(pre[pre != 0]).min() > 1e5
    for mode, qkind, vec in ((2, 0, 16), (3, 1, 32)):
        Dr, Sr = oracle.ref_gemm(0, mode, A, sfa, B, sfb, M, N, K, None, 1.0, 0.0, st)
        Do, So = oracle.quant(qkind, pre, st)
        idx = R.sf_index(M, N // vec)
        assert np.array_equal(Do, Dr), (mode, st)
        assert np.array_equal(So[idx], Sr[idx]), (mode, st)


@pytest.mark.skipif(ref_missing, reason="compiled reference driver (oracle/_ref) not present")
@pytest.mark.skipif(ref_missing, reason="compiled reference driver (oracle/_ref) not present")
@pytest.mark.parametrize("M,N,K", [(160, 200, 128), (128, 64, 64), (96, 333 // 3 * 3 + 1, 192)])
def test_column_major_quantised_output_is_the_row_major_routine_on_the_transpose(M, N, K):
    """The reference's M-major scale-factor output (D column-major, one scale factor per 16 / 32 consecutive rows of a
    column; gett.hpp:392-430 with Sm1xxBlockScaledOutputConfig<V, Major::MN>) equals the row-major routine applied to
    the transposed matrix, values and scale-factor bytes alike: that is the oracle of the kernels' column-major output."""
    rng = np.random.default_rng(M + N)
    A, _, sfa = G.nvfp4_operand(M, K, rng)
    B, _, sfb = G.nvfp4_operand(N, K, rng)
    Cb = G.bf16_normal((M, N), rng)
    pre = oracle.gemm_fp32(0, A, sfa, B, sfb, M, N, K, Cb, 1.0, 0.5)
    for mode, qkind, vec in ((4, 0, 16), (5, 1, 32)):
        Dr, Sr = oracle.ref_gemm(0, mode, A, sfa, B, sfb, M, N, K, Cb, 1.0, 0.5, 3.0)
        Do, So = oracle.quant(qkind, np.ascontiguousarray(pre.T), 3.0)
        idx = R.sf_index(N, M // vec)
        assert np.array_equal(Dr, Do) and np.array_equal(Sr[idx], So[idx])


@pytest.mark.skipif(ref_missing, reason="compiled reference driver (oracle/_ref) not present")
def test_nan_and_infinity_in_a_block_equal_compiled_reference():
    """The reference's block maximum and its clamp of the scale propagate NaN (maximum_with_nan_propogation,
    minimum_with_nan_propagation): one NaN makes the block's scale factor a NaN code and every value of the block the
    format's NaN code (e4m3) or its largest value (e2m1 has no NaN).  An infinite accumulator saturates the ue4m3
    scale factor; ue8m0 has no infinity and turns it into its NaN code."""
    rng = np.random.default_rng(1)
    M, N, K = 128, 64, 64
    A, _, sfa = G.nvfp4_operand(M, K, rng)
    B, _, sfb = G.nvfp4_operand(N, K, rng)
    Cb = G.bf16_normal((M, N), rng)
    Cb[3, 5], Cb[7, 40], Cb[9, 17], Cb[11, 3] = 0x7FC0, 0xFFC0, 0x7F80, 0xFF80        # NaN, -NaN, +inf, -inf
    pre = oracle.gemm_fp32(0, A, sfa, B, sfb, M, N, K, Cb, 1.0, 1.0)
    for mode, qkind, vec in ((2, 0, 16), (3, 1, 32)):
        Dr, Sr = oracle.ref_gemm(0, mode, A, sfa, B, sfb, M, N, K, Cb, 1.0, 1.0, 2.0)
        Do, So = oracle.quant(qkind, pre, 2.0)
        idx = R.sf_index(M, N // vec)
        assert np.array_equal(Do, Dr) and np.array_equal(So[idx], Sr[idx])
        # what those blocks look like
        nan_sf = 0x7F if qkind == 0 else 0xFF
        assert Sr[idx][3, 0] == nan_sf and Sr[idx][7, 40 // vec] == nan_sf
        if qkind == 0:
            assert np.all(Dr[3, :8] == 0x77) and Sr[idx][9, 1] == 0x7E
        else:
            assert np.all(Dr[3, :32] == 0x7F) and Sr[idx][9, 0] == 0xFF and np.all(Dr[9, :32] == 0x7F)


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("act,per_row", [(0, False), (1, True), (2, False), (3, True)])
def test_epilogue_with_bias_and_activation_equals_compiled_reference(kind, act, per_row):
    rng = np.random.default_rng(17 + act)
    gen = G.nvfp4_operand if kind == 0 else G.mxfp8_operand
    M, N, K = 70, 136, 192
    A, _, sfa = gen(M, K, rng)
    B, _, sfb = gen(N, K, rng)
    Cb = G.bf16_normal((M, N), rng)
    bias = (rng.standard_normal(M if per_row else N) * 3).astype(np.float32)
    r = oracle.ref_gemm_epi(kind, A, sfa, B, sfb, M, N, K, Cb, 0.75, 0.5, bias, per_row, act)
    o = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, 0.75, 0.5, bias=bias, bias_per_row=per_row, activation=act)
    assert np.array_equal(o.view(np.uint32), r.view(np.uint32))


@pytest.mark.skipif(ref_missing, reason="compiled reference driver (oracle/_ref) not present")
def test_codecs_exhaustive_against_compiled_reference():
    ref = oracle.load_ref()
    lib = oracle.load_oracle()
    rng = np.random.default_rng(9)
    xs = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in (1e-3, 1, 50, 1000)])
    for fmt in range(4):
        for c in range(16 if fmt == 0 else 256):
            a, b = ref.bsg_ref_decode(fmt, c), lib.bsg_oracle_decode(fmt, c)
            assert a == b or (np.isnan(a) and np.isnan(b)), (fmt, c)
        assert all(ref.bsg_ref_encode(fmt, float(x)) == lib.bsg_oracle_encode(fmt, float(x)) for x in xs), fmt
