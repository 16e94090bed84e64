"""-m gpu parity tests: the CUDA path, called through the C ABI, against the CPU oracle on the
same seeded inputs.  Exact-arithmetic fixtures ({-1,0,1} data, power-of-two scales) must match
bit for bit; realistic distributions must match within the stated tolerance (bf16 outputs:
relative 1e-2 against the fp32-accumulated oracle)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from cutlass_b200 import formats as F
from cutlass_b200 import generators as G
from cutlass_b200 import lib as L
from oracle import ref_numpy as R

from gpu_utils import assert_close_bf16, dev, make_operands, oracle_bf16, run_dense, run_grouped

pytestmark = pytest.mark.gpu

TILES = [(2, 256), (2, 128), (1, 256), (1, 128)]


@pytest.mark.parametrize("cta_group,tile_n", TILES)
@pytest.mark.parametrize("kind,M,N,K", [(0, 256, 512, 512), (1, 256, 512, 384), (0, 128, 128, 64), (1, 128, 128, 32)])
def test_exact_fixtures_bit_exact_all_tiles(cuda_lib, kind, M, N, K, cta_group, tile_n):
    _, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=M + N + K + tile_n, exact=True)
    got = run_dense(kind, M, N, K, A, sfa, B, sfb, tile_n=tile_n, cta_group=cta_group)
    assert np.array_equal(got, oracle_bf16(kind, M, N, K, A, sfa, B, sfb))


@pytest.mark.parametrize("kind", [0, 1])
def test_config0_shape_1024_cubed_with_c(cuda_lib, kind):
    """BASELINE config 0: M=N=K=1024, alpha=1, beta=0.5, C ~ N(0,1) bf16, realistic operand values."""
    M = N = K = 1024
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=0, exact=False)
    Cb = G.bf16_normal((M, N), rng)
    got = run_dense(kind, M, N, K, A, sfa, B, sfb, Cb, 1.0, 0.5)
    assert_close_bf16(got, oracle_bf16(kind, M, N, K, A, sfa, B, sfb, Cb, 1.0, 0.5))


@pytest.mark.parametrize("kind,M,N,K", [
    (0, 200, 200, 320),      # ragged M and N, K not a multiple of the k-tile
    (0, 1, 8, 32),           # smallest legal problem
    (1, 130, 264, 80),       # K tail of MXFP8 (80 = 2.5 MMA blocks -> 3 blocks, 16-byte aligned rows)
    (0, 384, 2056, 96),      # N tail of 8 columns, K = 1.5 MMA blocks
    (1, 513, 136, 4096),     # deep K, one row past a tile boundary
    (0, 4096, 4096, 2048),   # many tiles per CTA (persistent loop, accumulator double buffering)
])
def test_edge_shapes(cuda_lib, kind, M, N, K):
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=K, exact=True)
    Cb = G.bf16_normal((M, N), rng)
    got = run_dense(kind, M, N, K, A, sfa, B, sfb, Cb, 2.0, 1.0)
    assert_close_bf16(got, oracle_bf16(kind, M, N, K, A, sfa, B, sfb, Cb, 2.0, 1.0), rel_tol=4e-3)


def test_alpha_beta_from_device_pointers(cuda_lib):
    M, N, K = 256, 256, 256
    rng, A, sfa, B, sfb = make_operands(0, M, N, K, seed=5, exact=True)
    Cb = G.bf16_normal((M, N), rng)
    lib = L.load()
    t = [dev(x) for x in (A, B, sfa, sfb, Cb)]
    ab = torch.tensor([0.5, -2.0], dtype=torch.float32, device="cuda")
    D = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    a = L.GemmArgs()
    a.kind, a.batch, a.M, a.N, a.K = 0, 1, M, N, K
    a.A, a.B, a.SFA, a.SFB, a.C, a.D = (x.data_ptr() for x in (t[0], t[1], t[2], t[3], t[4], D))
    a.alpha, a.beta = 99.0, 99.0                       # overridden by the device scalars
    a.alpha_ptr, a.beta_ptr = ab.data_ptr(), ab.data_ptr() + 4
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), 16, None))
    L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
    assert np.array_equal(D.cpu().numpy().view(np.uint16), oracle_bf16(0, M, N, K, A, sfa, B, sfb, Cb, 0.5, -2.0))


@pytest.mark.parametrize("kind,M,N,K,sms", [(0, 768, 768, 512, 8), (1, 768, 768, 256, 8), (0, 1280, 640, 256, 12), (1, 512, 1280, 384, 6),
                                             (0, 2560, 2048, 256, 0)])
def test_last_wave_tiles_split_in_halves(cuda_lib, kind, M, N, K, sms):
    """Tile counts that leave a last wave at most half full (9 tiles on 4 clusters, 15 on 6, 10 on 3 with a partial
    tile column, 80 on the whole GPU): those tiles are computed as two column halves by different clusters, and the
    result must not change.  beta * C and the quantised output take the same path."""
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=40 + sms, exact=True)
    Cb = G.bf16_normal((M, N), rng)
    got = run_dense(kind, M, N, K, A, sfa, B, sfb, Cb, 1.0, 0.5, sm_count=sms)
    assert np.array_equal(got, oracle_bf16(kind, M, N, K, A, sfa, B, sfb, Cb, 1.0, 0.5))
    if kind == 0 and N % 32 == 0:
        pre = oracle.gemm_fp32(0, A, sfa, B, sfb, M, N, K)
        st = np.float32(448.0 * 6.0 / np.abs(pre).max())
        D, SFD = run_dense(0, M, N, K, A, sfa, B, sfb, out_kind=1, st=float(st), sm_count=sms)
        Dw, SFDw = oracle.quant_nvfp4(pre, st)
        idx = R.sf_index(M, N // 16)
        assert np.array_equal(D, Dw) and np.array_equal(SFD[idx], SFDw[idx])


@pytest.mark.parametrize("kind", [0, 1])
def test_batched(cuda_lib, kind):
    Lb, M, N, K = 3, 192, 256, 256
    outs, As, sfas, Bs, sfbs = [], [], [], [], []
    for l in range(Lb):
        _, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=100 + l, exact=True)
        As.append(A); sfas.append(sfa); Bs.append(B); sfbs.append(sfb)
        outs.append(oracle_bf16(kind, M, N, K, A, sfa, B, sfb))
    got = run_dense(kind, M, N, K, np.concatenate(As), np.concatenate(sfas), np.concatenate(Bs), np.concatenate(sfbs), batch=Lb)
    assert np.array_equal(got, np.concatenate(outs))


@pytest.mark.parametrize("exact,beta", [(True, 0.0), (False, 0.5)])
def test_fused_nvfp4_output_bit_exact(cuda_lib, exact, beta):
    """e2m1 data and ue4m3 scale factors of the fused re-quantisation are bit-exact against the
    oracle (NVFP4 products with power-of-two scales accumulate exactly in fp32)."""
    M, N, K = 512, 1024, 512
    rng, A, sfa, B, sfb = make_operands(0, M, N, K, seed=11, exact=exact)
    Cb = G.bf16_normal((M, N), rng) if beta else None
    pre = oracle.gemm_fp32(0, A, sfa, B, sfb, M, N, K, Cb, 1.0, beta)
    st = np.float32(448.0 * 6.0 / np.abs(pre).max())
    D, SFD = run_dense(0, M, N, K, A, sfa, B, sfb, Cb, 1.0, beta, out_kind=1, st=float(st))
    Dw, SFDw = oracle.quant_nvfp4(pre, st)
    idx = R.sf_index(M, N // 16)
    assert np.array_equal(D, Dw)
    assert np.array_equal(SFD[idx], SFDw[idx])


@pytest.mark.parametrize("out_kind", [1, 2])
def test_fused_quantisation_with_nan_and_infinity_matches_the_oracle(cuda_lib, out_kind):
    """NaN / infinity reaching the fused output quantisation (through C): the same bytes as the oracle, whose handling of
    such blocks is pinned against the compiled reference (NaN poisons its block; ue8m0 turns infinity into NaN)."""
    M, N, K = 256, 512, 256
    rng, A, sfa, B, sfb = make_operands(0, M, N, K, seed=13, exact=True)
    Cb = G.bf16_normal((M, N), rng)
    Cb[3, 5], Cb[7, 300], Cb[9, 17], Cb[200, 511], Cb[130, 64] = 0x7FC0, 0xFFC0, 0x7F80, 0xFF80, 0x7FC0
    pre = oracle.gemm_fp32(0, A, sfa, B, sfb, M, N, K, Cb, 1.0, 1.0)
    D, SFD = run_dense(0, M, N, K, A, sfa, B, sfb, Cb, 1.0, 1.0, out_kind=out_kind, st=2.0)
    Dw, SFDw = oracle.quant(0 if out_kind == 1 else 1, pre, 2.0)
    idx = R.sf_index(M, N // (16 if out_kind == 1 else 32))
    assert np.array_equal(D, Dw)
    assert np.array_equal(SFD[idx], SFDw[idx])


@pytest.mark.parametrize("kind,exact,beta,st", [(0, True, 0.0, None), (0, False, 0.5, 3.0), (1, True, 0.0, 0.25), (1, False, 0.5, None)])
def test_fused_mxfp8_output_bit_exact(cuda_lib, kind, exact, beta, st):
    """e4m3 data and ue8m0 scale factors (round-up conversion) of the fused MXFP8 re-quantisation against the oracle.
    With exact-arithmetic operands the accumulators are exact and every byte must agree; with realistic MXFP8
    operands the fp32 accumulation order differs, so a value that sits on a rounding boundary may move one code."""
    M, N, K = 384, 768, 512
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=21, exact=exact)
    Cb = G.bf16_normal((M, N), rng) if beta else None
    pre = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, 1.0, beta)
    D, SFD = run_dense(kind, M, N, K, A, sfa, B, sfb, Cb, 1.0, beta, out_kind=2, st=st)
    Dw, SFDw = oracle.quant(1, pre, 1.0 if st is None else st)
    idx = R.sf_index(M, N // 32)
    if exact or kind == 0:
        assert np.array_equal(SFD[idx], SFDw[idx])
        assert np.array_equal(D, Dw)
    else:
        assert (SFD[idx] != SFDw[idx]).mean() < 1e-3
        assert (D != Dw).mean() < 2e-2


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("act,per_row,beta", [(1, False, 0.0), (1, True, 0.5), (2, False, 0.5), (3, False, 0.0), (3, True, 0.5), (0, False, 0.5)])
def test_bias_and_activation_epilogue(cuda_lib, kind, act, per_row, beta):
    """act(alpha * acc + bias + beta * C): exact-arithmetic operands, so identity and ReLU must agree bit for bit
    with the oracle; GELU / SiLU go through erf / exp of two different math libraries (rel 1e-2 on bf16)."""
    M, N, K = 300, 456, 384          # ragged M, N not a multiple of the tile
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=31 + act, exact=True)
    Cb = G.bf16_normal((M, N), rng) if beta else None
    bias = (rng.standard_normal(M if per_row else N) * 4).astype(np.float32)
    got = run_dense(kind, M, N, K, A, sfa, B, sfb, Cb, 0.5, beta, bias=bias, bias_per_row=per_row, activation=act)
    want = oracle_bf16(kind, M, N, K, A, sfa, B, sfb, Cb, 0.5, beta, bias=bias, bias_per_row=per_row, activation=act)
    if act in (0, 1):
        assert np.array_equal(got, want)
    else:
        assert_close_bf16(got, want)
        assert (got != want).mean() < 0.05          # at most a bf16 ulp here and there


@pytest.mark.parametrize("kind", [0, 1])
def test_grouped_bias_per_group_and_activation(cuda_lib, kind):
    got, want = run_grouped(kind, [200, 0, 129, 384], 256, 256, seed=5, exact=True, alpha=1.0, beta=0.5, with_bias=True, activation=1)
    assert np.array_equal(got, want)
    got, want = run_grouped(kind, [64, 300], 384, 512, seed=6, exact=True, with_bias=True, activation=3)
    assert_close_bf16(got, want)


@pytest.mark.parametrize("kind", [0, 1])
def test_grouped_per_group_alpha_beta(cuda_lib, kind):
    """One alpha and one beta per expert (device arrays), beta = 0 for some groups."""
    got, want = run_grouped(kind, [130, 256, 0, 77, 512, 1], 256, 384, seed=8, exact=True, per_group_scalars=True)
    assert np.array_equal(got, want)


def test_activation_before_fused_quantisation(cuda_lib):
    """ReLU then NVFP4 / MXFP8 re-quantisation of the output: the quantiser sees the activated values."""
    M, N, K = 256, 512, 256
    rng, A, sfa, B, sfb = make_operands(0, M, N, K, seed=41, exact=True)
    bias = (rng.standard_normal(N) * 8).astype(np.float32)
    pre = oracle.gemm_fp32(0, A, sfa, B, sfb, M, N, K, bias=bias, activation=1)
    st = np.float32(448.0 * 6.0 / np.abs(pre).max())
    D, SFD = run_dense(0, M, N, K, A, sfa, B, sfb, out_kind=1, st=float(st), bias=bias, activation=1)
    Dw, SFDw = oracle.quant(0, pre, st)
    idx = R.sf_index(M, N // 16)
    assert np.array_equal(D, Dw) and np.array_equal(SFD[idx], SFDw[idx])
    D, SFD = run_dense(0, M, N, K, A, sfa, B, sfb, out_kind=2, bias=bias, activation=1)
    Dw, SFDw = oracle.quant(1, pre, 1.0)
    idx = R.sf_index(M, N // 32)
    assert np.array_equal(D, Dw) and np.array_equal(SFD[idx], SFDw[idx])


def test_quantisation_stage_in_isolation(cuda_lib):
    """K = 32 with identity-like operands turns the GEMM into a copy of chosen fp32 values, so the
    kernel's quantisation arithmetic is compared with the oracle on arbitrary magnitudes."""
    M, N, K = 128, 256, 32
    rng = np.random.default_rng(3)
    # A row m = one non-zero (value from the e2m1 grid) at k = m % 32, B row n likewise -> sparse exact products
    codesA = np.zeros((M, K), np.uint8); codesB = np.zeros((N, K), np.uint8)
    codesA[np.arange(M), np.arange(M) % K] = rng.integers(1, 8, M)
    codesB[np.arange(N), rng.integers(0, K, N)] = rng.integers(1, 16, N)
    codesB[codesB == 8] = 1
    A, B = F.pack_e2m1(codesA), F.pack_e2m1(codesB)
    sfa_codes = rng.integers(0x20, 0x60, (M, 2)).astype(np.uint8)
    sfb_codes = rng.integers(0x20, 0x60, (N, 2)).astype(np.uint8)
    sfa, sfb = F.swizzle_sf(sfa_codes), F.swizzle_sf(sfb_codes)
    pre = oracle.gemm_fp32(0, A, sfa, B, sfb, M, N, K)
    for st in (1.0, 0.37, 1e-3, 300.0):
        D, SFD = run_dense(0, M, N, K, A, sfa, B, sfb, out_kind=1, st=st)
        Dw, SFDw = oracle.quant_nvfp4(pre, st)
        idx = R.sf_index(M, N // 16)
        assert np.array_equal(SFD[idx], SFDw[idx]), st
        assert np.array_equal(D, Dw), st


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("sizes", [[256, 256], [100, 0, 300, 1, 515], [64] * 9, [700]])
def test_grouped_ragged(cuda_lib, kind, sizes):
    got, want = run_grouped(kind, np.array(sizes), N=384, K=512, seed=len(sizes), exact=True, alpha=1.0, beta=0.5)
    assert_close_bf16(got, want, rel_tol=4e-3)


def test_grouped_exact_and_canary_rows(cuda_lib):
    """Rows of neighbouring groups must not be touched by a partial tile at a group's end."""
    sizes = np.array([130, 5, 250, 127])
    got, want = run_grouped(0, sizes, N=256, K=256, seed=42, exact=True)
    assert np.array_equal(got, want)


def test_grouped_moe_distribution(cuda_lib):
    rng = np.random.default_rng(0)
    sizes = G.moe_group_sizes(16, 512, 8, rng)                   # 4096 rows over 16 experts, Dirichlet(1) skew
    got, want = run_grouped(0, sizes, N=512, K=1024, seed=1, exact=False)
    assert_close_bf16(got, want)


def test_grouped_rejects_bad_offsets(cuda_lib):
    lib = L.load()
    N, K = 256, 256
    A = torch.zeros((512, K // 2), dtype=torch.uint8, device="cuda")
    B = torch.zeros((2, N, K // 2), dtype=torch.uint8, device="cuda")
    sf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    D = torch.zeros((512, N), dtype=torch.int16, device="cuda")
    offs = torch.tensor([300, 200], dtype=torch.int32, device="cuda")       # not monotone
    a = L.GroupedArgs()
    a.kind, a.num_groups, a.total_M, a.N, a.K = 0, 2, 512, N, K
    a.A, a.B, a.SFA, a.SFB, a.D, a.offsets = (x.data_ptr() for x in (A, B, sf, sf, D, offs))
    a.alpha = 1.0
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    assert lib.bsg_grouped_run(C.byref(a), ws.data_ptr(), 16, None) == 0
    assert lib.bsg_read_device_status(ws.data_ptr(), None) == 2           # BSG_ERR_INVALID_PROBLEM, no fault
    assert lib.bsg_read_device_status(ws.data_ptr(), None) == 0           # reading clears the status


def test_linearity_and_scale_properties_at_full_size(cuda_lib):
    """Size-independent properties at the headline shape (8192^3): doubling every A scale factor
    (a power of two) doubles D exactly; a slab of rows matches the oracle."""
    M = N = K = 8192
    import bench
    gen = torch.Generator(device="cuda"); gen.manual_seed(0)
    A, SFA = bench.gpu_nvfp4_operand(M, K, gen, "cuda")
    B, SFB = bench.gpu_nvfp4_operand(N, K, gen, "cuda")
    lib = L.load()

    def run(sfa):
        D = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        a = L.GemmArgs()
        a.kind, a.batch, a.M, a.N, a.K = 0, 1, M, N, K
        a.A, a.B, a.SFA, a.SFB, a.D = A.data_ptr(), B.data_ptr(), sfa.data_ptr(), SFB.data_ptr(), D.data_ptr()
        a.alpha = 1.0
        ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
        L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), 16, None))
        L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
        return D

    D1 = run(SFA)
    D2 = run(SFA + 8)                                  # ue4m3 exponent + 1 = scale x 2
    assert torch.equal(D2.float(), D1.float() * 2)
    rows = 128
    want = oracle_bf16(0, rows, N, K, A[:rows].cpu().numpy(), SFA[: rows * (K // 16)].cpu().numpy(), B.cpu().numpy(), SFB.cpu().numpy())
    assert_close_bf16(D1[:rows].view(torch.int16).cpu().numpy().view(np.uint16), want)


def test_operator_api_end_to_end(cuda_lib):
    import cutlass_b200 as ops
    M, N, K = 256, 384, 512
    rng, A, sfa, B, sfb = make_operands(1, M, N, K, seed=8, exact=False)
    Cb = G.bf16_normal((M, N), rng)
    SW, mode = ops.ScaleSwizzleMode.Swizzle32x4x4, ops.ScaleMode.Blockwise1x32
    out = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    args = ops.GemmArguments(ops.ScaledOperand(dev(A).view(torch.float8_e4m3fn), dev(sfa), mode, SW),
                             ops.ScaledOperand(dev(B).view(torch.float8_e4m3fn).t(), dev(sfb), mode, SW), out, torch.float32,
                             epilogue=ops.EpilogueDescriptor(alpha=1.0, beta=0.5, C=dev(Cb).view(torch.bfloat16)))
    for op in ops.get_operators(args):
        out.zero_()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            op.run(args, stream=s)
        op.check_device_status(stream=s)
        assert_close_bf16(out.view(torch.int16).cpu().numpy().view(np.uint16), oracle_bf16(1, M, N, K, A, sfa, B, sfb, Cb, 1.0, 0.5))


def test_no_cpu_fallback_symbol_origin(cuda_lib):
    """The tested path is the native library: it is loaded from the package's lib/ directory."""
    assert L.LIB_PATH.endswith("cutlass_b200/lib/libbsgemm.so")
    assert cuda_lib.bsg_version() >= 100
