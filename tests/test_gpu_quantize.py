"""The block-scaled quantiser (bsg_quantize) against the CPU oracle: values and scale factors bit-exact."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from cutlass_b200 import formats as F
from cutlass_b200 import lib as L

pytestmark = pytest.mark.gpu


def _bf16_input(rows, K, seed):
    """bf16 matrix with blocks of very different magnitude, an all-zero block, tiny and huge values."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, K)).astype(np.float32)
    x *= np.exp2(rng.integers(-6, 7, size=(rows, K // 16))).repeat(16, axis=1).astype(np.float32)
    x[0, :32] = 0.0
    if rows > 2:
        x[1, 5] = 1.0e30
        x[2, :16] = 1e-30
        x[2, 40 % K] = -1e-38
    t = torch.from_numpy(x).to(torch.bfloat16)
    return t, t.to(torch.float32).numpy()


def _run(kind, xt, st=None, ldx=None):
    lib = L.load()
    rows, K = xt.shape
    if ldx is not None:
        buf = torch.zeros((rows, ldx), dtype=torch.bfloat16, device="cuda")
        buf[:, :K] = xt.cuda()
        dx = buf
    else:
        dx = xt.cuda().contiguous()
    vec = 16 if kind == 0 else 32
    q = torch.full((rows, K // 2 if kind == 0 else K), 0xEE, dtype=torch.uint8, device="cuda")
    sf = torch.full((F.numel_scale(rows, K, vec),), 0xEE, dtype=torch.uint8, device="cuda")
    a = L.QuantArgs()
    a.kind, a.rows, a.K, a.X, a.ldx, a.Q, a.SF = kind, rows, K, dx.data_ptr(), dx.stride(0), q.data_ptr(), sf.data_ptr()
    keep = None
    if st is not None:
        keep = torch.tensor([st], dtype=torch.float32, device="cuda")
        a.norm_constant = keep.data_ptr()
    L.check(lib.bsg_quantize(C.byref(a), None))
    torch.cuda.synchronize()
    return q.cpu().numpy(), sf.cpu().numpy()


def _valid_sf_index(rows, kblocks):
    k_atoms = F.ceil_div(kblocks, 4)
    r, kb = np.meshgrid(np.arange(rows), np.arange(kblocks), indexing="ij")
    return F.sf_offset(r, kb, k_atoms).ravel()


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("rows,K", [(128, 256), (70, 96), (300, 448), (1, 32), (257, 1056), (512, 4096)])
@pytest.mark.parametrize("st", [None, 37.5])
def test_quantiser_matches_oracle_bit_for_bit(kind, rows, K, st):
    xt, xf = _bf16_input(rows, K, seed=rows * 7 + K)
    q, sf = _run(kind, xt, st)
    want_q, want_sf = oracle.quant(kind, xf, 1.0 if st is None else st)
    assert np.array_equal(q, want_q), f"{int((q != want_q).sum())} quantised bytes differ"
    idx = _valid_sf_index(rows, K // (16 if kind == 0 else 32))
    assert np.array_equal(sf[idx], want_sf[idx])
    pad = np.ones(sf.size, dtype=bool)
    pad[idx] = False
    assert not sf[pad].any(), "scale factors of rows / K-blocks that do not exist must be zero"


@pytest.mark.parametrize("kind", [0, 1])
def test_quantiser_honours_row_pitch(kind):
    xt, xf = _bf16_input(96, 128, seed=3)
    q, sf = _run(kind, xt, 2.0, ldx=200)
    want_q, want_sf = oracle.quant(kind, xf, 2.0)
    assert np.array_equal(q, want_q)
    idx = _valid_sf_index(96, 128 // (16 if kind == 0 else 32))
    assert np.array_equal(sf[idx], want_sf[idx])


@pytest.mark.parametrize("kind", [0, 1])
def test_quantised_operands_feed_the_gemm(kind):
    """quantise -> GEMM through the operator API: equals the oracle's GEMM on the quantised operands,
    and approximates the bf16 product (scaled back by the two norm constants)."""
    import cutlass_b200 as ops
    from cutlass_b200.quantize import quantize_blockscaled
    import gpu_utils as U
    M, N, K = 256, 384, 512
    rng = np.random.default_rng(11)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16).cuda()
    w = torch.from_numpy(rng.standard_normal((N, K)).astype(np.float32)).to(torch.bfloat16).cuda()
    mode = ops.ScaleMode.Blockwise1x16 if kind == 0 else ops.ScaleMode.Blockwise1x32
    if kind == 0:
        stx = (448.0 * 6.0 / x.float().abs().max()).reshape(1).float()
        stw = (448.0 * 6.0 / w.float().abs().max()).reshape(1).float()
    else:
        stx = stw = None
    A = quantize_blockscaled(x, mode, norm_constant=stx)
    Bq = quantize_blockscaled(w, mode, norm_constant=stw)
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    Bop = ops.ScaledOperand(Bq.quantized.tensor.t(), Bq.scale.tensor, mode, ops.ScaleSwizzleMode.Swizzle32x4x4)
    alpha = 1.0 if kind == 1 else float(1.0 / (stx.item() * stw.item()))
    args = ops.GemmArguments(A, Bop, out, torch.float32, epilogue=ops.EpilogueDescriptor(alpha=alpha))
    op = ops.get_operators(args)[0]
    op.run(args)
    torch.cuda.synchronize()
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    want = U.oracle_bf16(kind, M, N, K, A.quantized.tensor.cpu().numpy(), A.scale.tensor.cpu().numpy(),
                         Bq.quantized.tensor.cpu().numpy(), Bq.scale.tensor.cpu().numpy(), alpha=alpha)
    U.assert_close_bf16(got, want)
    exact = (x.float() @ w.float().t()).cpu().numpy()
    err = np.abs(F.bf16_to_f32(got) - exact)
    assert float(err.max()) <= (0.3 if kind == 0 else 0.15) * float(np.abs(exact).max())


@pytest.mark.parametrize("kind", [0, 1])
def test_quantiser_full_size_matches_oracle(kind):
    """8192 x 8192 (the benchmark's operand): every byte against the C oracle."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    x = torch.randn((8192, 8192), device="cuda", generator=gen).to(torch.bfloat16)
    q, sf = _run(kind, x.cpu(), 3.0 if kind == 0 else None)
    want_q, want_sf = oracle.quant(kind, x.float().cpu().numpy(), 3.0 if kind == 0 else 1.0)
    assert np.array_equal(q, want_q)
    assert np.array_equal(sf, want_sf)          # no padding at this size: the whole buffer is defined


@pytest.mark.parametrize("kind", [0, 1])
def test_nan_and_infinity_inputs_match_the_oracle(cuda_lib, kind):
    """NaN and infinite inputs: the block maximum propagates NaN as the reference's does, so the kernel's bytes equal
    the oracle's (itself pinned against the compiled reference on such inputs)."""
    import cutlass_b200 as ops
    rng = np.random.default_rng(5)
    rows, K = 256, 512
    x = rng.standard_normal((rows, K)).astype(np.float32)
    x[3, 5], x[7, 300], x[9, 17], x[200, 511], x[130, 64] = np.nan, -np.nan, np.inf, -np.inf, np.nan
    xb = torch.from_numpy(x).to(torch.bfloat16).cuda()
    mode = ops.ScaleMode.Blockwise1x16 if kind == 0 else ops.ScaleMode.Blockwise1x32
    q = ops.quantize_blockscaled(xb, mode)
    torch.cuda.synchronize()
    want_q, want_sf = oracle.quant(kind, xb.float().cpu().numpy(), 1.0)
    vec = 16 if kind == 0 else 32
    r, kb = np.meshgrid(np.arange(rows), np.arange(K // vec), indexing="ij")
    idx = F.sf_offset(r, kb, F.sf_k_atoms(K, vec)).ravel()
    assert np.array_equal(q.quantized.tensor.cpu().numpy().view(np.uint8), want_q)
    assert np.array_equal(q.scale.tensor.cpu().numpy().view(np.uint8)[idx], want_sf[idx])


def test_quantise_gemm_chain_with_programmatic_dependent_launch(cuda_lib):
    """quantise(x) -> GEMM -> quantise(result) launched back to back with use_pdl on every kernel: each kernel's set-up
    overlaps its predecessor's tail, its first global read waits for the predecessor.  Results equal the plain launches'."""
    import cutlass_b200 as ops
    from cutlass_b200.quantize import quantize_blockscaled
    M, N, K = 512, 768, 1024
    rng = np.random.default_rng(19)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16).cuda()
    w = torch.from_numpy(rng.standard_normal((N, K)).astype(np.float32)).to(torch.bfloat16).cuda()
    mode = ops.ScaleMode.Blockwise1x32
    Bq = quantize_blockscaled(w, mode)
    Bop = ops.ScaledOperand(Bq.quantized.tensor.t(), Bq.scale.tensor, mode, ops.ScaleSwizzleMode.Swizzle32x4x4)
    results = []
    for pdl in (False, True):
        out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        for _ in range(3):                                   # repeated so that every kernel has a dependent predecessor
            A = quantize_blockscaled(x, mode, use_pdl=pdl)
            args = ops.GemmArguments(A, Bop, out, torch.float32)
            op = ops.get_operators(args)[0]
            abi = op.build_args(args)
            abi.use_pdl = int(pdl)
            ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
            L.check(L.load().bsg_gemm_run(C.byref(abi), ws.data_ptr(), 16, None))
            Y = quantize_blockscaled(out, mode, use_pdl=pdl)
        torch.cuda.synchronize()
        L.check(L.load().bsg_read_device_status(ws.data_ptr(), None))
        results.append((out.clone(), Y.quantized.tensor.clone(), Y.scale.tensor.clone()))
    for a, b in zip(*results):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
