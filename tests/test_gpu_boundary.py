"""-m gpu tests of the argument surface that mirrors cutlass::library::BlockScaledGemmArguments beyond the plain
dense call: row pitches and batch strides, programmatic dependent launch, cluster-shape fields, and quantised
output of the grouped GEMM.  Everything goes through the C ABI and is compared bit for bit with the oracle
(exact-arithmetic operands)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from cutlass_b200 import formats as F
from cutlass_b200 import generators as G
from cutlass_b200 import lib as L
from oracle import ref_numpy as R

from gpu_utils import dev, make_operands, oracle_bf16, run_dense, run_grouped

pytestmark = pytest.mark.gpu


def _run(a):
    lib = L.load()
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), 16, None))
    L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
    torch.cuda.synchronize()


@pytest.mark.parametrize("kind", [0, 1])
def test_pitched_k_major_views_and_strided_batches(cuda_lib, kind):
    """A and B are slices of larger buffers (row pitch > K, batch entries further apart than one matrix) and C / D
    carry their own pitch and batch stride: the result must equal the oracle's on the packed copies."""
    Lb, M, N, K = 3, 320, 384, 512
    kb = K // 2 if kind == 0 else K                       # bytes of K per row
    pa, pb = kb + 64, kb + 160                            # row pitches in bytes (16-byte multiples)
    unit = 2 if kind == 0 else 1                          # elements per byte
    bsa, bsb = (M + 5) * pa, (N + 3) * pb                 # batch strides in bytes
    ldc, ldd = N + 8, N + 24
    bsc, bsd = (M + 2) * ldc, (M + 1) * ldd
    rng = np.random.default_rng(5)
    bufA = rng.integers(0, 256, Lb * bsa, dtype=np.uint8)
    bufB = rng.integers(0, 256, Lb * bsb, dtype=np.uint8)
    bufC = G.bf16_normal((Lb * bsc,), rng)
    want, sfas, sfbs = [], [], []
    for l in range(Lb):
        _, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=200 + l, exact=True)
        bufA[l * bsa: l * bsa + M * pa].reshape(M, pa)[:, :kb] = A
        bufB[l * bsb: l * bsb + N * pb].reshape(N, pb)[:, :kb] = B
        Cl = bufC[l * bsc: l * bsc + M * ldc].reshape(M, ldc)[:, :N]
        sfas.append(sfa); sfbs.append(sfb)
        want.append(oracle_bf16(kind, M, N, K, A, sfa, B, sfb, np.ascontiguousarray(Cl), 2.0, 0.5))
    dA, dB, dC = dev(bufA), dev(bufB), dev(bufC)
    dSFA, dSFB = dev(np.concatenate(sfas)), dev(np.concatenate(sfbs))
    dD = torch.full((Lb * bsd,), 0x7FC0, dtype=torch.int16, device="cuda")
    a = L.GemmArgs()
    a.kind, a.batch, a.M, a.N, a.K = kind, Lb, M, N, K
    a.A, a.B, a.SFA, a.SFB, a.C, a.D = (x.data_ptr() for x in (dA, dB, dSFA, dSFB, dC, dD))
    a.alpha, a.beta = 2.0, 0.5
    a.lda, a.ldb, a.ldc, a.ldd = pa * unit, pb * unit, ldc, ldd
    a.batch_stride_A, a.batch_stride_B, a.batch_stride_C, a.batch_stride_D = bsa * unit, bsb * unit, bsc, bsd
    _run(a)
    got = dD.cpu().numpy().view(np.uint16)
    for l in range(Lb):
        blk = got[l * bsd: l * bsd + M * ldd].reshape(M, ldd)
        assert np.array_equal(blk[:, :N], want[l]), f"batch entry {l}"
        assert np.all(blk[:, N:] == 0x7FC0), "the pitch padding of D must stay untouched"
    assert np.all(got[(Lb - 1) * bsd + M * ldd:] == 0x7FC0)


@pytest.mark.parametrize("use_pdl", [0, 1])
def test_back_to_back_launches_with_programmatic_dependent_launch(cuda_lib, use_pdl):
    """A chain in which every GEMM reads what the previous one wrote as its C: with use_pdl the kernels' set-up
    overlaps the predecessor's tail, and the results must still be those of the serial chain."""
    M, N, K = 512, 512, 256
    rng, A, sfa, B, sfb = make_operands(0, M, N, K, seed=77, exact=True)
    dA, dB, dSFA, dSFB = dev(A), dev(B), dev(sfa), dev(sfb)
    bufs = [torch.zeros((M, N), dtype=torch.int16, device="cuda") for _ in range(2)]
    lib = L.load()
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    steps = 6
    for i in range(steps):
        a = L.GemmArgs()
        a.kind, a.batch, a.M, a.N, a.K = 0, 1, M, N, K
        a.A, a.B, a.SFA, a.SFB = dA.data_ptr(), dB.data_ptr(), dSFA.data_ptr(), dSFB.data_ptr()
        a.C, a.D = bufs[i % 2].data_ptr(), bufs[(i + 1) % 2].data_ptr()
        a.alpha, a.beta = 1.0, 0.5
        a.use_pdl = use_pdl
        L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), 16, None))
    L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
    torch.cuda.synchronize()
    cur = np.zeros((M, N), np.uint16)
    for i in range(steps):
        cur = oracle_bf16(0, M, N, K, A, sfa, B, sfb, cur, 1.0, 0.5)
    assert np.array_equal(bufs[steps % 2].cpu().numpy().view(np.uint16), cur)


def test_cluster_shape_fields(cuda_lib):
    """The reference's cluster_shape / cluster_shape_fallback fields: the CTA pair of one MMA is the only cluster here."""
    M, N, K = 256, 256, 256
    _, A, sfa, B, sfb = make_operands(0, M, N, K, seed=3, exact=True)
    t = [dev(x) for x in (A, B, sfa, sfb)]
    D = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    a = L.GemmArgs()
    a.kind, a.batch, a.M, a.N, a.K = 0, 1, M, N, K
    a.A, a.B, a.SFA, a.SFB, a.D = (x.data_ptr() for x in (*t, D))
    a.alpha = 1.0
    a.cluster_m, a.cluster_n, a.cluster_fallback_m, a.cluster_fallback_n = 2, 1, 2, 1
    _run(a)
    assert np.array_equal(D.cpu().numpy().view(np.uint16), oracle_bf16(0, M, N, K, A, sfa, B, sfb))
    a.cluster_n = 4
    assert L.load().bsg_gemm_query(C.byref(a), None) == 3          # BSG_ERR_NOT_SUPPORTED


@pytest.mark.parametrize("out_kind", [1, 2])
@pytest.mark.parametrize("sizes", [[256, 384], [100, 0, 300, 1, 515], [700]])
def test_grouped_quantised_output_per_group(cuda_lib, out_kind, sizes):
    """Grouped GEMM with fused NVFP4 / MXFP8 output: every group's values and scale factors (one interleaved layout
    per group, padded to 128 rows -- what the next grouped GEMM takes as A / SFA) equal the oracle's quantisation of
    that group's GEMM, bit for bit; rows of other groups and the bytes past a group's last row stay untouched."""
    kind, N, K = 0, 640, 512
    vec = 16 if out_kind == 1 else 32
    rng = np.random.default_rng(9)
    total = int(np.sum(sizes))
    As, sfas, Bs, sfbs = [], [], [], []
    for m in sizes:
        A, _, sfa = G.exact_nvfp4_operand(int(m), K, rng) if m > 0 else (np.zeros((0, K // 2), np.uint8), None, np.zeros(0, np.uint8))
        B, _, sfb = G.exact_nvfp4_operand(N, K, rng)
        As.append(A); sfas.append(sfa); Bs.append(B); sfbs.append(sfb)
    pres = [oracle.gemm_fp32(kind, As[g], sfas[g], Bs[g], sfbs[g], int(m), N, K) if m > 0 else None for g, m in enumerate(sizes)]
    amax = max(float(np.abs(x).max()) for x in pres if x is not None)
    st = np.float32(448.0 * 6.0 / amax) if out_kind == 1 else np.float32(0.5)
    dA, dB = dev(np.concatenate(As, axis=0)), dev(np.stack(Bs))
    dSFA, dSFB = dev(np.concatenate(sfas)), dev(np.concatenate(sfbs))
    offs = torch.tensor(np.cumsum(sizes), dtype=torch.int32, device="cuda")
    row_bytes = N // 2 if out_kind == 1 else N
    dD = torch.full((total, row_bytes), 0x77, dtype=torch.uint8, device="cuda")
    atoms = [-(-int(m) // 128) for m in sizes]
    katoms = F.sf_k_atoms(N, vec)
    dSFD = torch.full((sum(atoms) * 512 * katoms,), 0x7F, dtype=torch.uint8, device="cuda")
    nc = torch.tensor([st], dtype=torch.float32, device="cuda")
    a = L.GroupedArgs()
    a.kind, a.out_kind, a.num_groups = kind, out_kind, len(sizes)
    a.total_M, a.N, a.K = total, N, K
    a.A, a.B, a.SFA, a.SFB, a.D = dA.data_ptr(), dB.data_ptr(), dSFA.data_ptr(), dSFB.data_ptr(), dD.data_ptr()
    a.offsets, a.SFD, a.norm_constant = offs.data_ptr(), dSFD.data_ptr(), nc.data_ptr()
    a.alpha = 1.0
    lib = L.load()
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    L.check(lib.bsg_grouped_run(C.byref(a), ws.data_ptr(), 16, None))
    L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
    torch.cuda.synchronize()
    gotD, gotSFD = dD.cpu().numpy(), dSFD.cpu().numpy()
    row, atom = 0, 0
    for g, m in enumerate(sizes):
        m = int(m)
        if m:
            Dw, SFDw = oracle.quant(0 if out_kind == 1 else 1, pres[g], float(st))
            assert np.array_equal(gotD[row:row + m], Dw), f"group {g}: values"
            sfd_g = gotSFD[atom * 512 * katoms:(atom + atoms[g]) * 512 * katoms]
            idx = R.sf_index(m, N // vec)
            assert np.array_equal(sfd_g[idx], SFDw[idx]), f"group {g}: scale factors"
        row += m
        atom += atoms[g]


@pytest.mark.parametrize("kind,M,N,K,tile_n", [(0, 2048, 2048, 512, 0), (1, 1024, 1536, 384, 0), (0, 4096, 5120, 256, 0), (1, 4096, 2560, 256, 128),
                                              (0, 300, 456, 384, 0)])
def test_dynamic_scheduler_dense(cuda_lib, kind, M, N, K, tile_n):
    """BSG_SCHED_DYNAMIC: one cluster per tile is launched and running clusters take over the tiles of clusters that
    have not started (320 and 320 tiles on 74 resident clusters in the larger cases).  Same results, bit for bit."""
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=60, exact=True)
    Cb = G.bf16_normal((M, N), rng)
    got = run_dense(kind, M, N, K, A, sfa, B, sfb, Cb, 1.0, 0.5, scheduler=L.SCHED_DYNAMIC, tile_n=tile_n)
    assert np.array_equal(got, oracle_bf16(kind, M, N, K, A, sfa, B, sfb, Cb, 1.0, 0.5))


@pytest.mark.parametrize("kind", [0, 1])
def test_dynamic_scheduler_grouped_ragged(cuda_lib, kind):
    """Grouped GEMM under the dynamic scheduler: the launch only knows an upper bound of the tile count (the group
    sizes live on the device), surplus clusters find nothing to do."""
    got, want = run_grouped(kind, [100, 0, 300, 1, 515, 2048, 77], 640, 512, seed=61, scheduler=L.SCHED_DYNAMIC)
    assert np.array_equal(got, want)


def test_dynamic_scheduler_repeated_launches_and_pdl(cuda_lib):
    """Twenty launches in a row, alternately static and dynamic, with programmatic dependent launch."""
    M, N, K = 2048, 2048, 256
    rng, A, sfa, B, sfb = make_operands(0, M, N, K, seed=62, exact=True)
    want = oracle_bf16(0, M, N, K, A, sfa, B, sfb)
    t = [dev(x) for x in (A, B, sfa, sfb)]
    outs = [torch.zeros((M, N), dtype=torch.int16, device="cuda") for _ in range(20)]
    lib = L.load()
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    for i, D in enumerate(outs):
        a = L.GemmArgs()
        a.kind, a.batch, a.M, a.N, a.K = 0, 1, M, N, K
        a.A, a.B, a.SFA, a.SFB, a.D = (x.data_ptr() for x in (*t, D))
        a.alpha, a.use_pdl, a.scheduler = 1.0, 1, i % 2
        L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), 16, None))
    L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
    torch.cuda.synchronize()
    for i, D in enumerate(outs):
        assert np.array_equal(D.cpu().numpy().view(np.uint16), want), f"launch {i}"


@pytest.mark.parametrize("kind", [2, 3])
@pytest.mark.parametrize("M,N,K,tile_n,exact", [(256, 512, 512, 0, True), (384, 640, 1024, 0, True), (512, 384, 256, 128, True),
                                               (1024, 1024, 2048, 0, False)])
def test_mxfp4_and_mixed_operands(cuda_lib, kind, M, N, K, tile_n, exact):
    """MXFP4 (e2m1 with ue8m0 scale per 32) and the mixed MXFP8 x MXFP4 form against the oracle: bit for bit on
    exact-arithmetic operands, within the bf16 tolerance on realistic ones (with beta * C)."""
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=70 + kind, exact=exact)
    Cb = G.bf16_normal((M, N), rng)
    got = run_dense(kind, M, N, K, A, sfa, B, sfb, Cb, 1.0, 0.5, tile_n=tile_n)
    want = oracle_bf16(kind, M, N, K, A, sfa, B, sfb, Cb, 1.0, 0.5)
    if exact:
        assert np.array_equal(got, want)
    else:
        from gpu_utils import assert_close_bf16
        assert_close_bf16(got, want)


@pytest.mark.parametrize("kind", [2, 3])
def test_mxfp4_and_mixed_grouped(cuda_lib, kind):
    got, want = run_grouped(kind, [300, 0, 129, 512], 384, 512, seed=75 + kind)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("out_kind", [1, 2])
@pytest.mark.parametrize("kind,M,N,K,pitch", [(0, 256, 512, 256, 0), (1, 384, 200, 512, 448), (0, 1280, 1096, 256, 0)])
def test_column_major_quantised_output(cuda_lib, kind, out_kind, M, N, K, pitch):
    """BSG_LAYOUT_COL_MAJOR: D stored as (N, M) with M contiguous, scale factors per 16 / 32 consecutive rows of a
    column, in the K-major scale layout of the transposed matrix.  Bit for bit the oracle's row-major routine on the
    transpose (pinned against the compiled reference's M-major output)."""
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, seed=80, exact=True)
    Cb = G.bf16_normal((M, N), rng)
    pre = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, 1.0, 0.5)
    st = float(np.float32(448.0 * 6.0 / np.abs(pre).max())) if out_kind == 1 else 0.25
    vec = 16 if out_kind == 1 else 32
    ldd = pitch or M
    col_bytes = ldd // 2 if out_kind == 1 else ldd
    dD = torch.full((N, col_bytes), 0x55, dtype=torch.uint8, device="cuda")
    dSFD = torch.full((F.numel_scale(N, M, vec),), 0x7F, dtype=torch.uint8, device="cuda")
    nc = torch.tensor([st], dtype=torch.float32, device="cuda")
    t = [dev(x) for x in (A, B, sfa, sfb, Cb)]
    a = L.GemmArgs()
    a.kind, a.out_kind, a.batch, a.M, a.N, a.K = kind, out_kind, 1, M, N, K
    a.A, a.B, a.SFA, a.SFB, a.C, a.D = (x.data_ptr() for x in (*t, dD))
    a.SFD, a.norm_constant = dSFD.data_ptr(), nc.data_ptr()
    a.alpha, a.beta, a.ldd, a.out_layout = 1.0, 0.5, ldd, L.LAYOUT_COL_MAJOR
    _run(a)
    Dw, SFDw = oracle.quant(0 if out_kind == 1 else 1, np.ascontiguousarray(pre.T), st)
    got = dD.cpu().numpy()
    used = M // 2 if out_kind == 1 else M
    assert np.array_equal(got[:, :used], Dw)
    assert np.all(got[:, used:] == 0x55), "the pitch padding of D must stay untouched"
    idx = R.sf_index(N, M // vec)
    assert np.array_equal(dSFD.cpu().numpy()[idx], SFDw[idx])


def _plain_out(out_kind, shape):
    dt = {0: torch.bfloat16, 3: torch.float16, 4: torch.float32}[out_kind]
    return torch.full(shape, float("nan"), dtype=dt, device="cuda")       # NaN: cells that are never written show up


def _as_out(pre_fp32, out_kind):
    """The oracle's fp32 epilogue value in the output type (round to nearest even, as the device conversions)."""
    if out_kind == 4:
        return pre_fp32.astype(np.float32)
    if out_kind == 3:
        return pre_fp32.astype(np.float16)
    return oracle.to_bf16(pre_fp32)


@pytest.mark.parametrize("out_kind", [3, 4])
@pytest.mark.parametrize("kind,M,N,K,batch,tile_n", [(0, 512, 512, 256, 1, 0), (1, 300, 392, 512, 1, 0), (0, 256, 1096, 256, 2, 0), (1, 640, 128, 256, 1, 128)])
def test_fp16_and_fp32_outputs(cuda_lib, kind, out_kind, M, N, K, batch, tile_n):
    """Unquantised outputs other than bf16 (the reference's operator offers Float16 / Float32 outputs too): the same
    epilogue value, converted to fp16 or stored as fp32; C stays bf16.  Bit for bit on exact operands, ragged M and N."""
    rng = np.random.default_rng(41)
    gen_a, gen_b = G.operand_generators(kind, True)
    As, Bs, pres = [], [], []
    Cb = G.bf16_normal((batch * M, N), rng)
    for b in range(batch):
        A, _, sfa = gen_a(M, K, rng)
        B, _, sfb = gen_b(N, K, rng)
        As.append((A, sfa)); Bs.append((B, sfb))
        pres.append(oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb[b * M:(b + 1) * M], 0.5, 2.0))
    want = _as_out(np.concatenate(pres, axis=0), out_kind)
    dA, dSFA = dev(np.concatenate([a for a, _ in As], axis=0)), dev(np.concatenate([s for _, s in As]))
    dB, dSFB = dev(np.concatenate([b for b, _ in Bs], axis=0)), dev(np.concatenate([s for _, s in Bs]))
    dC = dev(Cb)
    dD = _plain_out(out_kind, (batch * M, N))
    a = L.GemmArgs()
    a.kind, a.out_kind, a.batch, a.M, a.N, a.K = kind, out_kind, batch, M, N, K
    a.A, a.SFA, a.B, a.SFB, a.C, a.D = (t.data_ptr() for t in (dA, dSFA, dB, dSFB, dC, dD))
    a.alpha, a.beta, a.tile_n = 0.5, 2.0, tile_n
    _run(a)
    got = dD.cpu().numpy()
    assert not np.isnan(got).any(), "unwritten outputs"
    assert np.array_equal(got.view(np.uint16 if out_kind == 3 else np.uint32), want.view(np.uint16 if out_kind == 3 else np.uint32))


@pytest.mark.parametrize("out_kind", [3, 4])
def test_fp16_and_fp32_outputs_grouped_ragged(cuda_lib, out_kind):
    """The same through the grouped call with ragged groups: the warp that holds a group's last rows stores row by row."""
    kind, N, K = 0, 392, 256
    sizes = [100, 0, 300, 1, 515]
    rng = np.random.default_rng(43)
    total = int(np.sum(sizes))
    As, sfas, Bs, sfbs = [], [], [], []
    for m in sizes:
        A, _, sfa = G.exact_nvfp4_operand(int(m), K, rng) if m > 0 else (np.zeros((0, K // 2), np.uint8), None, np.zeros(0, np.uint8))
        B, _, sfb = G.exact_nvfp4_operand(N, K, rng)
        As.append(A); sfas.append(sfa); Bs.append(B); sfbs.append(sfb)
    want = np.concatenate([_as_out(oracle.gemm_fp32(kind, As[g], sfas[g], Bs[g], sfbs[g], int(m), N, K), out_kind)
                           for g, m in enumerate(sizes) if m > 0], axis=0)
    dA, dB = dev(np.concatenate(As, axis=0)), dev(np.stack(Bs))
    dSFA, dSFB = dev(np.concatenate(sfas)), dev(np.concatenate(sfbs))
    offs = torch.tensor(np.cumsum(sizes), dtype=torch.int32, device="cuda")
    dD = _plain_out(out_kind, (total, N))
    g = L.GroupedArgs()
    g.kind, g.out_kind, g.num_groups, g.total_M, g.N, g.K = kind, out_kind, len(sizes), total, N, K
    g.A, g.B, g.SFA, g.SFB, g.D, g.offsets = (t.data_ptr() for t in (dA, dB, dSFA, dSFB, dD, offs))
    g.alpha = 1.0
    lib = L.load()
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    L.check(lib.bsg_grouped_run(C.byref(g), ws.data_ptr(), 16, None))
    L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
    torch.cuda.synchronize()
    got = dD.cpu().numpy()
    assert not np.isnan(got).any(), "unwritten outputs"
    assert np.array_equal(got.view(np.uint16 if out_kind == 3 else np.uint32), want.view(np.uint16 if out_kind == 3 else np.uint32))


def test_fp32_output_through_the_operator_api(cuda_lib):
    import cutlass_b200 as ops
    kind, M, N, K = 0, 384, 512, 512
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, 47, True)
    Aop = ops.ScaledOperand(dev(A), dev(sfa), ops.ScaleMode.Blockwise1x16, ops.ScaleSwizzleMode.Swizzle32x4x4)
    Bop = ops.ScaledOperand(dev(B).t(), dev(sfb), ops.ScaleMode.Blockwise1x16, ops.ScaleSwizzleMode.Swizzle32x4x4)
    out = torch.empty((M, N), dtype=torch.float32, device="cuda")
    args = ops.GemmArguments(Aop, Bop, out, torch.float32)
    op = ops.get_operators(args)[0]
    op.run(args)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K).astype(np.float32))


@pytest.mark.parametrize("out_kind", [5, 6])
@pytest.mark.parametrize("kind,M,N,K,alpha", [(0, 512, 512, 256, 1.0), (1, 300, 400, 512, 0.37), (0, 256, 1104, 256, 700.0), (1, 384, 208, 128, 1.0e4)])
def test_e4m3_and_e5m2_outputs_without_scale_factors(cuda_lib, kind, out_kind, M, N, K, alpha):
    """8-bit floating-point outputs (no scale factors): the epilogue value converted with round-to-nearest-even and
    saturation, as the reference's float_e4m3_t / float_e5m2_t do (the numpy codecs are pinned to those in the golden
    vectors).  The alphas spread the results over the formats' ranges, past their largest finite values and into the
    subnormals; ragged M and N."""
    rng = np.random.default_rng(51)
    gen_a, gen_b = G.operand_generators(kind, True)
    A, _, sfa = gen_a(M, K, rng)
    B, _, sfb = gen_b(N, K, rng)
    Cb = G.bf16_normal((M, N), rng)
    pre = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, alpha, 0.125)
    want = (F.encode_e4m3 if out_kind == 5 else F.encode_e5m2)(pre)
    dD = torch.full((M, N), 0x7F, dtype=torch.uint8, device="cuda")
    a = L.GemmArgs()
    a.kind, a.out_kind, a.batch, a.M, a.N, a.K = kind, out_kind, 1, M, N, K
    dA, dSFA, dB, dSFB, dC = dev(A), dev(sfa), dev(B), dev(sfb), dev(Cb)
    a.A, a.SFA, a.B, a.SFB, a.C, a.D = (t.data_ptr() for t in (dA, dSFA, dB, dSFB, dC, dD))
    a.alpha, a.beta = alpha, 0.125
    _run(a)
    got = dD.cpu().numpy()
    assert np.array_equal(got, want), f"{int((got != want).sum())} of {got.size} differ"


def test_e5m2_output_through_the_operator_api(cuda_lib):
    import cutlass_b200 as ops
    kind, M, N, K = 1, 256, 320, 256
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, 53, True)
    Aop = ops.ScaledOperand(dev(A).view(torch.float8_e4m3fn), dev(sfa), ops.ScaleMode.Blockwise1x32, ops.ScaleSwizzleMode.Swizzle32x4x4)
    Bop = ops.ScaledOperand(dev(B).view(torch.float8_e4m3fn).t(), dev(sfb), ops.ScaleMode.Blockwise1x32, ops.ScaleSwizzleMode.Swizzle32x4x4)
    out = torch.empty((M, N), dtype=torch.float8_e5m2, device="cuda")
    args = ops.GemmArguments(Aop, Bop, out, torch.float32)
    op = ops.get_operators(args)[0]
    op.run(args)
    torch.cuda.synchronize()
    assert np.array_equal(out.view(torch.uint8).cpu().numpy(), F.encode_e5m2(oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K)))


@pytest.mark.parametrize("tile_n", [64, 192])
@pytest.mark.parametrize("kind,M,N,K,batch", [(0, 512, 768, 512, 1), (1, 300, 456, 384, 1), (0, 256, 1160, 256, 2), (1, 1024, 64, 1024, 1), (0, 384, 192, 2048, 1)])
def test_tiles_of_64_and_192_columns(cuda_lib, kind, M, N, K, batch, tile_n):
    """Tile widths 64 and 192 (the reference offers MMA tile N in {64, 128, 192, 256}): such tiles start in the middle of
    a 128-row scale-factor atom of B every other time.  Bit for bit on exact operands with C, ragged M and N, batches."""
    rng = np.random.default_rng(61)
    gen_a, gen_b = G.operand_generators(kind, True)
    parts = [(gen_a(M, K, rng), gen_b(N, K, rng)) for _ in range(batch)]
    A = np.concatenate([p[0][0] for p in parts]); sfa = np.concatenate([p[0][2] for p in parts])
    B = np.concatenate([p[1][0] for p in parts]); sfb = np.concatenate([p[1][2] for p in parts])
    Cb = G.bf16_normal((batch * M, N), rng)
    got = run_dense(kind, M, N, K, A, sfa, B, sfb, Cb=Cb, alpha=0.5, beta=1.0, tile_n=tile_n, batch=batch)
    want = np.concatenate([oracle_bf16(kind, M, N, K, parts[b][0][0], parts[b][0][2], parts[b][1][0], parts[b][1][2], Cb[b * M:(b + 1) * M], 0.5, 1.0)
                           for b in range(batch)])
    assert np.array_equal(got, want), f"{int((got != want).sum())} of {got.size} differ"


@pytest.mark.parametrize("tile_n", [64, 192])
def test_tiles_of_64_and_192_columns_realistic_and_requantised(cuda_lib, tile_n):
    kind, M, N, K = 0, 384, 960, 1024
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, 63, False)
    got = run_dense(kind, M, N, K, A, sfa, B, sfb, tile_n=tile_n)
    want = oracle_bf16(kind, M, N, K, A, sfa, B, sfb)
    from gpu_utils import assert_close_bf16
    assert_close_bf16(got, want, rel_tol=1e-2)
    # fused NVFP4 output on exact operands: values and scale factors bit for bit
    rng, A, sfa, B, sfb = make_operands(kind, M, N, K, 65, True)
    pre = oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K)
    st = float(np.float32(448.0 * 6.0 / np.abs(pre).max()))
    gotD, gotSFD = run_dense(kind, M, N, K, A, sfa, B, sfb, out_kind=1, st=st, tile_n=tile_n)
    Dw, SFDw = oracle.quant(0, pre, st)
    idx = R.sf_index(M, N // 16)
    assert np.array_equal(gotD, Dw) and np.array_equal(gotSFD[idx], SFDw[idx])


@pytest.mark.parametrize("tile_n", [64, 192])
def test_tiles_of_64_and_192_columns_grouped(cuda_lib, tile_n):
    got, want = run_grouped(1, [100, 0, 300, 1, 515], 448, 512, seed=67, tile_n=tile_n)
    assert np.array_equal(got, want)
