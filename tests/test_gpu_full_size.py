"""-m gpu checks at the full BASELINE sizes, through properties that do not need a full CPU run:
row slabs against the oracle, exact scaling by powers of two, and grouped == dense per group."""
import ctypes as C

import numpy as np
import pytest
import torch

import bench
import oracle
from cutlass_b200 import formats as F
from cutlass_b200 import generators as G
from cutlass_b200 import lib as L
from oracle import ref_numpy as R

from gpu_utils import assert_close_bf16

pytestmark = pytest.mark.gpu


def _run(a, check=True):
    lib = L.load()
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), 16, None))
    if check:
        L.check(lib.bsg_read_device_status(ws.data_ptr(), None))


def _dense_args(kind, M, N, K, A, SFA, B, SFB, D):
    a = L.GemmArgs()
    a.kind, a.batch, a.M, a.N, a.K = kind, 1, M, N, K
    a.A, a.B, a.SFA, a.SFB, a.D = A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), D.data_ptr()
    a.alpha = 1.0
    return a


def _np(t):
    return t.cpu().numpy()


def test_config1_mxfp8_8192_cubed(cuda_lib):
    M = N = K = 8192
    gen = torch.Generator(device="cuda"); gen.manual_seed(1)
    A, SFA = bench.gpu_mxfp8_operand(M, K, gen, "cuda")
    B, SFB = bench.gpu_mxfp8_operand(N, K, gen, "cuda")
    D1 = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    D2 = torch.empty_like(D1)
    _run(_dense_args(1, M, N, K, A, SFA, B, SFB, D1))
    _run(_dense_args(1, M, N, K, A, SFA + 1, B, SFB, D2))          # ue8m0 exponent + 1 = every A scale x 2
    assert torch.equal(D2.float(), D1.float() * 2)
    rows, r0 = 128, 4096                                           # a slab in the middle: one 128-row SF atom
    katoms = K // 128
    want = oracle.to_bf16(oracle.gemm_fp32(1, _np(A[r0:r0 + rows]), _np(SFA[(r0 // 128) * 512 * katoms:(r0 // 128 + 1) * 512 * katoms]),
                                           _np(B), _np(SFB), rows, N, K))
    assert_close_bf16(_np(D1[r0:r0 + rows].view(torch.int16)).view(np.uint16), want)


def test_config2_nvfp4_requant_8192x14336x4096(cuda_lib):
    M, N, K = 8192, 14336, 4096
    gen = torch.Generator(device="cuda"); gen.manual_seed(2)
    A, SFA = bench.gpu_nvfp4_operand(M, K, gen, "cuda")
    B, SFB = bench.gpu_nvfp4_operand(N, K, gen, "cuda")
    Dbf = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    _run(_dense_args(0, M, N, K, A, SFA, B, SFB, Dbf))
    amax = float(Dbf.float().abs().max())
    st = np.float32(448.0 * 6.0 / amax)
    Dq = torch.zeros((M, N // 2), dtype=torch.uint8, device="cuda")
    SFD = torch.zeros(F.numel_scale(M, N, 16), dtype=torch.uint8, device="cuda")
    nc = torch.tensor([st], dtype=torch.float32, device="cuda")
    a = _dense_args(0, M, N, K, A, SFA, B, SFB, Dq)
    a.out_kind, a.SFD, a.norm_constant = L.OUT_NVFP4, SFD.data_ptr(), nc.data_ptr()
    _run(a)
    # slab: rows 256..383 (one SF row atom of A and of SFD); NVFP4 products accumulate exactly -> bit-exact
    r0, rows = 256, 128
    katoms = K // 64
    pre = oracle.gemm_fp32(0, _np(A[r0:r0 + rows]), _np(SFA[(r0 // 128) * 512 * katoms:(r0 // 128 + 1) * 512 * katoms]), _np(B), _np(SFB), rows, N, K)
    Dw, SFDw = oracle.quant_nvfp4(pre, st)
    natoms = F.sf_k_atoms(N, 16)
    got_sfd = _np(SFD[(r0 // 128) * 512 * natoms:(r0 // 128 + 1) * 512 * natoms])
    idx = R.sf_index(rows, N // 16)
    assert np.array_equal(_np(Dq[r0:r0 + rows]), Dw)
    assert np.array_equal(got_sfd[idx], SFDw[idx])
    # the quantised output dequantises back to the bf16 result within the e2m1 step (half of 1/6..1/4 of the block max)
    deq = F.decode_e2m1_codes(F.unpack_e2m1(Dw)) * np.repeat(F.decode_ue4m3(SFDw[idx]), 16, axis=1) / st
    ref = F.bf16_to_f32(_np(Dbf[r0:r0 + rows].view(torch.int16)).view(np.uint16))
    blockmax = np.repeat(np.abs(ref).reshape(rows, -1, 16).max(axis=2), 16, axis=1)
    assert np.all(np.abs(deq - ref) <= 0.26 * blockmax + 1e-3 * amax)


def test_config3_grouped_moe_64_experts(cuda_lib):
    E, K, N, tokens, topk = 64, 7168, 2048, 16384, 8
    rng = np.random.default_rng(0)
    sizes = G.moe_group_sizes(E, tokens, topk, rng)
    total = int(sizes.sum())
    assert total == 131072
    gen = torch.Generator(device="cuda"); gen.manual_seed(3)
    A, _ = bench.gpu_nvfp4_operand(total, K, gen, "cuda")
    katoms = K // 64
    atoms = [-(-int(m) // 128) for m in sizes]
    lut = torch.tensor([0x28, 0x30, 0x38, 0x40, 0x48], dtype=torch.uint8, device="cuda")
    SFA = lut[torch.randint(0, 5, (sum(atoms) * 512 * katoms,), device="cuda", generator=gen)]
    B, SFB = bench.gpu_nvfp4_operand(E * N, K, gen, "cuda")
    D = torch.full((total, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    offs = torch.tensor(np.cumsum(sizes), dtype=torch.int32, device="cuda")
    g = L.GroupedArgs()
    g.kind, g.num_groups, g.total_M, g.N, g.K = 0, E, total, N, K
    g.A, g.B, g.SFA, g.SFB, g.D, g.offsets = (x.data_ptr() for x in (A, B, SFA, SFB, D, offs))
    g.alpha = 1.0
    lib = L.load()
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    L.check(lib.bsg_grouped_run(C.byref(g), ws.data_ptr(), 16, None))
    L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
    assert not torch.isnan(D).any(), "every row of every expert must be written"
    starts = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    atom0 = np.concatenate([[0], np.cumsum(atoms)[:-1]])
    nat = N // 128
    for e in (0, int(np.argmax(sizes)), int(np.argmin(np.where(sizes > 0, sizes, 1 << 30))), E - 1):
        m = int(sizes[e])
        if m == 0:
            continue
        r0 = int(starts[e])
        sfa_e = SFA[int(atom0[e]) * 512 * katoms:(int(atom0[e]) + atoms[e]) * 512 * katoms]
        Be, SFBe = B[e * N:(e + 1) * N], SFB[e * nat * 512 * katoms:(e + 1) * nat * 512 * katoms]
        # (1) the expert's block equals the dense entry point run on that expert alone
        Dd = torch.empty((m, N), dtype=torch.bfloat16, device="cuda")
        _run(_dense_args(0, m, N, K, A[r0:r0 + m], sfa_e, Be, SFBe, Dd))
        assert torch.equal(Dd.view(torch.int16), D[r0:r0 + m].view(torch.int16)), f"expert {e}"
        # (2) its last rows (the ragged tail) match the oracle
        tail = min(m, 40)
        lo = m - tail
        a0 = lo // 128
        want = oracle.to_bf16(oracle.gemm_fp32(0, _np(A[r0 + a0 * 128:r0 + m]), _np(sfa_e[a0 * 512 * katoms:]), _np(Be), _np(SFBe),
                                               m - a0 * 128, N, K))
        assert np.array_equal(_np(D[r0 + a0 * 128:r0 + m].view(torch.int16)).view(np.uint16), want), f"expert {e} tail"
