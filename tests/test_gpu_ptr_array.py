"""Pointer-array grouped GEMM on the GPU: every group has its own (M, N, K), tensors and pitches; one launch.
Each group's result equals the oracle's GEMM of that group (the check of the reference's grouped example,
examples/75_blackwell_grouped_gemm/75_blackwell_grouped_gemm_block_scaled.cu:735-790: per-group host reference)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from cutlass_b200 import formats as F
from cutlass_b200 import generators as G
from cutlass_b200 import lib as L
from cutlass_b200.ptr_array import GroupProblem, PtrArrayGemm
from oracle import ref_numpy as R
from tests.gpu_utils import assert_close_bf16, dev

pytestmark = pytest.mark.gpu


def _group(kind, M, N, K, rng, exact, pitch_pad=0, with_c=False, out_kind=0):
    gen_a, gen_b = G.operand_generators(kind, exact)
    A, _, sfa = gen_a(M, K, rng)
    B, _, sfb = gen_b(N, K, rng)
    kb = A.shape[1]
    # a pitch larger than the row: the group's A is a column slice of a wider buffer
    dA_full = torch.zeros((M, kb + pitch_pad), dtype=torch.uint8, device="cuda")
    dA_full[:, :kb] = dev(A)
    dA = dA_full[:, :kb]
    Cb = G.bf16_normal((M, N), rng) if with_c else None
    if out_kind == 0:
        dD = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
        dSFD = None
    else:
        vec = 16 if out_kind == 1 else 32
        dD = torch.full((M, N // 2 if out_kind == 1 else N), 0x77, dtype=torch.uint8, device="cuda")
        dSFD = torch.full((F.numel_scale(M, N, vec),), 0x7F, dtype=torch.uint8, device="cuda")
    host = dict(A=A, sfa=sfa, B=B, sfb=sfb, C=Cb, M=M, N=N, K=K)
    g = GroupProblem(A=dA, SFA=dev(sfa), B=dev(B), SFB=dev(sfb), D=dD, C=dev(Cb) if with_c else None, SFD=dSFD)
    return host, g


SHAPES = [
    # (M, N, K) per group: different N and K, ragged M, a group smaller than a tile, one that is empty
    [(300, 640, 512), (1, 128, 256), (0, 256, 256), (517, 384, 1024), (256, 1024, 128)],
    [(128, 128, 128), (1000, 256, 384)],
]


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("shapes", SHAPES)
def test_every_group_matches_its_own_oracle_gemm(cuda_lib, kind, shapes):
    rng = np.random.default_rng(31 + kind)
    hosts, groups = [], []
    for i, (M, N, K) in enumerate(shapes):
        if M == 0:
            M_alloc = 1        # a group with no rows still needs valid pointers in the arrays
            h, g = _group(kind, M_alloc, N, K, rng, exact=True)
            g = GroupProblem(A=g.A[:0], SFA=g.SFA, B=g.B, SFB=g.SFB, D=g.D[:0])
            h["M"] = 0
        else:
            h, g = _group(kind, M, N, K, rng, exact=True, pitch_pad=64 if i % 2 else 0)
        hosts.append(h); groups.append(g)
    op = PtrArrayGemm(kind, groups)
    op.run()
    op.check_device_status()
    torch.cuda.synchronize()
    for i, (h, g) in enumerate(zip(hosts, groups)):
        if h["M"] == 0:
            continue
        want = oracle.to_bf16(oracle.gemm_fp32(kind, h["A"], h["sfa"], h["B"], h["sfb"], h["M"], h["N"], h["K"]))
        got = g.D.cpu().numpy().view(np.uint16)
        assert np.array_equal(got, want), f"group {i} {h['M']}x{h['N']}x{h['K']}: {int((got != want).sum())} cells differ"


def test_per_group_scalars_and_addend(cuda_lib):
    kind = 0
    rng = np.random.default_rng(77)
    shapes = [(200, 256, 256), (384, 512, 512), (64, 128, 128)]
    hosts, groups = zip(*[_group(kind, M, N, K, rng, exact=True, with_c=True) for (M, N, K) in shapes])
    alphas = np.array([0.5, 2.0, 1.0], np.float32)
    betas = np.array([1.0, 0.0, -2.0], np.float32)
    op = PtrArrayGemm(kind, list(groups))
    op.run(alpha_array=dev(alphas), beta_array=dev(betas), activation=L.ACT_RELU)
    op.check_device_status()
    torch.cuda.synchronize()
    for i, (h, g) in enumerate(zip(hosts, groups)):
        want = oracle.to_bf16(oracle.gemm_fp32(kind, h["A"], h["sfa"], h["B"], h["sfb"], h["M"], h["N"], h["K"], h["C"],
                                               float(alphas[i]), float(betas[i]), activation=L.ACT_RELU))
        assert np.array_equal(g.D.cpu().numpy().view(np.uint16), want), f"group {i}"


def test_realistic_mxfp8_groups_within_tolerance(cuda_lib):
    kind = 1
    rng = np.random.default_rng(5)
    shapes = [(700, 768, 2048), (130, 256, 4096)]
    hosts, groups = zip(*[_group(kind, M, N, K, rng, exact=False) for (M, N, K) in shapes])
    op = PtrArrayGemm(kind, list(groups))
    op.run()
    op.check_device_status()
    torch.cuda.synchronize()
    for h, g in zip(hosts, groups):
        want = oracle.to_bf16(oracle.gemm_fp32(kind, h["A"], h["sfa"], h["B"], h["sfb"], h["M"], h["N"], h["K"]))
        assert_close_bf16(g.D.cpu().numpy().view(np.uint16), want, rel_tol=1e-2)      # the tolerance north_star states for bf16 outputs


@pytest.mark.parametrize("out_kind", [1, 2])
def test_quantised_output_per_group(cuda_lib, out_kind):
    """Fused NVFP4 / MXFP8 output with the groups' own SFD tensors: values and scale factors bit for bit."""
    kind = 0
    vec = 16 if out_kind == 1 else 32
    rng = np.random.default_rng(13)
    shapes = [(200, 256, 256), (384, 640, 512), (77, 128, 128)]
    hosts, groups = zip(*[_group(kind, M, N, K, rng, exact=True, out_kind=out_kind) for (M, N, K) in shapes])
    pres = [oracle.gemm_fp32(kind, h["A"], h["sfa"], h["B"], h["sfb"], h["M"], h["N"], h["K"]) for h in hosts]
    amax = max(float(np.abs(x).max()) for x in pres)
    st = np.float32(448.0 * 6.0 / amax) if out_kind == 1 else np.float32(0.5)
    nc = torch.tensor([st], dtype=torch.float32, device="cuda")
    op = PtrArrayGemm(kind, list(groups), out_kind=out_kind, norm_constant=nc)
    op.run()
    op.check_device_status()
    torch.cuda.synchronize()
    for i, (h, g) in enumerate(zip(hosts, groups)):
        Dw, SFDw = oracle.quant(0 if out_kind == 1 else 1, pres[i], float(st))
        assert np.array_equal(g.D.cpu().numpy(), Dw), f"group {i}: values"
        idx = R.sf_index(h["M"], h["N"] // vec)
        assert np.array_equal(g.SFD.cpu().numpy()[idx], SFDw[idx]), f"group {i}: scale factors"


def test_run_without_initialize_and_changed_sizes_are_refused(cuda_lib):
    kind = 0
    rng = np.random.default_rng(3)
    _, g = _group(kind, 128, 128, 128, rng, exact=True)
    op = PtrArrayGemm(kind, [g])
    lib = L.load()
    other = torch.zeros(op._ws_bytes + 128, dtype=torch.uint8, device="cuda")
    ptr = (other.data_ptr() + 127) & ~127
    rc = lib.bsg_ptr_array_run(C.byref(op.args), ptr, op._ws_bytes, None)
    assert rc == 2 and "initialize" in L.last_error()
    op._host["sizes"][0] = 64            # M of group 0 changed behind the table's back
    rc = lib.bsg_ptr_array_run(C.byref(op.args), op._ws_ptr, op._ws_bytes, None)
    assert rc == 2 and "differ" in L.last_error()


def test_argument_arrays_in_device_memory(cuda_lib):
    """The reference keeps the pointer, pitch and size arrays in device memory: the same table results when they are
    handed over there (bsg_ptr_array_initialize_from_device copies them to the host first)."""
    kind = 1
    rng = np.random.default_rng(21)
    shapes = [(300, 256, 512), (129, 384, 256)]
    hosts, groups = zip(*[_group(kind, M, N, K, rng, exact=True) for (M, N, K) in shapes])
    n = len(groups)
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device="cuda")  # noqa: E731
    sizes = torch.tensor([v for s in shapes for v in s], dtype=torch.int32, device="cuda")
    arrays = {k: i64([getattr(g, k).data_ptr() for g in groups]) for k in ("A", "B", "SFA", "SFB", "D")}
    a = L.PtrArrayArgs()
    a.kind, a.out_kind, a.num_groups = kind, 0, n
    a.problem_sizes = sizes.data_ptr()
    for k, t in arrays.items():
        setattr(a, k, t.data_ptr())
    a.alpha = 1.0
    lib = L.load()
    need = C.c_size_t()
    L.check(lib.bsg_ptr_array_workspace_size(C.byref(a), C.byref(need)))
    ws = torch.zeros(need.value + 128, dtype=torch.uint8, device="cuda")
    ptr = (ws.data_ptr() + 127) & ~127
    L.check(lib.bsg_ptr_array_initialize_from_device(C.byref(a), ptr, need.value, None))
    host_sizes = (C.c_int32 * (3 * n))(*[v for s in shapes for v in s])
    a.problem_sizes = C.cast(host_sizes, C.c_void_p)          # a run reads the sizes on the host
    L.check(lib.bsg_ptr_array_run(C.byref(a), ptr, need.value, None))
    L.check(lib.bsg_read_device_status(ptr, None))
    torch.cuda.synchronize()
    for i, (h, g) in enumerate(zip(hosts, groups)):
        want = oracle.to_bf16(oracle.gemm_fp32(kind, h["A"], h["sfa"], h["B"], h["sfb"], h["M"], h["N"], h["K"]))
        assert np.array_equal(g.D.cpu().numpy().view(np.uint16), want), f"group {i}"
