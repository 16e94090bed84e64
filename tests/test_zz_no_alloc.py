"""The entry point that allocates nothing (bsg_gemm_run_static).

Some callers may not allocate device memory at all -- a serving process whose framework has
reserved every byte up front, a plug-in hook that is forbidden to touch the allocator -- so they
cannot pass a workspace to bsg_gemm_run.  For them the library keeps the kernel's scratch in a small
fixed array inside the library itself.  This test calls that entry point through the C ABI twice in a
row (the array is shared and keeps the previous call's contents, so the second call must be as good
as the first) and compares each result with what the ordinary entry point produces for the same
arguments: the outputs must be identical bit for bit, which is the tolerance the other exact-input
GPU tests use.  Both are also compared with the CPU oracle, so the test stands on its own.  The file
name keeps it last in collection order.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from cutlass_b200 import generators as G
from cutlass_b200 import lib as L

pytestmark = pytest.mark.gpu


def _problem(kind, M, N, K, seed):
    rng = np.random.default_rng(seed)
    gen = G.exact_nvfp4_operand if kind == 0 else G.exact_mxfp8_operand
    A, _, sfa = gen(M, K, rng)
    B, _, sfb = gen(N, K, rng)
    Cb = G.bf16_normal((M, N), rng)
    t = [torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in (A, B, sfa, sfb, Cb)]
    a = L.GemmArgs()
    a.kind, a.out_kind, a.batch = kind, L.OUT_BF16, 1
    a.M, a.N, a.K = M, N, K
    a.A, a.B, a.SFA, a.SFB, a.C = (x.data_ptr() for x in t)
    a.alpha, a.beta = 1.0, 0.5
    import oracle
    want = oracle.to_bf16(oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, 1.0, 0.5))
    return a, t, want


def test_static_scratch_entry_matches_workspace_entry_twice(cuda_lib):
    lib = cuda_lib
    for call, (kind, M, N, K) in enumerate([(0, 384, 512, 768), (1, 512, 264, 384)]):
        a, keep, oracle_bits = _problem(kind, M, N, K, seed=call)
        want = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
        got = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
        ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
        a.D = want.data_ptr()
        L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), 16, None))
        L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
        a.D = got.data_ptr()
        status = C.c_uint32(0xFFFFFFFF)
        L.check(lib.bsg_gemm_run_static(C.byref(a), None, C.byref(status)))
        assert status.value == 0, f"call {call}: device status {status.value:#x}"
        torch.cuda.synchronize()
        assert not torch.any(got == 0x7FC0), f"call {call}: some outputs were never written"
        assert torch.equal(got, want), f"call {call}: static-scratch result differs from the workspace result"
        assert np.array_equal(got.cpu().numpy().view(np.uint16), oracle_bits), f"call {call}: result differs from the CPU oracle"
        del keep


def test_static_scratch_entry_rejects_what_the_ordinary_entry_rejects(cuda_lib):
    a, keep, _ = _problem(0, 128, 128, 64, seed=9)
    a.D = torch.zeros((128, 128), dtype=torch.int16, device="cuda").data_ptr()
    a.K = 48                                   # not a multiple of 32: refused by the argument check, which runs first
    assert cuda_lib.bsg_gemm_run_static(C.byref(a), None, None) == 1
    assert "multiple of" in L.last_error()
