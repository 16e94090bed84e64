"""Helpers of the -m gpu parity tests: run a problem through the C ABI (ctypes, raw device
pointers) and compute the oracle's answer for the same seeded inputs."""
import ctypes as C

import numpy as np
import torch

import oracle
from cutlass_b200 import formats as F
from cutlass_b200 import generators as G
from cutlass_b200 import lib as L


def dev(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def make_operands(kind: int, M: int, N: int, K: int, seed: int, exact: bool):
    rng = np.random.default_rng(seed)
    gen_a, gen_b = G.operand_generators(kind, exact)
    A, _, sfa = gen_a(M, K, rng)
    B, _, sfb = gen_b(N, K, rng)
    return rng, A, sfa, B, sfb


def run_dense(kind, M, N, K, A, sfa, B, sfb, Cb=None, alpha=1.0, beta=0.0, out_kind=0, st=None, tile_n=0, cta_group=0,
              batch=1, check_status=True, bias=None, bias_per_row=False, activation=0, sm_count=0, scheduler=0, use_pdl=0):
    """-> bf16 bits (batch*M, N), or (quantised values, SFD buffer) for out_kind 1 (NVFP4) / 2 (MXFP8)."""
    lib = L.load()
    dA, dB, dSFA, dSFB = dev(A), dev(B), dev(sfa), dev(sfb)
    dC = dev(Cb) if Cb is not None else None
    a = L.GemmArgs()
    a.kind, a.out_kind, a.batch = kind, out_kind, batch
    a.M, a.N, a.K = M, N, K
    a.A, a.B, a.SFA, a.SFB = dA.data_ptr(), dB.data_ptr(), dSFA.data_ptr(), dSFB.data_ptr()
    a.C = dC.data_ptr() if dC is not None else None
    a.alpha, a.beta = alpha, beta
    a.tile_n, a.cta_group = tile_n, cta_group
    a.sm_count, a.scheduler, a.use_pdl = sm_count, scheduler, use_pdl
    dbias = dev(np.asarray(bias, dtype=np.float32)) if bias is not None else None
    if dbias is not None:
        a.bias, a.bias_mode = dbias.data_ptr(), (L.BIAS_PER_ROW if bias_per_row else L.BIAS_PER_COLUMN)
    a.activation = activation
    rows = batch * M
    keep = []
    if out_kind == 0:
        dD = torch.full((rows, N), 0x7FC0, dtype=torch.int16, device="cuda")      # NaN pattern: unwritten cells show up
    else:
        dD = torch.full((rows, N // 2 if out_kind == 1 else N), 0x77, dtype=torch.uint8, device="cuda")
        dSFD = torch.full((batch * F.numel_scale(M, N, 16 if out_kind == 1 else 32),), 0x7F, dtype=torch.uint8, device="cuda")
        a.SFD = dSFD.data_ptr()
        keep += [dSFD]
        if st is not None:
            dst = torch.tensor([st], dtype=torch.float32, device="cuda")
            a.norm_constant = dst.data_ptr()
            keep += [dst]
    a.D = dD.data_ptr()
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), 16, None))
    if check_status:
        L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
    torch.cuda.synchronize()
    if out_kind == 0:
        return dD.cpu().numpy().view(np.uint16)
    return dD.cpu().numpy(), keep[0].cpu().numpy()


def oracle_bf16(kind, M, N, K, A, sfa, B, sfb, Cb=None, alpha=1.0, beta=0.0, bias=None, bias_per_row=False, activation=0):
    return oracle.to_bf16(oracle.gemm_fp32(kind, A, sfa, B, sfb, M, N, K, Cb, alpha, beta, bias=bias, bias_per_row=bias_per_row,
                                           activation=activation))


def assert_close_bf16(got_bits, want_bits, rel_tol=1e-2):
    """bf16 outputs must match the oracle within rel_tol of the largest magnitude, element-wise
    within rel_tol relative error where the reference is not tiny, and contain no NaN."""
    got, want = F.bf16_to_f32(got_bits), F.bf16_to_f32(want_bits)
    assert not np.isnan(got).any(), f"{int(np.isnan(got).sum())} NaN / unwritten outputs"
    scale = max(float(np.max(np.abs(want))), 1e-30)
    err = np.abs(got - want)
    assert float(err.max()) <= rel_tol * scale, f"max abs err {err.max()} vs scale {scale}"
    big = np.abs(want) > 0.05 * scale
    if big.any():
        assert float((err[big] / np.abs(want[big])).max()) <= rel_tol


def run_grouped(kind, sizes, N, K, seed, exact=True, alpha=1.0, beta=0.0, tile_n=0, cta_group=0, with_bias=False, activation=0,
                per_group_scalars=False, scheduler=0):
    """Ragged grouped GEMM through the C ABI and the per-group oracle.  -> (got bits, want bits)."""
    rng = np.random.default_rng(seed)
    gen, gen_b = G.operand_generators(kind, exact)
    total = int(np.sum(sizes))
    As, sfas, Bs, sfbs = [], [], [], []
    for m in sizes:
        A, _, sfa = gen(int(m), K, rng) if m > 0 else (np.zeros((0, K // 2 if kind in (0, 2) else K), np.uint8), None, np.zeros(0, np.uint8))
        B, _, sfb = gen_b(N, K, rng)
        As.append(A); sfas.append(sfa); Bs.append(B); sfbs.append(sfb)
    Cb = G.bf16_normal((total, N), rng) if beta != 0 else None
    A_all = np.concatenate(As, axis=0)
    bias = (rng.standard_normal((len(sizes), N)) * 2).astype(np.float32) if with_bias else None
    # per-group alpha / beta: powers of two keep the exact-arithmetic property; alpha stays positive because the oracle
    # adds 0 * C where the kernel skips C (beta == 0), which differs in the sign of a zero result only
    alphas = rng.choice([0.5, 1.0, 2.0, 4.0, 0.25], len(sizes)).astype(np.float32) if per_group_scalars else None
    betas = rng.choice([0.0, 0.5, 1.0, -2.0], len(sizes)).astype(np.float32) if per_group_scalars else None
    if per_group_scalars and Cb is None:
        Cb = G.bf16_normal((total, N), rng)
    want = np.zeros((total, N), np.uint16)
    row = 0
    for g, m in enumerate(sizes):
        m = int(m)
        if m:
            cg = Cb[row:row + m] if Cb is not None else None
            ag, bg = (float(alphas[g]), float(betas[g])) if per_group_scalars else (alpha, beta)
            want[row:row + m] = oracle_bf16(kind, m, N, K, As[g], sfas[g], Bs[g], sfbs[g], cg, ag, bg,
                                            bias=bias[g] if with_bias else None, activation=activation)
        row += m
    lib = L.load()
    dA, dB = dev(A_all), dev(np.stack(Bs))
    dSFA = dev(np.concatenate(sfas) if total else np.zeros(16, np.uint8))
    dSFB = dev(np.concatenate(sfbs))
    dC = dev(Cb) if Cb is not None else None
    offs = torch.tensor(np.cumsum(sizes), dtype=torch.int32, device="cuda")
    dD = torch.full((max(total, 1), N), 0x7FC0, dtype=torch.int16, device="cuda")
    a = L.GroupedArgs()
    a.kind, a.out_kind, a.num_groups = kind, 0, len(sizes)
    a.total_M, a.N, a.K = total, N, K
    a.A, a.B, a.SFA, a.SFB, a.D = dA.data_ptr(), dB.data_ptr(), dSFA.data_ptr(), dSFB.data_ptr(), dD.data_ptr()
    a.C = dC.data_ptr() if dC is not None else None
    a.offsets = offs.data_ptr()
    a.alpha, a.beta = alpha, beta
    a.tile_n, a.cta_group = tile_n, cta_group
    dbias = dev(bias) if with_bias else None
    a.bias = dbias.data_ptr() if with_bias else None
    dal, dbe = (dev(alphas), dev(betas)) if per_group_scalars else (None, None)
    if per_group_scalars:
        a.alpha_array, a.beta_array = dal.data_ptr(), dbe.data_ptr()
    a.activation = activation
    a.scheduler = scheduler
    ws = torch.zeros(16, dtype=torch.uint8, device="cuda")
    L.check(lib.bsg_grouped_run(C.byref(a), ws.data_ptr(), 16, None))
    L.check(lib.bsg_read_device_status(ws.data_ptr(), None))
    torch.cuda.synchronize()
    return dD.cpu().numpy().view(np.uint16)[:total], want
