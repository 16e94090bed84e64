"""COMPARISON INFRASTRUCTURE: this library against the reference's own sm_100 block-scaled GEMM kernels on the SAME
seeded operands, timed by the same event loop, outputs compared bit for bit.

  make -C baseline          (once, where the reference tree is mounted; several minutes per kernel)
  python baseline/compare.py [nvfp4] [zero] [mxfp8] [c2] [c0]

Prints one JSON line per (case, implementation).  Single GPU only; nothing in the library depends on this file.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import torch  # noqa: E402

from cutlass_b200 import formats as F  # noqa: E402
from cutlass_b200 import generators as G  # noqa: E402
from cutlass_b200 import lib as L  # noqa: E402


def _ref_lib(name: str):
    path = os.path.join(HERE, "_ref", f"libref_gpu_{name}.so")
    if not os.path.exists(path):
        return None
    rl = C.CDLL(path)
    rl.ref_gpu_describe.restype = C.c_char_p
    rl.ref_gpu_workspace_size.restype = C.c_int64
    rl.ref_gpu_init.argtypes = [C.c_void_p] * 8 + [C.c_int] * 3 + [C.c_float] * 2 + [C.c_int, C.c_void_p, C.c_void_p]
    rl.ref_gpu_launch.argtypes = [C.c_void_p]
    return rl


def _time(fn, iters: int, warm: int = 5) -> float:
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main() -> None:
    which = sys.argv[1:] or ["nvfp4", "zero", "mxfp8", "c2", "c0"]
    dev = torch.device("cuda", 0)
    lib = L.load()
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.zeros(16, dtype=torch.uint8, device=dev)

    def args_for(kind, M, N, K, A, SFA, B, SFB, D, out_kind=0, SFD=None, norm=None):
        a = L.GemmArgs()
        a.kind, a.batch, a.M, a.N, a.K, a.out_kind = kind, 1, M, N, K, out_kind
        a.A, a.B, a.SFA, a.SFB, a.D = A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), D.data_ptr()
        a.SFD = SFD.data_ptr() if SFD is not None else None
        a.norm_constant = norm.data_ptr() if norm is not None else None
        a.alpha = 1.0
        return a

    def ours(a):
        L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), 16, stream))

    def dense(tag, kind, M, N, K, ref_names, sets=3, iters=40, zero=False):
        gen = torch.Generator(device=dev)
        gen.manual_seed(0)
        make = G.gpu_nvfp4_operand if kind == 0 else G.gpu_mxfp8_operand
        S = []
        for _ in range(sets):
            A, SFA = make(M, K, gen, dev)
            B, SFB = make(N, K, gen, dev)
            if zero:
                A.zero_()
                B.zero_()
            S.append((A, SFA, B, SFB, torch.empty((M, N), dtype=torch.bfloat16, device=dev)))
        abi = [args_for(kind, M, N, K, *s) for s in S]
        ms = _time(lambda i: ours(abi[i % sets]), iters)
        L.check(lib.bsg_read_device_status(ws.data_ptr(), stream))
        fl = 2.0 * M * N * K
        print(json.dumps({"case": tag, "impl": "this library", "ms": round(ms, 5), "tflops": round(fl / ms / 1e9, 1)}), flush=True)
        for name in ref_names:
            rl = _ref_lib(name)
            if rl is None:
                print(json.dumps({"case": tag, "impl": "reference:" + name, "missing": True}), flush=True)
                continue
            rws = torch.zeros(max(int(rl.ref_gpu_workspace_size(M, N, K)), 16), dtype=torch.uint8, device=dev)
            Dr = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(sets)]

            def ref_run(i, rl=rl):
                A, SFA, B, SFB, _ = S[i % sets]
                rc = rl.ref_gpu_init(A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), None, Dr[i % sets].data_ptr(), None, None,
                                     M, N, K, 1.0, 0.0, 0, rws.data_ptr(), stream)
                assert rc == 0, rc
                assert rl.ref_gpu_launch(stream) == 0
            msr = _time(ref_run, iters)
            for i in range(sets):
                ours(abi[i])
                ref_run(i)
            torch.cuda.synchronize()
            same = all(torch.equal(S[i][4].view(torch.int16), Dr[i].view(torch.int16)) for i in range(sets))
            print(json.dumps({"case": tag, "impl": "reference:" + name, "kernel": rl.ref_gpu_describe().decode(), "ms": round(msr, 5),
                              "tflops": round(fl / msr / 1e9, 1), "output_bit_identical_to_this_library": same}), flush=True)
        del S, abi
        torch.cuda.empty_cache()

    if "nvfp4" in which:
        dense("NVFP4 8192^3 -> bf16", 0, 8192, 8192, 8192, ["nvfp4"])
    if "zero" in which:
        dense("NVFP4 8192^3 -> bf16, all-zero data", 0, 8192, 8192, 8192, ["nvfp4"], zero=True)
    if "mxfp8" in which:
        dense("MXFP8 8192^3 -> bf16", 1, 8192, 8192, 8192, ["mxfp8"])
    if "c0" in which:
        dense("NVFP4 1024^3 -> bf16", 0, 1024, 1024, 1024, ["nvfp4"], sets=4, iters=200)
    if "c2" in which:
        M, N, K = 8192, 14336, 4096
        gen = torch.Generator(device=dev)
        gen.manual_seed(2)
        A, SFA = G.gpu_nvfp4_operand(M, K, gen, dev)
        B, SFB = G.gpu_nvfp4_operand(N, K, gen, dev)
        Dbf = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        a_bf = args_for(0, M, N, K, A, SFA, B, SFB, Dbf)
        fl = 2.0 * M * N * K
        ms = _time(lambda i: ours(a_bf), 30)
        print(json.dumps({"case": "c2 shape -> bf16", "impl": "this library", "ms": round(ms, 5), "tflops": round(fl / ms / 1e9, 1)}), flush=True)
        norm = torch.tensor([448.0 * 6.0 / float(Dbf.float().abs().max())], dtype=torch.float32, device=dev)
        Dq = torch.zeros((M, N // 2), dtype=torch.uint8, device=dev)
        SFD = torch.zeros(F.numel_scale(M, N, 16), dtype=torch.uint8, device=dev)
        a_q = args_for(0, M, N, K, A, SFA, B, SFB, Dq, 1, SFD, norm)
        ms = _time(lambda i: ours(a_q), 30)
        print(json.dumps({"case": "c2 -> e2m1 + ue4m3 scale factors", "impl": "this library", "ms": round(ms, 5), "tflops": round(fl / ms / 1e9, 1)}),
              flush=True)
        rl = _ref_lib("nvfp4_sfd")
        if rl is not None:
            rws = torch.zeros(max(int(rl.ref_gpu_workspace_size(M, N, K)), 16), dtype=torch.uint8, device=dev)
            Dr, SFDr = torch.zeros_like(Dq), torch.zeros_like(SFD)

            def ref_run(i):
                rc = rl.ref_gpu_init(A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), None, Dr.data_ptr(), SFDr.data_ptr(),
                                     norm.data_ptr(), M, N, K, 1.0, 0.0, 0, rws.data_ptr(), stream)
                assert rc == 0, rc
                assert rl.ref_gpu_launch(stream) == 0
            msr = _time(ref_run, 30)
            ours(a_q)
            ref_run(0)
            torch.cuda.synchronize()
            print(json.dumps({"case": "c2 -> e2m1 + ue4m3 scale factors", "impl": "reference:nvfp4_sfd", "kernel": rl.ref_gpu_describe().decode(),
                              "ms": round(msr, 5), "tflops": round(fl / msr / 1e9, 1), "values_bit_identical": bool(torch.equal(Dq, Dr)),
                              "scale_factors_bit_identical": bool(torch.equal(SFD, SFDr))}), flush=True)


if __name__ == "__main__":
    main()
