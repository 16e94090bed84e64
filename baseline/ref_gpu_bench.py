"""COMPARISON INFRASTRUCTURE: times the reference's own sm_100 block-scaled GEMM kernel (baseline/_ref/libref_gpu_*.so,
built from the reference's headers by baseline/Makefile) with the benchmark's event loop.  Used by the reference arm of
``bench.py`` on single-GPU runs only; the library never loads it."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))


def time_kernel(name: str, kind: int, M: int, N: int, K: int, steps: int) -> dict | None:
    """Time of the reference's own sm_100 kernel (baseline/_ref/libref_gpu_<name>.so, built from the reference's
    headers by baseline/Makefile) on seeded operands of the same distribution, by the same event loop."""
    path = os.path.join(HERE, "_ref", f"libref_gpu_{name}.so")
    if not os.path.exists(path):
        return None
    try:
        import torch
        import bench
        from cutlass_b200 import generators as G
        if not torch.cuda.is_available():
            return None
        dev = torch.device("cuda", 0)
        rl = C.CDLL(path)
        rl.ref_gpu_describe.restype = C.c_char_p
        rl.ref_gpu_workspace_size.restype = C.c_int64
        rl.ref_gpu_init.argtypes = [C.c_void_p] * 8 + [C.c_int] * 3 + [C.c_float] * 2 + [C.c_int, C.c_void_p, C.c_void_p]
        rl.ref_gpu_launch.argtypes = [C.c_void_p]
        gen = torch.Generator(device=dev)
        gen.manual_seed(0)
        make = G.gpu_nvfp4_operand if kind == 0 else G.gpu_mxfp8_operand
        kb = K // 2 if kind == 0 else K
        n_sets = max(2, -(-2 * bench.L2_BYTES // ((M + N) * kb + M * N * 2)))
        sets = [(*make(M, K, gen, dev), *make(N, K, gen, dev), torch.empty((M, N), dtype=torch.bfloat16, device=dev)) for _ in range(n_sets)]
        rws = torch.zeros(max(int(rl.ref_gpu_workspace_size(M, N, K)), 16), dtype=torch.uint8, device=dev)
        stream = torch.cuda.current_stream()

        def launch(i):
            A, SFA, B, SFB, D = sets[i % n_sets]
            rc = rl.ref_gpu_init(A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), None, D.data_ptr(), None, None, M, N, K,
                                 1.0, 0.0, 0, rws.data_ptr(), stream.cuda_stream)
            if rc == 0:
                rc = rl.ref_gpu_launch(stream.cuda_stream)
            if rc != 0:
                raise RuntimeError(f"reference kernel status {rc}")
        ms = bench.time_steps(launch, steps, 3, stream)
        return {"ms_per_step": round(ms, 5), "value": round(2.0 * M * N * K / ms / 1e9, 1), "unit": "TFLOP/s", "steps": steps,
                "kernel": rl.ref_gpu_describe().decode(), "what": "the reference's CollectiveBuilder kernel for its example tile / cluster shape"}
    except Exception as exc:  # noqa: BLE001
        return {"error": repr(exc)}


