"""Run one dense block-scaled GEMM shape (or the quantiser in front of it) through the C ABI and time it.

  python -m cutlass_b200.gemm_cli --kind mxfp8 --m 16384 --n 3584 --k 8192 [--iters 20] [--sets 3]
  python -m cutlass_b200.gemm_cli --op quantize --kind nvfp4 --m 8192 --k 8192

Operands are seeded and generated on the device; ``--sets`` operand/output sets are rotated so
that consecutive launches do not find their inputs in L2.  Prints one JSON line (milliseconds per
launch by CUDA events, TFLOP/s, the device status).  Meant for shape sweeps and for profiler
captures of a single shape; ``bench.py`` is the benchmark of record.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json


def run(kind: int, M: int, N: int, K: int, iters: int = 20, warmup: int = 5, sets: int = 3, tile_n: int = 0, cta_group: int = 0,
        raster_band: int = 0) -> dict:
    import torch
    from . import generators as G
    from . import lib as L
    lib = L.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    make = G.gpu_nvfp4_operand if kind == L.KIND_NVFP4 else G.gpu_mxfp8_operand
    bufs, args = [], []
    for _ in range(sets):
        A, SFA = make(M, K, gen, dev)
        B, SFB = make(N, K, gen, dev)
        D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        a = L.GemmArgs()
        a.kind, a.batch, a.M, a.N, a.K = kind, 1, M, N, K
        a.A, a.B, a.SFA, a.SFB, a.D = A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), D.data_ptr()
        a.alpha, a.tile_n, a.cta_group, a.raster_band = 1.0, tile_n, cta_group, raster_band
        bufs.append((A, SFA, B, SFB, D))
        args.append(a)
    ws = torch.zeros(16, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def launch(i):
        L.check(lib.bsg_gemm_run(C.byref(args[i % sets]), ws.data_ptr(), 16, stream))

    for i in range(warmup):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        launch(i)
    e1.record()
    torch.cuda.synchronize()
    L.check(lib.bsg_read_device_status(ws.data_ptr(), stream))
    ms = e0.elapsed_time(e1) / iters
    return {"kind": "nvfp4" if kind == L.KIND_NVFP4 else "mxfp8", "M": M, "N": N, "K": K, "iters": iters, "sets": sets,
            "ms": round(ms, 5), "tflops": round(2.0 * M * N * K / ms / 1e9, 1)}


def run_quantize(kind: int, rows: int, K: int, iters: int = 30, warmup: int = 3, sets: int = 3) -> dict:
    """bf16 (rows x K) -> block-scaled operand, `sets` inputs / outputs rotated (no launch finds its input in L2)."""
    import torch
    from . import lib as L
    from .arguments import ScaleMode
    from .quantize import quantize_blockscaled
    mode = ScaleMode.Blockwise1x16 if kind == L.KIND_NVFP4 else ScaleMode.Blockwise1x32
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    xs = [torch.randn((rows, K), device="cuda", generator=gen).to(torch.bfloat16) for _ in range(sets)]
    outs = [quantize_blockscaled(x, mode) for x in xs]
    for i in range(warmup):
        quantize_blockscaled(xs[i % sets], mode, out=outs[i % sets].quantized.tensor, scale_out=outs[i % sets].scale.tensor)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        quantize_blockscaled(xs[i % sets], mode, out=outs[i % sets].quantized.tensor, scale_out=outs[i % sets].scale.tensor)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    nbytes = rows * K * 2 + outs[0].quantized.tensor.numel() + outs[0].scale.tensor.numel()
    return {"op": "quantize", "kind": "nvfp4" if kind == L.KIND_NVFP4 else "mxfp8", "rows": rows, "K": K, "iters": iters,
            "ms": round(ms, 5), "algorithmic_bytes": nbytes, "GBs": round(nbytes / ms / 1e6, 1)}


def main() -> None:
    from . import lib as L
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm", choices=["gemm", "quantize"])
    ap.add_argument("--kind", default="nvfp4", choices=["nvfp4", "mxfp8"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--sets", type=int, default=3)
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--cta-group", type=int, default=0)
    ap.add_argument("--raster-band", type=int, default=0)
    a = ap.parse_args()
    kind = L.KIND_NVFP4 if a.kind == "nvfp4" else L.KIND_MXFP8
    if a.op == "quantize":
        print(json.dumps(run_quantize(kind, a.m, a.k, a.iters, a.warmup, a.sets)))
        return
    print(json.dumps(run(kind, a.m, a.n, a.k, a.iters, a.warmup, a.sets, a.tile_n, a.cta_group, a.raster_band)))


if __name__ == "__main__":
    main()
