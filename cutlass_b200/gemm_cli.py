"""Run one dense block-scaled GEMM shape (or the quantiser in front of it) through the C ABI and time it.

  python -m cutlass_b200.gemm_cli --kind mxfp8 --m 16384 --n 3584 --k 8192 [--iters 20] [--sets 3]
  python -m cutlass_b200.gemm_cli --op quantize --kind nvfp4 --m 8192 --k 8192
  BSG_PROFILE=1 python -m cutlass_b200.gemm_cli --timeline --kind nvfp4 --m 8192 --n 8192 --k 8192

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


def run_timeline(kind: int, M: int, N: int, K: int, burst: int = 40) -> dict:
    """In-kernel timeline of the instrumented build (BSG_PROFILE=1: ``python -m cutlass_b200.build`` with that variable
    set, then this command with it).  The first cluster's leader CTA stamps the SM clock in shared memory -- the MMA warp
    at every k-tile (operands ready: 11, instructions issued: 12) and around its wait for the accumulator (9, 10), the
    epilogue when the accumulator is complete (20), read (22) and handed back (21) -- and copies the stamps behind the
    first 1024 bytes of the workspace.  The last launch of a burst of `burst` is read out; cycle counts are medians over
    its tiles (first and last tile left out)."""
    import os

    import numpy as np
    import torch
    from . import formats as F
    from . import lib as L
    if os.environ.get("BSG_PROFILE") != "1":
        raise SystemExit("set BSG_PROFILE=1 (the instrumented library) for --timeline")
    os.environ["BSG_DEBUG_FLAGS"] = "1"
    lib = L.load()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    from . import generators as G
    make = G.gpu_nvfp4_operand if kind == L.KIND_NVFP4 else G.gpu_mxfp8_operand
    A, SFA = make(M, K, gen, dev)
    B, SFB = make(N, K, gen, dev)
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    ws = torch.zeros(1024 + 1792 * 4, dtype=torch.uint8, device=dev)
    a = L.GemmArgs()
    a.kind, a.batch, a.M, a.N, a.K = kind, 1, M, N, K
    a.A, a.B, a.SFA, a.SFB, a.D = A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), D.data_ptr()
    a.alpha = 1.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(burst):
        if i == burst - 1:
            torch.cuda.synchronize()
            ws.zero_()
            e0.record()
        L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), ws.numel(), None))
    e1.record()
    torch.cuda.synchronize()
    raw = ws[1024:].cpu().numpy().view(np.uint32)

    def region(off):
        n = int(raw[off])
        e = raw[off + 1: off + max(n, 1)].astype(np.int64)
        code, clk = e >> 26, e & 0x3FFFFFF
        if len(clk) > 1:
            clk = clk + np.concatenate([[0], np.cumsum(np.diff(clk) < 0)]) * (1 << 26)      # the stamps hold 26 bits of the clock
        return code, clk
    mc, mt = region(512)
    ec, et = region(1536)
    if len(mt) and len(et) and abs(int(et[0]) - int(mt[0])) > (1 << 25):
        et = et + (1 << 26) * (1 if et[0] < mt[0] else -1)
    i9, i10 = np.nonzero(mc == 9)[0], np.nonzero(mc == 10)[0]
    per_k, acc_wait, span = [], [], []
    for t in range(1, min(len(i9), len(i10)) - 1):
        seg_c, seg_t = mc[i10[t]: i9[t + 1]], mt[i10[t]: i9[t + 1]]
        t11 = seg_t[seg_c == 11]
        if len(t11) > 2:
            per_k.append(float(np.median(np.diff(t11))))
        acc_wait.append(int(mt[i10[t]] - mt[i9[t]]))
        span.append(int(seg_t[-1] - mt[i10[t]]))
    e20, e21, e22 = et[ec == 20], et[ec == 21], et[ec == 22]
    n = min(len(e20), len(e21), len(e22))
    ms = e0.elapsed_time(e1)
    total = int(max(mt[-1], et[-1]) - mt[0]) if len(mt) and len(et) else 0
    med = lambda v: float(np.median(v)) if len(v) else None  # noqa: E731
    return {"kind": "nvfp4" if kind == L.KIND_NVFP4 else "mxfp8", "M": M, "N": N, "K": K, "kernel_ms": round(ms, 4),
            "first_cluster_cycles": total, "implied_sm_mhz": round(total / ms / 1e3) if ms else None, "tiles_measured": len(acc_wait),
            "cycles_per_k_tile": med(per_k), "mma_warp_accumulator_wait_cycles": med(acc_wait), "mainloop_span_cycles": med(span),
            "tile_period_cycles": med(np.diff(e20)) if len(e20) > 2 else None,
            "epilogue_ready_to_first_columns_read": med(e22[:n] - e20[:n]) if n else None,
            "epilogue_read_to_accumulator_handed_back": med(e21[:n] - e22[:n]) if n else None}


def main() -> None:
    from . import lib as L
    ap = argparse.ArgumentParser()
    ap.add_argument("--timeline", action="store_true", help="in-kernel cycle stamps of the instrumented build (BSG_PROFILE=1)")
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
    if a.timeline:
        print(json.dumps(run_timeline(kind, a.m, a.n, a.k)))
        return
    if a.op == "quantize":
        print(json.dumps(run_quantize(kind, a.m, a.k, a.iters, a.warmup, a.sets)))
        return
    print(json.dumps(run(kind, a.m, a.n, a.k, a.iters, a.warmup, a.sets, a.tile_n, a.cta_group, a.raster_band)))


if __name__ == "__main__":
    main()
