"""In-kernel timeline of one GEMM launch (profiling aid).

  BSG_PROFILE=1 python -m cutlass_b200.timeline --kind nvfp4 --m 8192 --n 8192 --k 8192 [--flags 0]

Needs the instrumented build (``BSG_PROFILE=1 python -m cutlass_b200.build``; done on demand).
The first cluster of the kernel records SM-clock stamps into the workspace: the MMA warp stamps
every k-tile (operands seen ready, instructions issued) and every tile (accumulator wait), the
epilogue warp stamps accumulator-ready and accumulator-released, the producer stamps every stage
it refills.  The summary printed here is per-k-tile and per-tile cycle counts.

``--flags`` sets the ablation switches of the instrumented build (bit 1 skip scale-factor copies,
2 skip A/B loads, 4 skip epilogue stores, 8 skip MMAs, 16 skip scale-factor loads).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os

import numpy as np


def capture(kind: int, M: int, N: int, K: int, flags: int = 0, cta_group: int = 2, tile_n: int = 256, warm: int = 60) -> dict:
    os.environ["BSG_PROFILE"] = "1"
    os.environ["BSG_DEBUG_FLAGS"] = str(256 | flags)
    import torch
    from . import build as B
    from . import formats as F
    from . import lib as L
    B.PROFILE = True
    B.OUT = os.path.join(os.path.dirname(B.OUT), B.lib_name(True, B.SF2))
    B.build()
    L.LIB_PATH = B.OUT
    lib = L.load()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    vec = 16 if kind == 0 else 32
    row_bytes = K // 2 if kind == 0 else K
    A = torch.randint(0, 255, (M, row_bytes), dtype=torch.uint8, device=dev, generator=gen)
    Bm = torch.randint(0, 255, (N, row_bytes), dtype=torch.uint8, device=dev, generator=gen)
    lo, hi = (0x28, 0x49) if kind == 0 else (124, 131)
    SFA = torch.randint(lo, hi, (F.numel_scale(M, K, vec),), dtype=torch.uint8, device=dev, generator=gen)
    SFB = torch.randint(lo, hi, (F.numel_scale(N, K, vec),), dtype=torch.uint8, device=dev, generator=gen)
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    ws = torch.zeros(1024 + 3 * 4096 * 8, dtype=torch.uint8, device=dev)
    a = L.GemmArgs()
    a.kind, a.batch, a.M, a.N, a.K = kind, 1, M, N, K
    a.A, a.B, a.SFA, a.SFB, a.D = A.data_ptr(), Bm.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), D.data_ptr()
    a.alpha, a.tile_n, a.cta_group = 1.0, tile_n, cta_group
    # Same regime as a benchmark loop: a burst of back-to-back launches, the last one is read out.
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(warm):
        if i == warm - 1:
            torch.cuda.synchronize()
            ws.zero_()
            e0.record()
        L.check(lib.bsg_gemm_run(C.byref(a), ws.data_ptr(), ws.numel(), None))
    e1.record()
    torch.cuda.synchronize()
    ev = ws[1024:].cpu().numpy().view(np.uint64).reshape(3, 4096)
    out = {"kernel_ms": e0.elapsed_time(e1)}
    for r, name in enumerate(("producer", "mma", "epilogue")):
        e = ev[r][ev[r] != 0]
        out[name] = np.stack([(e >> np.uint64(48)).astype(np.int64), (e & np.uint64(0xFFFFFFFFFFFF)).astype(np.int64)], axis=1)
    return out


def summarise(tl: dict) -> dict:
    m, e = tl["mma"], tl["epilogue"]
    i9, i10 = np.nonzero(m[:, 0] == 9)[0], np.nonzero(m[:, 0] == 10)[0]
    tiles = []
    for t in range(1, len(i10) - 1):                     # skip the first (cold) and last tile
        seg = m[i10[t]: i9[t + 1]]
        t11, t12 = seg[seg[:, 0] == 11][:, 1], seg[seg[:, 0] == 12][:, 1]
        tiles.append({"acc_wait": int(m[i10[t], 1] - m[i9[t], 1]), "k_tiles": len(t11),
                      "cycles_per_k_tile_median": float(np.median(np.diff(t11))),
                      "first4_k_tiles": int(t11[min(4, len(t11) - 1)] - t11[0]), "span": int(t12[-1] - m[i10[t], 1])})
    e20, e21 = e[e[:, 0] == 20][:, 1], e[e[:, 0] == 21][:, 1]
    n = min(len(e20), len(e21))
    med = lambda k: float(np.median([x[k] for x in tiles])) if tiles else None  # noqa: E731
    span = int(max(m[-1, 1], e[-1, 1]) - min(m[0, 1], tl["producer"][0, 1]))
    return {"kernel_ms": round(tl["kernel_ms"], 4), "first_cluster_span_cycles": span,
            "implied_sm_mhz": round(span / tl["kernel_ms"] / 1e3, 0),
            "tiles_measured": len(tiles), "k_tiles_per_tile": tiles[0]["k_tiles"] if tiles else None,
            "cycles_per_k_tile": med("cycles_per_k_tile_median"), "accumulator_wait_cycles": med("acc_wait"),
            "first4_k_tiles_cycles": med("first4_k_tiles"), "mainloop_span_cycles": med("span"),
            "tile_period_cycles": float(np.median(np.diff(e20))) if len(e20) > 2 else None,
            "epilogue_release_after_ready_cycles": float(np.median(e21[:n] - e20[:n])) if n else None}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", default="nvfp4", choices=["nvfp4", "mxfp8"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--flags", type=int, default=0)
    args = ap.parse_args()
    tl = capture(0 if args.kind == "nvfp4" else 1, args.m, args.n, args.k, args.flags)
    print(json.dumps({"kind": args.kind, "M": args.m, "N": args.n, "K": args.k, "flags": args.flags, **summarise(tl)}))


if __name__ == "__main__":
    main()
