"""Timing and in-kernel trace of the tensor-parallel GEMM (profiling aid), one process per GPU:

  BSG_PROFILE=1 python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 \\
      --master-port 29511 -m cutlass_b200.tp_trace --cases 28672:0,28672:1024 [--trace] [--out-dir DIR]

A case is ``N:flags[:mode]``: N = all columns of the problem (M = 16384, K = 8192, MXFP8), ``flags`` the
ablation switches of the instrumented build (1024: the TMA producer does not wait for row blocks; 2048: nothing
is pushed -- run such a case last, it leaves the arrival counters behind; 4096 / 8192 / 12288: other shapes
of the staging ring; 32768: stage but do not store), ``mode`` = kernel | copy_engine, optionally +single.
Per case rank 0 prints one JSON line: milliseconds per call over a back-to-back loop that rotates two output
buffers (max over ranks), of isolated calls, and per rank.  With ``--trace`` one more call runs with the trace
switch (16384) set: the first and last CTA of every rank print when their push started and ended, where the
push warp waited, when the epilogue finished, and every wait of the TMA producer for a row block longer than
2 us; ranks other than 0 write to ``DIR/tp_trace_r<rank>.log``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="28672:0")
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--out-dir", default=".")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    from . import generators as G
    from . import tp as TP

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    if args.trace and rank != 0:
        sys.stdout.flush()
        os.dup2(os.open(os.path.join(args.out_dir, f"tp_trace_r{rank}.log"), os.O_WRONLY | os.O_CREAT | os.O_TRUNC), 1)

    def parse(c):
        parts = c.split(":")
        return int(parts[0]), int(parts[1]), (parts[2] if len(parts) > 2 else "kernel")

    cases = [parse(c) for c in args.cases.split(",")]
    M, K = 16384, 8192
    ms = M // world
    tp = TP.TpGemm(1, M, K)
    gen = torch.Generator(device=dev)
    gen.manual_seed(rank)
    A, SFA = G.gpu_mxfp8_operand(ms, K, gen, dev)
    tp.a_shard.copy_(A)
    tp.sfa_shard.copy_(SFA)
    Bm, SFBm = G.gpu_mxfp8_operand(max(c[0] for c in cases) // world, K, gen, dev)
    st = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for N, flags, mode in cases:
        ns = N // world
        torch.cuda.synchronize()
        dist.barrier()
        tp.set_mode(mode)
        B, SFB = Bm[:ns], SFBm[: ((ns + 127) // 128) * 128 * (K // 32)]
        outs = [torch.empty((M, ns), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        os.environ["BSG_DEBUG_FLAGS"] = str(flags)
        abis = [tp.build_args(B, SFB, o) for o in outs]
        for i in range(3):
            tp.run(B, SFB, outs[0], stream=st, abi_args=abis[0])
        torch.cuda.synchronize()
        dist.barrier()
        e0.record(st)
        for i in range(args.steps):
            tp.run(B, SFB, outs[i % 2], stream=st, abi_args=abis[i % 2])
        e1.record(st)
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
        per_rank = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(per_rank, t)
        iso = []
        for i in range(5):
            torch.cuda.synchronize()
            dist.barrier()
            e0.record(st)
            tp.run(B, SFB, outs[0], stream=st, abi_args=abis[0])
            e1.record(st)
            torch.cuda.synchronize()
            iso.append(e0.elapsed_time(e1))
        ti = torch.tensor([min(iso)], dtype=torch.float64, device=dev)
        dist.all_reduce(ti, op=dist.ReduceOp.MAX)
        if args.trace:
            os.environ["BSG_DEBUG_FLAGS"] = str(flags | 16384)
            torch.cuda.synchronize()
            dist.barrier()
            tp.run(B, SFB, outs[0], stream=st, abi_args=abis[0])
            torch.cuda.synchronize()
            os.environ["BSG_DEBUG_FLAGS"] = str(flags)
            dist.barrier()
        try:
            tp.check_device_status(st)
            status = "ok"
        except Exception as exc:  # noqa: BLE001
            status = str(exc)
        if rank == 0:
            pushed = (world - 1) * (ms * K + SFA.numel())
            print(json.dumps({"N": N, "flags": flags, "mode": mode, "world": world, "ms": round(max(x.item() for x in per_rank), 4),
                              "iso_ms": round(ti.item(), 4), "per_rank_ms": [round(x.item(), 4) for x in per_rank],
                              "bytes_pushed_per_rank": pushed, "status": status}), flush=True)
    tp.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
