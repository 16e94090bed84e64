"""Multi-GPU leg of ``bench.py``: the tensor-parallel MXFP8 GEMM (M=16384, N=28672, K=8192),
A row-sharded and gathered inside the kernel, B / D column-sharded.  Strong scaling: the whole
problem is fixed, every rank computes D[:, its columns]; time = max over ranks (device events).

After the timed loop a parity leg runs calls whose A differs from call to call, back to back, and
compares EVERY row of the output (the rank's own rows and every remote shard's) for one band of
256 columns with the CPU oracle: a rank that read a peer's rows before they had arrived, or rows
of an earlier call, cannot pass it."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

M_TP, N_TP, K_TP = 16384, 28672, 8192
PARITY_CALLS = int(os.environ.get("BSG_BENCH_PARITY_CALLS", "3"))
PARITY_COLS = 256


def _shard_operand(rows: int, K: int, seed: int, device):
    """Seeded MXFP8 operand rows (same values on whichever rank generates them)."""
    import torch
    import bench
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    return bench.gpu_mxfp8_operand(rows, K, gen, device)


def _reduce_scatter_leg(dev, rank: int, world: int, stream, steps: int) -> dict:
    """Times bsg_rs_gemm_run (MXFP8, M = 16384, N = 8192, K = 28672 / world per rank) against the unfused form (the dense
    kernel into a bf16 M x N buffer, then ncclReduceScatter), and compares the two results (they differ by the bf16
    rounding of the running sums at every hop of the ring, so the check is a tolerance, not bit equality)."""
    import torch
    import torch.distributed as dist
    from cutlass_b200 import lib as L
    from cutlass_b200 import tp as TP
    M, N, K = 16384, 8192, 28672
    kl, ms = K // world, M // world
    kind = L.KIND_MXFP8
    A, SFA = _shard_operand(M, kl, 7000 + rank, dev)
    B, SFB = _shard_operand(N, kl, 8000 + rank, dev)
    rs = TP.RsGemm(M, N)
    outs = [torch.empty((ms, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    abi = [rs.build_args(kind, A, SFA, B, SFB, o) for o in outs]
    for i in range(3):
        rs.run(kind, A, SFA, B, SFB, outs[i % 2], stream=stream, abi_args=abi[i % 2])
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        rs.run(kind, A, SFA, B, SFB, outs[i % 2], stream=stream, abi_args=abi[i % 2])
    e1.record(stream)
    torch.cuda.synchronize()
    rs.check_device_status(stream)
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    fused_ms = float(t.item()) / steps
    # unfused: every rank's full partial product in bf16, then NCCL's reduce-scatter
    lib = L.load()
    full = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    ref_out = torch.empty((ms, N), dtype=torch.bfloat16, device=dev)
    d = L.GemmArgs()
    d.kind, d.batch, d.M, d.N, d.K = kind, 1, M, N, kl
    d.A, d.SFA, d.B, d.SFB, d.D = A.data_ptr(), SFA.data_ptr(), B.data_ptr(), SFB.data_ptr(), full.data_ptr()
    d.alpha = 1.0
    ws = torch.zeros(16, dtype=torch.uint8, device=dev)

    def unfused():
        rc = lib.bsg_gemm_run(C.byref(d), ws.data_ptr(), 16, stream.cuda_stream)
        assert rc == 0, L.last_error()
        if world > 1:
            dist.reduce_scatter_tensor(ref_out, full)
        else:
            ref_out.copy_(full)
    for _ in range(2):
        unfused()
    torch.cuda.synchronize()
    dist.barrier()
    e0.record(stream)
    for _ in range(steps):
        unfused()
    e1.record(stream)
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    unfused_ms = float(t.item()) / steps
    diff = (outs[(steps - 1) % 2].float() - ref_out.float()).abs().max() / ref_out.float().abs().max().clamp_min(1e-30)
    dt = torch.tensor([float(diff)], dtype=torch.float64, device=dev)
    dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    rs.close()
    flops = 2.0 * M * N * K
    # GEMM + all-reduce: the same ring, every finished slice stored into every rank's output by the epilogue; against the
    # dense kernel followed by ncclAllReduce of the M x N bf16 partial products
    all_reduce = None
    try:
        # Legs beside the headline run by default only at the GPU counts at which their multi-rank tests have been seen
        # green (tests/test_gpu_tp.py, so far on 2 and 4 GPUs): a fault in a side leg must not cost the line.
        if os.environ.get("BSG_BENCH_AR", "1" if world <= 4 else "0") == "0":
            raise RuntimeError("not run at this GPU count by default (BSG_BENCH_AR=1 runs it)")
        ar = TP.RsGemm(M, N, all_reduce=True)
        res = None
        for _ in range(3):
            res = ar.run_all_reduce(kind, A, SFA, B, SFB, stream=stream)
        torch.cuda.synchronize()
        dist.barrier()
        e0.record(stream)
        for _ in range(steps):
            res = ar.run_all_reduce(kind, A, SFA, B, SFB, stream=stream)
        e1.record(stream)
        torch.cuda.synchronize()
        ar.check_device_status(stream)
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ar_ms = float(t.item()) / steps

        def unfused_ar():
            rc = lib.bsg_gemm_run(C.byref(d), ws.data_ptr(), 16, stream.cuda_stream)
            assert rc == 0, L.last_error()
            if world > 1:
                dist.all_reduce(full)
        for _ in range(2):
            unfused_ar()
        torch.cuda.synchronize()
        dist.barrier()
        e0.record(stream)
        for _ in range(steps):
            unfused_ar()
        e1.record(stream)
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ar_unfused_ms = float(t.item()) / steps
        ardiff = (res.float() - full.float()).abs().max() / full.float().abs().max().clamp_min(1e-30)
        adt = torch.tensor([float(ardiff)], dtype=torch.float64, device=dev)
        dist.all_reduce(adt, op=dist.ReduceOp.MAX)
        all_reduce = {"ms_per_step": round(ar_ms, 4), "value": round(flops / ar_ms / 1e9, 1), "unit": "TFLOP/s",
                      "unfused_nccl": {"ms_per_step": round(ar_unfused_ms, 4), "value": round(flops / ar_unfused_ms / 1e9, 1),
                                       "what": "the dense kernel into a bf16 M x N buffer, then ncclAllReduce in place"},
                      "max_rel_diff_vs_unfused": float(adt.item())}
        ar.close()
    except Exception as exc:  # noqa: BLE001
        all_reduce = {"error": repr(exc)}
    return {"all_reduce": all_reduce, "workload": f"MXFP8 GEMM + reduce-scatter M={M} N={N} K={K}: K sharded over the ranks, D reduced and scattered over M",
            "ms_per_step": round(fused_ms, 4), "value": round(flops / fused_ms / 1e9, 1), "unit": "TFLOP/s", "steps": steps,
            "unfused_nccl": {"ms_per_step": round(unfused_ms, 4), "value": round(flops / unfused_ms / 1e9, 1),
                             "what": "the dense kernel into a bf16 M x N buffer, then ncclReduceScatter"},
            "max_rel_diff_vs_unfused": float(dt.item()),
            "note": "the fused form rounds the running sum to bf16 at every hop, NCCL's reduction rounds once"}


def run(args) -> dict:
    import torch
    import torch.distributed as dist
    import bench
    from cutlass_b200 import formats as F
    from cutlass_b200 import lib as L
    from cutlass_b200 import tp as TP

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    M, N, K = M_TP, N_TP, K_TP
    ms, ns = M // world, N // world
    kind = L.KIND_MXFP8

    # Clocks of rank 0's GPU, sampled by a child process (nothing in this process polls during the timed region).
    smi = bench.SmiClockSampler(local).start() if rank == 0 and os.environ.get("BSG_BENCH_CLOCKS", "1") != "0" else None
    tp = TP.TpGemm(kind, M, K)
    A, SFA = _shard_operand(ms, K, 1000 + rank, dev)
    tp.a_shard.copy_(A)
    tp.sfa_shard.copy_(SFA)
    B, SFB = _shard_operand(ns, K, 2000 + rank, dev)
    n_out = 2
    outs = [torch.empty((M, ns), dtype=torch.bfloat16, device=dev) for _ in range(n_out)]
    abi = [tp.build_args(B, SFB, o) for o in outs]
    stream = torch.cuda.current_stream()
    torch.cuda.synchronize()
    dist.barrier()

    def step(i):
        tp.run(B, SFB, outs[i % n_out], stream=stream, abi_args=abi[i % n_out])

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if smi is not None:
        smi.begin()
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    torch.cuda.synchronize()
    if smi is not None:
        smi.end()
    clocks = smi.summary() if smi is not None else None
    tp.check_device_status(stream)
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    region_ms = float(t.item())
    ms_step = region_ms / args.steps
    flops = 2.0 * M * N * K
    tflops = flops / ms_step / 1e9

    # ---- parity: PARITY_CALLS calls back to back, every one with a different A on every rank; all M rows of a
    # 256-column band of every call's output against the CPU oracle
    import oracle
    oracle.set_threads(max(1, len(os.sched_getaffinity(0)) // world))
    shards = [_shard_operand(ms, K, 5000 + 100 * c + rank, dev) for c in range(PARITY_CALLS)]
    p_outs = [torch.full((M, ns), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(PARITY_CALLS)]
    p_abi = [tp.build_args(B, SFB, o) for o in p_outs]
    dist.barrier()
    for c in range(PARITY_CALLS):
        tp.a_shard.copy_(shards[c][0], non_blocking=True)          # stream-ordered after the previous call
        tp.sfa_shard.copy_(shards[c][1], non_blocking=True)
        tp.run(B, SFB, p_outs[c], stream=stream, abi_args=p_abi[c])
    torch.cuda.synchronize()
    tp.check_device_status(stream)
    cols = min(PARITY_COLS, ns)
    B_np = B[:cols].cpu().numpy()
    SFB_np = SFB[: (-(-cols // 128)) * 512 * (K // 128)].cpu().numpy()
    worst, nan_count, rows_checked = 0.0, 0, 0
    for c in range(PARITY_CALLS):
        full = [_shard_operand(ms, K, 5000 + 100 * c + q, dev) for q in range(world)]       # what every rank held in call c
        A_np = torch.cat([x[0] for x in full]).cpu().numpy()
        SFA_np = torch.cat([x[1] for x in full]).cpu().numpy()
        want = oracle.to_bf16(oracle.gemm_fp32(kind, A_np, SFA_np, B_np, SFB_np, M, cols, K))
        got = p_outs[c][:, :cols].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        gf, wf = F.bf16_to_f32(got), F.bf16_to_f32(want)
        nan_count += int(np.isnan(gf).sum())
        worst = max(worst, float(np.max(np.abs(np.nan_to_num(gf) - wf)) / max(float(np.max(np.abs(wf))), 1e-30)))
        rows_checked = M
        del full
    pt = torch.tensor([worst, float(nan_count)], dtype=torch.float64, device=dev)
    dist.all_reduce(pt, op=dist.ReduceOp.MAX)
    parity = {"calls_checked": PARITY_CALLS, "a_varies_per_step": True, "calls_back_to_back": True,
              "rows_checked_per_rank": rows_checked, "remote_rows_checked_per_rank": rows_checked - ms, "columns_checked_per_rank": cols,
              "max_rel_err_vs_cpu_oracle": float(pt[0].item()), "unwritten_or_nan_outputs": int(pt[1].item()), "tolerance": 1e-2,
              "ok": bool(pt[0].item() <= 1e-2 and pt[1].item() == 0)}
    del shards, p_outs
    tp.a_shard.copy_(A)
    tp.sfa_shard.copy_(SFA)

    # ---- unfused baseline: NCCL all-gather of A and SFA, then the plain dense kernel
    lib = L.load()
    a_full, sfa_full = torch.empty_like(tp.a_full), torch.empty_like(tp.sfa_full)
    dense = L.GemmArgs()
    dense.kind, dense.batch, dense.M, dense.N, dense.K = kind, 1, M, ns, K
    dense.A, dense.SFA, dense.B, dense.SFB, dense.D = a_full.data_ptr(), sfa_full.data_ptr(), B.data_ptr(), SFB.data_ptr(), outs[0].data_ptr()
    dense.alpha = 1.0
    ws = torch.zeros(16, dtype=torch.uint8, device=dev)

    def unfused():
        if world > 1:
            dist.all_gather_into_tensor(a_full.view(-1), A.view(-1))
            dist.all_gather_into_tensor(sfa_full, SFA)
        rc = lib.bsg_gemm_run(C.byref(dense), ws.data_ptr(), 16, stream.cuda_stream)
        assert rc == 0, L.last_error()

    if world == 1:
        a_full.copy_(A)
        sfa_full.copy_(SFA)
    for _ in range(3):
        unfused()
    torch.cuda.synchronize()
    dist.barrier()
    n_unf = max(3, min(args.steps, 20))
    e0.record(stream)
    for _ in range(n_unf):
        unfused()
    e1.record(stream)
    torch.cuda.synchronize()
    tu = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(tu, op=dist.ReduceOp.MAX)
    unfused_ms = float(tu.item()) / n_unf

    # ---- the whole problem (all N columns) on ONE GPU: the base of the strong-scaling series,
    # measured on every rank's GPU at the same time (max over ranks), A already resident
    base = None
    if world > 1:
        Bf, SFBf = _shard_operand(N, K, 3000, dev)
        Df = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        full = L.GemmArgs()
        full.kind, full.batch, full.M, full.N, full.K = kind, 1, M, N, K
        full.A, full.SFA, full.B, full.SFB, full.D = a_full.data_ptr(), sfa_full.data_ptr(), Bf.data_ptr(), SFBf.data_ptr(), Df.data_ptr()
        full.alpha = 1.0
        n_base = max(3, min(args.steps, 10))
        for i in range(3 + n_base):
            if i == 3:
                torch.cuda.synchronize()
                dist.barrier()
                e0.record(stream)
            rc = lib.bsg_gemm_run(C.byref(full), ws.data_ptr(), 16, stream.cuda_stream)
            assert rc == 0, L.last_error()
        e1.record(stream)
        torch.cuda.synchronize()
        tb = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(tb, op=dist.ReduceOp.MAX)
        base_ms = float(tb.item()) / n_base
        base = {"value": round(flops / base_ms / 1e9, 1), "unit": "TFLOP/s", "ms_per_step": round(base_ms, 4), "n_gpus": 1,
                "what": "the same M x N x K problem, all N columns, on one GPU with A resident (slowest of this run's GPUs)"}
        del Bf, SFBf, Df

    # ---- end to end with host buffers: this rank's A shard and B shard in, its D shard out, every step; two
    # output buffers and separate copy streams, so a step costs the slowest stage (all copies inside the timed region)
    hA, hSFA, hB, hSFB = (x.cpu().pin_memory() for x in (A, SFA, B, SFB))
    hD = [torch.empty((M, ns), dtype=torch.bfloat16).pin_memory() for _ in range(n_out)]
    h2d = sum(x.numel() * x.element_size() for x in (hA, hSFA, hB, hSFB))
    d2h = hD[0].numel() * hD[0].element_size()
    s_out = torch.cuda.Stream(dev)
    ev_mm = [torch.cuda.Event() for _ in range(n_out)]
    ev_out = [torch.cuda.Event() for _ in range(n_out)]

    def e2e_step(i):
        b = i % n_out
        # the shard and B live in single buffers that the GEMM reads, so their copies stay on the GEMM's stream
        tp.a_shard.copy_(hA, non_blocking=True)
        tp.sfa_shard.copy_(hSFA, non_blocking=True)
        B.copy_(hB, non_blocking=True)
        SFB.copy_(hSFB, non_blocking=True)
        if i >= n_out:
            stream.wait_event(ev_out[b])
        tp.run(B, SFB, outs[b], stream=stream, abi_args=abi[b])
        ev_mm[b].record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_mm[b])
            hD[b].copy_(outs[b], non_blocking=True)
            ev_out[b].record(s_out)

    for i in range(n_out):
        e2e_step(i)
    torch.cuda.synchronize()
    dist.barrier()
    n_e2e = max(4, min(args.steps, 10))
    e0.record(stream)
    for i in range(n_out, n_out + n_e2e):
        e2e_step(i)
    s_out.wait_event(ev_out[(n_out + n_e2e - 1) % n_out])
    e1.record(s_out)
    torch.cuda.synchronize()
    te = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item()) / n_e2e
    tp.check_device_status(stream)

    # ---- the row-parallel counterpart: GEMM + reduce-scatter (K sharded, the result reduced and scattered over M),
    # the shape of the MLP's second projection: M = 16384, N = 8192, K = 28672 over all ranks
    rs_out = None
    if os.environ.get("BSG_BENCH_RS", "1" if world <= 4 else "0") != "0":
        try:
            rs_out = _reduce_scatter_leg(dev, rank, world, stream, max(3, min(args.steps, 20)))
        except Exception as exc:  # noqa: BLE001
            rs_out = {"error": repr(exc)}

    peaks = bench.measured_peaks()
    long_region = region_ms >= 1000.0
    key = "bf16_tflops_sustained" if long_region else "bf16_tflops"
    bf16 = peaks.get(key)
    peak = (2.0 * bf16 if bf16 else 2.0 * (1400.0 if long_region else 1590.0)) * world
    link_bytes = (world - 1) * (ms * K + SFA.numel())                     # received per rank per step
    out = {
        "metric": "tp_mxfp8_gemm_tflops", "value": round(tflops, 1), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "mxfp8 (e4m3 x ue8m0/32), fp32 accumulate, bf16 out", "data": "synthetic",
        "config": bench.tp_config(world),
        "kernel_config": {"l2": f"operands per rank {(ms * K + ns * K) >> 20} MiB + gathered A {(M * K) >> 20} MiB > L2; {n_out} output buffers rotated",
                          "nvlink_bytes_received_per_rank_per_step": link_bytes,
                          "pct_of_nominal_fp8_peak": round(100.0 * tflops / (bench.NOMINAL_FP8_TFLOPS * world), 1)},
        "e2e": {"value": round(flops / e2e_ms / 1e9, 1), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": d2h * world, "ms_per_step": round(e2e_ms, 4), "steps": n_e2e,
                "how": "per rank: shard and B from pinned host memory, D shard back to the host on its own stream; all copies timed"},
        "gpu_launches": args.steps * world,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": round(tflops, 1), "peak": round(peak, 1), "unit": "TFLOP/s",
                     "frac": round(tflops / peak, 4),
                     "peak_source": f"n_gpus x 2 x {key} of MEASURED_PEAKS.json (no fp8 figure is measured); the timed region is "
                                    f"{region_ms:.0f} ms long, so the {'sustained' if long_region else 'burst'} figure applies",
                     "frac_of_nominal": round(tflops / (bench.NOMINAL_FP8_TFLOPS * world), 4),
                     "nvlink_time_floor_ms": round(link_bytes / 770e9 * 1e3, 4), "traffic": None},
        "unfused_nccl": {"value": round(flops / unfused_ms / 1e9, 1), "unit": "TFLOP/s", "ms_per_step": round(unfused_ms, 4),
                         "what": "ncclAllGather(A), ncclAllGather(SFA), then the same dense kernel"},
        "scaling_base": base,
        "efficiency_vs_scaling_base": round(tflops / (world * base["value"]), 4) if base else None,
        "parity": parity,
        "reduce_scatter": rs_out,
    }
    tp.close()
    dist.barrier()
    if os.environ.get("BSG_BENCH_KEEP_PG") != "1":
        dist.destroy_process_group()
    return out
