"""Benchmark of the block-scaled GEMM path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1: NVFP4 GEMM, M = N = K = 8192 (bf16 output, alpha = 1, beta = 0), the shape the
headline metric is quoted on.  A "step" is one GEMM over one set of operands resident in
HBM; several operand sets are rotated so that every step starts with a cold L2.  The same
line carries, under ``configs``, the other single-GPU configurations (NVFP4 1024^3 with C,
MXFP8 8192^3, the 8192 x 14336 x 4096 GEMM with bf16 and with fused NVFP4 output, the
64-expert grouped GEMM), each with its own time, fraction of peak, CPU baseline and parity.
N > 1: tensor-parallel MXFP8 GEMM (M = 16384, N = 28672, K = 8192), A row-sharded and
all-gathered over NVLink inside the GEMM, B column-sharded; strong scaling, one rank per GPU.

One JSON line is printed by rank 0.  ``value`` is kernel throughput with operands in HBM;
``e2e`` is the same metric through the operator API with host buffers (pinned host -> device
copies of the operands and a device -> host read of D inside the timed region, pipelined over
three streams); ``roofline`` compares against the tensor-core peak; ``cpu_baseline`` is the
reference's host GEMM timed on this machine's CPU cores on a row slab of the same problem.

``--impl reference`` times that CPU implementation alone on the same configuration (at N > 1:
on the tensor-parallel configuration) and, at N = 1 where the reference's own sm_100 kernel has been
built (baseline/Makefile), reports its time on operands of the same distribution beside it.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

NOMINAL_FP4_TFLOPS = 9000.0
NOMINAL_FP8_TFLOPS = 4500.0
L2_BYTES = 126 * 1024 * 1024
HEADLINE_WORKLOAD = "NVFP4 block-scaled GEMM M=N=K=8192, alpha=1, beta=0, bf16 D"
TP_WORKLOAD = "tensor-parallel MXFP8 GEMM M=16384 N=28672 K=8192: A row-sharded, gathered in-kernel over NVLink; B, D column-sharded"
L2_POLICY = "operand / output sets larger than L2 (126 MiB) in total are rotated, so no step finds its inputs in L2"


def headline_config() -> dict:
    """The ``config`` object of the N = 1 line; both arms print exactly this."""
    return {"workload": HEADLINE_WORKLOAD, "M": 8192, "N": 8192, "K": 8192, "l2_policy": L2_POLICY}


def tp_config(world: int) -> dict:
    """The ``config`` object of the N > 1 lines; both arms print exactly this."""
    return {"workload": TP_WORKLOAD, "M": 16384, "N": 28672, "K": 8192, "parallelism": f"tp{world}", "l2_policy": L2_POLICY}


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {}


def tensor_peak(kind: int, sustained: bool = False) -> tuple[float, str]:
    """Roofline denominator for one GPU: no fp4 / fp8 figure is measured on this pool, so the measured bf16 GEMM
    figure is scaled by the nominal ratio (x4 for fp4, x2 for fp8); burst for kernels timed in a short region."""
    peaks = measured_peaks()
    key = "bf16_tflops_sustained" if sustained else "bf16_tflops"
    mult = 4.0 if kind == 0 else 2.0
    if peaks.get(key):
        return mult * peaks[key], f"{int(mult)} x {key} of MEASURED_PEAKS.json (no fp{'4' if kind == 0 else '8'} figure is measured)"
    return mult * (1400.0 if sustained else 1590.0), f"{int(mult)} x fallback bf16 {'1400 (sustained)' if sustained else '1590 (burst)'}"


def recorded_traffic(name: str) -> dict:
    """DRAM traffic per launch of a kernel as captured by ncu, with the commit it was captured at
    (profiles/ncu_traffic.json, written by hand from the capture named there)."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            return json.load(f).get(name, {})
    except (OSError, ValueError):
        return {}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


class SmiClockSampler:
    """Clock and throttle-reason samples from an ``nvidia-smi`` child process (one line every 10 ms), for timed regions
    that must not be disturbed: NVML polling inside the launching process slowed the multi-GPU kernel launches.
    ``start()`` early (the tool needs a moment), ``begin()`` / ``end()`` around the timed region, then ``summary()``."""

    FIELDS = "timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.t0, self.t1 = index, None, None, None

    def start(self):
        import subprocess
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index),
                                          "-lms", "10"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def begin(self):
        import datetime
        self.t0 = datetime.datetime.now()

    def end(self):
        import datetime
        self.t1 = datetime.datetime.now()

    def summary(self):
        import datetime
        if self.proc is None:
            return None
        time.sleep(0.03)                       # let the sample that covers the end of the region arrive
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
            return None
        mhz, reasons, max_mhz, total = [], set(), None, 0
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) != 7:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f")
                clk, mx = float(f[1]), float(f[2])
            except ValueError:
                continue
            total += 1
            max_mhz = mx
            if self.t0 is not None and self.t1 is not None and not (self.t0 <= ts <= self.t1 + datetime.timedelta(milliseconds=15)):
                continue
            mhz.append(clk)
            reasons.update(n for n, v in zip(self.NAMES, f[3:]) if v == "Active")
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max_mhz, "reasons": sorted(reasons),
                "samples": len(mhz), "samples_whole_run": total, "source": "nvidia-smi child process, 10 ms period"}


# --------------------------------------------------------------------------- operands
from cutlass_b200.generators import gpu_mxfp8_operand, gpu_nvfp4_operand  # noqa: E402,F401  (seeded, generated on the device)


# --------------------------------------------------------------------------- CPU baseline
def cpu_gemm_slab(kind: int, A_slab, SFA_slab, B, SFB, N: int, K: int, out_mode: int = 1, C_bits=None, alpha=1.0, beta=0.0, st=0.0):
    """One run of the reference's host GEMM (oracle/_ref when present, else the C port) on a row slab.
    -> (result, seconds, "reference" | "port").  out_mode 1: bf16 bits; 2: (packed e2m1, SFD)."""
    import oracle
    rows = A_slab.shape[0]
    ref = oracle.load_ref()
    t0 = time.perf_counter()
    if ref is not None:
        out = oracle.ref_gemm(kind, out_mode, A_slab, SFA_slab, B, SFB, rows, N, K, C_bits, alpha, beta, st)
    else:
        pre = oracle.gemm_fp32(kind, A_slab, SFA_slab, B, SFB, rows, N, K, C_bits, alpha, beta)
        out = oracle.to_bf16(pre) if out_mode == 1 else oracle.quant_nvfp4(pre, st)
    return out, time.perf_counter() - t0, ("reference" if ref is not None else "port")


def cpu_baseline_entry(rows: int, N: int, K: int, seconds: float, kind_name: str, what: str) -> dict:
    import oracle
    return {"value": round(2.0 * rows * N * K / seconds / 1e12, 5), "unit": "TFLOP/s", "cores": oracle.load_oracle().bsg_oracle_threads(),
            "kind": kind_name, "sample": f"{what} (full N={N}, K={K}); {seconds:.2f} s; scaled linearly in M", "seconds": round(seconds, 3)}


def bf16_rel_err(got_bits: np.ndarray, want_bits: np.ndarray) -> float:
    from cutlass_b200 import formats as F
    gf, wf = F.bf16_to_f32(got_bits), F.bf16_to_f32(want_bits)
    return float(np.max(np.abs(gf - wf)) / max(float(np.max(np.abs(wf))), 1e-30))


# --------------------------------------------------------------------------- timing helpers
def time_steps(launch, steps: int, warmup: int, stream) -> float:
    """Milliseconds per step: `warmup` untimed launches, then exactly `steps` launches between two events on `stream`."""
    import torch
    for i in range(warmup):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        launch(i)
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def fractions(kind: int, tflops: float) -> dict:
    peak, src = tensor_peak(kind)
    nominal = NOMINAL_FP4_TFLOPS if kind == 0 else NOMINAL_FP8_TFLOPS
    return {"frac_of_nominal": round(tflops / nominal, 4), "frac_of_measured": round(tflops / peak, 4), "measured_peak": round(peak, 1),
            "measured_peak_source": src}


class DenseCase:
    """Operand / output sets of one dense configuration, resident on the device, with their C-ABI argument blocks."""

    def __init__(self, kind, M, N, K, dev, gen, out="bf16", with_c=False, beta=0.0, min_sets=2, max_sets=8):
        import torch
        from cutlass_b200 import formats as F
        from cutlass_b200 import lib as L
        self.kind, self.M, self.N, self.K, self.out = kind, M, N, K, out
        make = gpu_nvfp4_operand if kind == 0 else gpu_mxfp8_operand
        kb = K // 2 if kind == 0 else K
        vec = 16 if kind == 0 else 32
        out_bytes = M * N * 2 if out == "bf16" else M * N // 2 + M * N // 16
        self.bytes_per_set = (M + N) * kb + (M + N) * (K // vec) + out_bytes + (M * N * 2 if with_c else 0)
        self.n_sets = min(max_sets, max(min_sets, -(-2 * L2_BYTES // self.bytes_per_set)))
        self.sets, self.args = [], []
        self.norm = None
        for _ in range(self.n_sets):
            A, SFA = make(M, K, gen, dev)
            B, SFB = make(N, K, gen, dev)
            Cm = torch.randn((M, N), device=dev, generator=gen).to(torch.bfloat16) if with_c else None
            if out == "bf16":
                D, SFD = torch.empty((M, N), dtype=torch.bfloat16, device=dev), None
            else:
                D = torch.empty((M, N // 2), dtype=torch.uint8, device=dev)
                SFD = torch.empty(F.numel_scale(M, N, 16), dtype=torch.uint8, device=dev)
            a = L.GemmArgs()
            a.kind, a.batch, a.M, a.N, a.K = kind, 1, M, N, K
            a.out_kind = L.OUT_BF16 if out == "bf16" else L.OUT_NVFP4
            a.A, a.B, a.SFA, a.SFB, a.D = A.data_ptr(), B.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), D.data_ptr()
            a.C = Cm.data_ptr() if Cm is not None else None
            a.SFD = SFD.data_ptr() if SFD is not None else None
            a.alpha, a.beta = 1.0, beta
            self.sets.append({"A": A, "SFA": SFA, "B": B, "SFB": SFB, "C": Cm, "D": D, "SFD": SFD})
            self.args.append(a)

    def set_norm(self, tensor) -> None:
        self.norm = tensor
        for a in self.args:
            a.norm_constant = tensor.data_ptr()

    def flops(self) -> float:
        return 2.0 * self.M * self.N * self.K


def run_case(lib, L, case: DenseCase, ws, stream, steps: int, warmup: int) -> float:
    def launch(i):
        rc = lib.bsg_gemm_run(C.byref(case.args[i % case.n_sets]), ws.data_ptr(), 16, stream.cuda_stream)
        if rc != 0:
            raise RuntimeError(L.last_error())
    ms = time_steps(launch, steps, warmup, stream)
    L.check(lib.bsg_read_device_status(ws.data_ptr(), stream.cuda_stream))
    return ms


def slab_of(case: DenseCase, s: dict, rows: int):
    """Host copies of the first `rows` rows of a set's A (whole atoms of SFA) and of all of B."""
    vec = 16 if case.kind == 0 else 32
    k_atoms = -(-(case.K // vec) // 4)
    A = s["A"][:rows].cpu().numpy()
    SFA = s["SFA"][: -(-rows // 128) * 512 * k_atoms].cpu().numpy()
    return A, SFA, s["B"].cpu().numpy(), s["SFB"].cpu().numpy()


# --------------------------------------------------------------------------- end to end
def e2e_pipelined(op, ops, artifact, case: DenseCase, dev, steps: int) -> dict:
    """The same GEMM through the operator API with HOST buffers: every step copies the operands from pinned host
    memory, runs the operator and copies D back.  Two operand / output sets and three streams (host -> device,
    compute, device -> host) are used, so a step costs the slowest of the three stages, not their sum; every copy
    lies inside the timed region."""
    import torch
    M, N, K = case.M, case.N, case.K
    mode, SW = ops.ScaleMode.Blockwise1x16, ops.ScaleSwizzleMode.Swizzle32x4x4
    src = case.sets[0]
    host_in = [t.cpu().pin_memory() for t in (src["A"], src["SFA"], src["B"], src["SFB"])]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = M * N * 2
    n_buf = 2
    dev_in = [[torch.empty_like(src[k]) for k in ("A", "SFA", "B", "SFB")] for _ in range(n_buf)]
    dev_out = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(n_buf)]
    host_out = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(n_buf)]
    args = [ops.GemmArguments(ops.ScaledOperand(d[0], d[1], mode, SW), ops.ScaledOperand(d[2].t(), d[3], mode, SW), o, torch.float32)
            for d, o in zip(dev_in, dev_out)]
    s_in, s_mm, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ws = torch.zeros(16, dtype=torch.uint8, device=dev)
    ev_in = [torch.cuda.Event() for _ in range(n_buf)]
    ev_mm = [torch.cuda.Event() for _ in range(n_buf)]
    ev_out = [torch.cuda.Event() for _ in range(n_buf)]

    def step(i):
        b = i % n_buf
        with torch.cuda.stream(s_in):
            if i >= n_buf:
                s_in.wait_event(ev_mm[b])            # the GEMM that last read this input set is done
            for d, h in zip(dev_in[b], host_in):
                d.copy_(h, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_mm):
            s_mm.wait_event(ev_in[b])
            if i >= n_buf:
                s_mm.wait_event(ev_out[b])           # the copy that last read this output buffer is done
            op.run(args[b], compiled_artifact=artifact, stream=s_mm, workspace=ws)
            ev_mm[b].record(s_mm)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_mm[b])
            host_out[b].copy_(dev_out[b], non_blocking=True)
            ev_out[b].record(s_out)

    for i in range(n_buf):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s_in)
    for i in range(n_buf, n_buf + steps):
        step(i)
    s_out.wait_event(ev_out[(n_buf + steps - 1) % n_buf])
    e1.record(s_out)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    op.check_device_status(workspace=ws, stream=s_mm)
    ok = bool(torch.equal(host_out[(n_buf + steps - 1) % n_buf].view(torch.int16), src["D"].cpu().view(torch.int16)))
    return {"value": round(case.flops() / ms / 1e9, 1), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": round(ms, 4), "steps": steps,
            "how": "operator API; pinned host buffers; 2 buffer sets, 3 streams (H2D, GEMM, D2H) with events; all copies timed",
            "result_equals_device_resident_run": ok}


# --------------------------------------------------------------------------- single GPU
def run_single(args) -> dict:
    import torch
    import cutlass_b200 as ops
    import oracle
    from cutlass_b200 import formats as F
    from cutlass_b200 import generators as G
    from cutlass_b200 import lib as L

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    lib = L.load()
    stream = torch.cuda.current_stream()
    ws = torch.zeros(16, dtype=torch.uint8, device=dev)
    side_steps = max(3, min(args.steps, 20))
    launches = 0

    # ---- headline: NVFP4 8192^3
    M = N = K = 8192
    head = DenseCase(0, M, N, K, dev, gen)

    def launch(i):
        rc = lib.bsg_gemm_run(C.byref(head.args[i % head.n_sets]), ws.data_ptr(), 16, stream.cuda_stream)
        if rc != 0:
            raise RuntimeError(L.last_error())

    for i in range(args.warmup):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clk:
        e0.record(stream)
        for i in range(args.steps):
            launch(i)
        e1.record(stream)
        torch.cuda.synchronize()
    L.check(lib.bsg_read_device_status(ws.data_ptr(), stream.cuda_stream))
    launches += args.steps
    ms = e0.elapsed_time(e1) / args.steps
    flops = head.flops()
    tflops = flops / ms / 1e9

    # ---- the same launches for at least a second: the clock the power limit settles at
    sustained = None
    if not args.no_sustained:
        n_long = max(200, int(1.2e3 / ms))
        with ClockSampler(0, period_s=0.01) as clk_long:
            long_ms = time_steps(launch, n_long, 0, stream)
        cs = clk_long.summary()
        sustained = {"value": round(flops / long_ms / 1e9, 1), "ms_per_step": round(long_ms, 5), "steps": n_long, "sm_mhz": cs["sm_mhz"],
                     "reasons": cs["reasons"], "ms_times_mhz": round(long_ms * cs["sm_mhz"], 1) if cs["sm_mhz"] else None,
                     "frac_of_sustained_measured": round(flops / long_ms / 1e9 / tensor_peak(0, sustained=True)[0], 4)}
        time.sleep(0.5)

    # ---- with programmatic dependent launch (bsg_gemm_args.use_pdl): set-up overlaps the previous kernel's tail
    for a in head.args:
        a.use_pdl = 1
    pdl_ms = time_steps(launch, args.steps, 3, stream)
    for a in head.args:
        a.use_pdl = 0
    L.check(lib.bsg_read_device_status(ws.data_ptr(), stream.cuda_stream))

    # ---- CPU baseline and parity on a row slab of set 0
    slab = args.cpu_rows
    launch(0)
    torch.cuda.synchronize()
    A_np, SFA_np, B_np, SFB_np = slab_of(head, head.sets[0], slab)
    want, secs, kname = cpu_gemm_slab(0, A_np, SFA_np, B_np, SFB_np, N, K)
    cpu = cpu_baseline_entry(slab, N, K, secs, kname, f"rows 0..{slab - 1} of M")
    rel = bf16_rel_err(head.sets[0]["D"][:slab].view(torch.int16).cpu().numpy().view(np.uint16), want)

    # ---- end to end through the operator API with host buffers
    mode, SW = ops.ScaleMode.Blockwise1x16, ops.ScaleSwizzleMode.Swizzle32x4x4
    s0 = head.sets[0]
    op_args = ops.GemmArguments(ops.ScaledOperand(s0["A"], s0["SFA"], mode, SW), ops.ScaledOperand(s0["B"].t(), s0["SFB"], mode, SW),
                                s0["D"], torch.float32)
    op = ops.get_operators(op_args)[0]
    artifact = op.compile(op_args)
    e2e = e2e_pipelined(op, ops, artifact, head, dev, max(4, min(args.steps, 20)))
    caps = L.Caps()
    lib.bsg_gemm_query(C.byref(head.args[0]), C.byref(caps))
    head_tile = {"tile": [caps.tile_m, caps.tile_n, caps.tile_k], "cta_group": caps.cta_group, "stages": caps.stages,
                 "operand_sets_rotated": head.n_sets, "bytes_per_set": head.bytes_per_set}
    algorithmic_bytes = head.bytes_per_set
    del head, op_args, s0
    torch.cuda.empty_cache()

    # ---- the other single-GPU configurations
    configs = {}

    def record(name, kind, case_flops, ms_case, extra):
        tf = case_flops / ms_case / 1e9
        configs[name] = {"ms": round(ms_case, 5), "tflops": round(tf, 1), **fractions(kind, tf), **extra}

    try:
        # c0: NVFP4 1024^3 with C, alpha = 1, beta = 0.5; the CPU runs it whole (this is also a full parity run)
        c0 = DenseCase(0, 1024, 1024, 1024, dev, gen, with_c=True, beta=0.5, min_sets=8, max_sets=64)
        ms0 = run_case(lib, L, c0, ws, stream, max(side_steps, 50), 5)
        launches += max(side_steps, 50)
        # the same launches replayed from a CUDA graph, with and without programmatic dependent launch: what the device
        # needs per call when the host's launch rate is out of the picture
        graph_ms = {}
        for pdl in (0, 1):
            try:
                cap = torch.cuda.Stream()
                ws_g = torch.zeros(16, dtype=torch.uint8, device=dev)
                for a0 in c0.args:
                    a0.use_pdl = pdl
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=cap):
                    for i in range(c0.n_sets):
                        rc = lib.bsg_gemm_run(C.byref(c0.args[i]), ws_g.data_ptr(), 16, cap.cuda_stream)
                        if rc != 0:
                            raise RuntimeError(L.last_error())
                with torch.cuda.stream(cap):
                    graph.replay()
                    cap.synchronize()
                    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    g0.record(cap)
                    for _ in range(4):
                        graph.replay()
                    g1.record(cap)
                torch.cuda.synchronize()
                L.check(lib.bsg_read_device_status(ws_g.data_ptr(), None))
                graph_ms["with_pdl" if pdl else "plain"] = round(g0.elapsed_time(g1) / (4 * c0.n_sets), 5)
                launches += 5 * c0.n_sets
                del graph
            except Exception as exc:  # noqa: BLE001
                graph_ms["with_pdl" if pdl else "plain"] = repr(exc)
        for a0 in c0.args:
            a0.use_pdl = 0
        s = c0.sets[0]
        A0, SFA0, B0, SFB0 = slab_of(c0, s, 1024)
        Cb = s["C"].view(torch.int16).cpu().numpy().view(np.uint16)
        lib.bsg_gemm_run(C.byref(c0.args[0]), ws.data_ptr(), 16, stream.cuda_stream)
        torch.cuda.synchronize()
        want0, secs0, kn0 = cpu_gemm_slab(0, A0, SFA0, B0, SFB0, 1024, 1024, 1, Cb, 1.0, 0.5)
        record("c0_nvfp4_1024", 0, c0.flops(), ms0, {
            "workload": "NVFP4 GEMM M=N=K=1024, alpha=1, beta=0.5, bf16 C and D", "operand_sets_rotated": c0.n_sets,
            "cpu_baseline": cpu_baseline_entry(1024, 1024, 1024, secs0, kn0, "the whole problem"),
            "parity_max_rel_err": bf16_rel_err(s["D"].view(torch.int16).cpu().numpy().view(np.uint16), want0),
            "ms_per_call_replayed_from_a_cuda_graph": graph_ms,
            "note": "16 output tiles on 148 SMs: the time is launch latency plus one tile, not throughput"})
        del c0, s
        torch.cuda.empty_cache()

        # c1: MXFP8 8192^3
        c1 = DenseCase(1, 8192, 8192, 8192, dev, gen)
        ms1 = run_case(lib, L, c1, ws, stream, side_steps, 3)
        launches += side_steps
        rows1 = 1024
        lib.bsg_gemm_run(C.byref(c1.args[0]), ws.data_ptr(), 16, stream.cuda_stream)
        torch.cuda.synchronize()
        A1, SFA1, B1, SFB1 = slab_of(c1, c1.sets[0], rows1)
        want1, secs1, kn1 = cpu_gemm_slab(1, A1, SFA1, B1, SFB1, 8192, 8192)
        record("c1_mxfp8_8192", 1, c1.flops(), ms1, {
            "workload": "MXFP8 GEMM M=N=K=8192, alpha=1, beta=0, bf16 D", "operand_sets_rotated": c1.n_sets,
            "cpu_baseline": cpu_baseline_entry(rows1, 8192, 8192, secs1, kn1, f"rows 0..{rows1 - 1} of M"),
            "parity_max_rel_err": bf16_rel_err(c1.sets[0]["D"][:rows1].view(torch.int16).cpu().numpy().view(np.uint16), want1),
            "parity_tolerance": 1e-2})
        del c1
        torch.cuda.empty_cache()

        # c2: NVFP4 8192 x 14336 x 4096, bf16 output and fused NVFP4 output (values + interleaved scale factors)
        M2, N2, K2 = 8192, 14336, 4096
        c2b = DenseCase(0, M2, N2, K2, dev, gen)
        ms2b = run_case(lib, L, c2b, ws, stream, side_steps, 3)
        launches += side_steps
        lib.bsg_gemm_run(C.byref(c2b.args[0]), ws.data_ptr(), 16, stream.cuda_stream)
        torch.cuda.synchronize()
        amax = float(c2b.sets[0]["D"].float().abs().max())
        st = np.float32(448.0 * 6.0 / amax)
        keep = c2b.sets[0]
        c2q = DenseCase(0, M2, N2, K2, dev, gen, out="nvfp4")
        for k in ("A", "SFA", "B", "SFB"):          # set 0 of the quantised case takes the operands whose amax is known
            c2q.sets[0][k] = keep[k]
        c2q.args[0].A, c2q.args[0].SFA, c2q.args[0].B, c2q.args[0].SFB = (keep[k].data_ptr() for k in ("A", "SFA", "B", "SFB"))
        norm = torch.tensor([st], dtype=torch.float32, device=dev)
        c2q.set_norm(norm)
        ms2q = run_case(lib, L, c2q, ws, stream, side_steps, 3)
        launches += side_steps
        rows2 = 512
        lib.bsg_gemm_run(C.byref(c2q.args[0]), ws.data_ptr(), 16, stream.cuda_stream)
        torch.cuda.synchronize()
        A2, SFA2, B2, SFB2 = slab_of(c2q, c2q.sets[0], rows2)
        (Dw, SFDw), secs2, kn2 = cpu_gemm_slab(0, A2, SFA2, B2, SFB2, N2, K2, 2, None, 1.0, 0.0, float(st))
        n_at = F.sf_k_atoms(N2, 16)
        r_idx, kb_idx = np.meshgrid(np.arange(rows2), np.arange(N2 // 16), indexing="ij")
        idx = F.sf_offset(r_idx, kb_idx, n_at).ravel()
        got_sfd = c2q.sets[0]["SFD"][: (rows2 // 128) * 512 * n_at].cpu().numpy()
        record("c2_nvfp4_mlp_up_fused_requant", 0, c2q.flops(), ms2q, {
            "workload": "NVFP4 GEMM M=8192 N=14336 K=4096, output re-quantised in the epilogue: e2m1 D + ue4m3 scale factors per 16, norm = 448*6/amax",
            "bf16_output_same_shape": {"ms": round(ms2b, 5), "tflops": round(c2b.flops() / ms2b / 1e9, 1)},
            "fused_over_bf16_time": round(ms2q / ms2b, 4), "operand_sets_rotated": c2q.n_sets,
            "cpu_baseline": cpu_baseline_entry(rows2, N2, K2, secs2, kn2, f"rows 0..{rows2 - 1} of M, with the quantising epilogue"),
            "parity": {"values_bit_exact": bool(np.array_equal(c2q.sets[0]["D"][:rows2].cpu().numpy(), Dw)),
                       "scale_factors_bit_exact": bool(np.array_equal(got_sfd[idx], SFDw[idx])), "slab_rows": rows2}})
        del c2b, c2q, keep
        torch.cuda.empty_cache()

        # c3: grouped NVFP4 GEMM, 64 experts, ragged M_g (seeded Dirichlet / multinomial), sum 131072
        E, K3, N3, tokens, topk = 64, 7168, 2048, 16384, 8
        sizes = G.moe_group_sizes(E, tokens, topk, np.random.default_rng(0))
        total = int(sizes.sum())
        A3, _ = gpu_nvfp4_operand(total, K3, gen, dev)
        katoms = K3 // 64
        atoms = [-(-int(m) // 128) for m in sizes]
        lut = torch.tensor([0x28, 0x30, 0x38, 0x40, 0x48], dtype=torch.uint8, device=dev)
        SFA3 = lut[torch.randint(0, 5, (sum(atoms) * 512 * katoms,), device=dev, generator=gen)]
        B3, SFB3 = gpu_nvfp4_operand(E * N3, K3, gen, dev)
        D3 = [torch.empty((total, N3), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        offs = torch.tensor(np.cumsum(sizes), dtype=torch.int32, device=dev)
        gargs = []
        for d in D3:
            g = L.GroupedArgs()
            g.kind, g.num_groups, g.total_M, g.N, g.K = 0, E, total, N3, K3
            g.A, g.B, g.SFA, g.SFB, g.D, g.offsets = (x.data_ptr() for x in (A3, B3, SFA3, SFB3, d, offs))
            g.alpha = 1.0
            gargs.append(g)

        def launch3(i):
            rc = lib.bsg_grouped_run(C.byref(gargs[i % 2]), ws.data_ptr(), 16, stream.cuda_stream)
            if rc != 0:
                raise RuntimeError(L.last_error())
        ms3 = time_steps(launch3, max(3, side_steps // 2), 2, stream)
        launches += max(3, side_steps // 2)
        L.check(lib.bsg_read_device_status(ws.data_ptr(), stream.cuda_stream))
        e_big = int(np.argmax(sizes))
        r0 = int(np.concatenate([[0], np.cumsum(sizes)[:-1]])[e_big])
        a0 = int(np.concatenate([[0], np.cumsum(atoms)[:-1]])[e_big])
        rows3 = min(512, int(sizes[e_big]) // 128 * 128)
        nat = N3 // 128
        want3, secs3, kn3 = cpu_gemm_slab(0, A3[r0:r0 + rows3].cpu().numpy(), SFA3[a0 * 512 * katoms:(a0 + rows3 // 128) * 512 * katoms].cpu().numpy(),
                                          B3[e_big * N3:(e_big + 1) * N3].cpu().numpy(),
                                          SFB3[e_big * nat * 512 * katoms:(e_big + 1) * nat * 512 * katoms].cpu().numpy(), N3, K3)
        # the same 64 problems through the pointer-array form (per-group tensors: views of the same buffers)
        ptr_form = None
        try:
            from cutlass_b200.ptr_array import GroupProblem, PtrArrayGemm
            row0s = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int64)
            atom0s = np.concatenate([[0], np.cumsum(atoms)[:-1]]).astype(np.int64)
            sfb_g = (N3 // 128) * 512 * katoms
            pa_ops = []
            for d in D3:
                groups = [GroupProblem(A=A3[int(row0s[e]):int(row0s[e]) + int(sizes[e])],
                                       SFA=SFA3[int(atom0s[e]) * 512 * katoms:],
                                       B=B3[e * N3:(e + 1) * N3], SFB=SFB3[e * sfb_g:(e + 1) * sfb_g],
                                       D=d[int(row0s[e]):int(row0s[e]) + int(sizes[e])]) for e in range(E)]
                pa_ops.append(PtrArrayGemm(0, groups, stream=stream))
            ms3p = time_steps(lambda i: pa_ops[i % 2].run(stream=stream), max(3, side_steps // 2), 2, stream)
            launches += max(3, side_steps // 2)
            for o in pa_ops:
                o.check_device_status(stream)
            same = bool(torch.equal(D3[0].view(torch.int16), D3[1].view(torch.int16)))
            ptr_form = {"ms": round(ms3p, 5), "tflops": round(2.0 * total * N3 * K3 / ms3p / 1e9, 1),
                        "what": "bsg_ptr_array_run: one problem per expert with its own pointers, extents and tensor maps",
                        "output_equals_contiguous_form": same}
            del pa_ops
        except Exception as exc:  # noqa: BLE001
            ptr_form = {"error": repr(exc)}
        record("c3_grouped_moe_64_experts", 0, 2.0 * total * N3 * K3, ms3, {
            "pointer_array_form": ptr_form,
            "workload": "grouped NVFP4 GEMM, 64 experts, K=7168 -> N=2048, ragged M_g from a seeded Dirichlet(1) / multinomial draw, sum M_g = 131072, bf16 D",
            "group_rows_min_max": [int(sizes.min()), int(sizes.max())],
            "l2": "A 470 MB + B 470 MB + D 537 MB per launch: larger than L2 by itself; two output buffers rotated",
            "cpu_baseline": cpu_baseline_entry(rows3, N3, K3, secs3, kn3, f"the first {rows3} rows of the largest expert"),
            "parity_bit_exact": bool(np.array_equal(D3[(max(3, side_steps // 2) - 1) % 2][r0:r0 + rows3].view(torch.int16).cpu().numpy().view(np.uint16), want3))})
        del A3, SFA3, B3, SFB3, D3
        torch.cuda.empty_cache()
    except Exception as exc:  # noqa: BLE001
        configs["error"] = repr(exc)

    # ---- the quantiser in front of the GEMM on an operand of the same size (HBM-bound; reported beside the headline)
    quant = None
    try:
        xs = [torch.randn((M, K), device=dev, generator=gen).to(torch.bfloat16) for _ in range(3)]   # 3 x 134 MB > L2
        qo = [ops.quantize_blockscaled(x, mode) for x in xs]
        torch.cuda.synchronize()
        q_launch = lambda i, s=stream: ops.quantize_blockscaled(xs[i % 3], mode, out=qo[i % 3].quantized.tensor,  # noqa: E731
                                                                scale_out=qo[i % 3].scale.tensor, stream=s)
        q_ms_loop = time_steps(q_launch, 30, 3, stream)
        # A 30 us kernel launched from Python is bound by the host's launch rate whenever the host is busy: the same 30
        # launches captured once in a CUDA graph give the device time.
        q_ms, q_how = q_ms_loop, "30 launches from the host"
        try:
            graph = torch.cuda.CUDAGraph()
            cap = torch.cuda.Stream()          # a capture needs a stream of its own
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=cap):
                for i in range(30):
                    q_launch(i, cap)
            with torch.cuda.stream(cap):
                graph.replay()
                cap.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(cap)
                for _ in range(3):
                    graph.replay()
                e1.record(cap)
            torch.cuda.synchronize()
            q_ms, q_how = e0.elapsed_time(e1) / 90, "3 replays of a CUDA graph of 30 launches (three operand sets rotated)"
            launches += 120
            del graph
        except Exception as exc:  # noqa: BLE001
            q_how += f" (graph capture failed: {exc!r})"
        q_bytes = M * K * 2 + M * K // 2 + M * K // 16
        hbm = measured_peaks().get("hbm_gbs") or 6650.0
        quant = {"workload": f"bf16 {M}x{K} -> NVFP4 values + interleaved ue4m3 scale factors", "ms": round(q_ms, 4),
                 "achieved_gbs": round(q_bytes / q_ms / 1e6, 1), "peak_gbs": hbm, "frac": round(q_bytes / q_ms / 1e6 / hbm, 4),
                 "algorithmic_bytes": q_bytes, "bound": "hbm", "timed_as": q_how, "ms_launched_from_the_host": round(q_ms_loop, 4)}
        del xs, qo
    except Exception as exc:  # noqa: BLE001
        quant = {"error": str(exc)}

    # ---- the tensor-parallel workload on this one GPU: the base of the 1/2/4/8-GPU scaling series
    tp_base = None
    if not args.no_tp_base:
        torch.cuda.empty_cache()
        for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29533")):
            os.environ.setdefault(k, v)
        import bench_tp as tp_bench
        tp_args = argparse.Namespace(steps=max(3, min(args.steps, 30)), warmup=3)
        r = tp_bench.run(tp_args)
        tp_base = {"metric": r["metric"], "value": r["value"], "unit": r["unit"], "ms_per_step": r["ms_per_step"],
                   "workload": r["config"]["workload"], "parity": r["parity"]}

    peak, peak_src = tensor_peak(0)
    traffic = recorded_traffic("nvfp4_8192")
    return {
        "metric": "nvfp4_gemm_8192_tflops", "value": round(tflops, 1), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3/16), fp32 accumulate, bf16 out",
        "data": "synthetic", "config": headline_config(),
        "kernel_config": {**head_tile, "pct_of_nominal_fp4_peak": round(100.0 * tflops / NOMINAL_FP4_TFLOPS, 1)},
        "e2e": e2e,
        "gpu_launches": args.steps,
        "gpu_launches_whole_run": launches,
        "clocks": clk.summary(),
        "roofline": {"bound": "tensor", "achieved": round(tflops, 1), "peak": round(peak, 1), "unit": "TFLOP/s",
                     "frac": round(tflops / peak, 4), "peak_source": peak_src + "; burst figure, the timed region is milliseconds long",
                     "frac_of_nominal_9000": round(tflops / NOMINAL_FP4_TFLOPS, 4),
                     "traffic": traffic.get("traffic_bytes"), "traffic_commit": traffic.get("commit"),
                     "traffic_source": traffic.get("source"), "algorithmic_bytes": algorithmic_bytes},
        "with_pdl": {"ms_per_step": round(pdl_ms, 5), "value": round(flops / pdl_ms / 1e9, 1),
                     "what": "the same launches with use_pdl = 1 (programmatic dependent launch)"},
        "sustained": sustained,
        "cpu_baseline": cpu,
        "parity": {"slab_rows": slab, "max_rel_err_vs_cpu_reference": rel},
        "configs": configs,
        "scaling_base": tp_base,
        "quantiser": quant,
    }


# --------------------------------------------------------------------------- reference arm
def run_reference(args) -> dict:
    """The reference's host GEMM on this machine's CPU cores, same configuration, a bounded row slab per step."""
    import oracle
    from cutlass_b200 import generators as G
    world = args.gpus
    tp = world > 1
    kind = 1 if tp else 0
    M, N, K = (16384, 28672, 8192) if tp else (8192, 8192, 8192)
    rng = np.random.default_rng(0)
    # a step = one slab of rows; sized so that steps + warmup slabs stay within a few minutes at ~0.1 TFLOP/s
    total_slabs = max(1, args.steps + args.warmup)
    budget_s = 120.0
    slab = args.cpu_rows
    est = 2.0 * slab * N * K / 0.09e12
    while slab > 128 and est * total_slabs > budget_s:
        slab //= 2
        est = 2.0 * slab * N * K / 0.09e12
    # tensor parallel: the columns of one rank's shard stand for all N (the CPU rate does not depend on which columns)
    n_cols = N // world if tp else N
    if tp:
        import torch
        from cutlass_b200 import formats as F
        tg = torch.Generator()
        tg.manual_seed(0)

        def gen_op(rows, K_, _rng):     # N(0,1) -> e4m3 (round to nearest, saturating) by torch's CPU cast: fast enough for 10^8 elements
            codes = torch.randn((rows, K_), generator=tg).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
            sf = _rng.integers(124, 131, size=(rows, K_ // 32), dtype=np.uint8)
            return codes, sf, F.swizzle_sf(sf)
    else:
        gen_op = G.nvfp4_operand
    A, _, SFA = gen_op(slab, K, rng)
    B, _, SFB = gen_op(n_cols, K, rng)
    for _ in range(args.warmup):
        cpu_gemm_slab(kind, A, SFA, B, SFB, n_cols, K)
    times, kname = [], "port"
    for _ in range(max(1, args.steps)):
        _, secs, kname = cpu_gemm_slab(kind, A, SFA, B, SFB, n_cols, K)
        times.append(secs)
    mean_s = sum(times) / len(times)
    tflops = 2.0 * slab * n_cols * K / mean_s / 1e12
    cores = oracle.load_oracle().bsg_oracle_threads()
    sample = (f"each step = rows 0..{slab - 1} of M against {'the N=' + str(n_cols) + ' columns of one rank' if tp else 'all N=' + str(n_cols) + ' columns'}, "
              f"K={K}; {mean_s:.2f} s per step on {cores} threads")
    out = {
        "impl": "reference", "metric": "tp_mxfp8_gemm_tflops" if tp else "nvfp4_gemm_8192_tflops", "value": round(tflops, 5), "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": max(1, args.steps), "warmup": args.warmup, "ms_per_step": round(mean_s * 1e3, 2),
        "ms_per_step_is": "the measured time of one slab step",
        "whole_problem_ms_extrapolated": round(2.0 * M * N * K / (tflops * 1e12) * 1e3, 1),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": ("mxfp8 (e4m3 x ue8m0/32)" if tp else "nvfp4 (e2m1 x ue4m3/16)") + ", fp32 accumulate, bf16 out",
        "data": "synthetic", "config": tp_config(world) if tp else headline_config(),
        "cpu_baseline": {"value": round(tflops, 5), "unit": "TFLOP/s", "cores": cores, "kind": kname, "sample": sample},
        "e2e": {"value": round(tflops, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if not args.no_reference_gpu and not tp:
        # The reference's own GPU kernel on the same shape, where it has been built (baseline/; single-GPU runs only:
        # that directory does not travel with multi-GPU runs).
        try:
            from baseline import ref_gpu_bench
            g = ref_gpu_bench.time_kernel("nvfp4", 0, M, N, K, 20)
        except ImportError:
            g = None
        if g is not None:
            out["reference_gpu_kernel"] = g
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=2048, help="rows of M in the CPU baseline sample")
    ap.add_argument("--no-tp-base", action="store_true", help="skip the 1-GPU run of the tensor-parallel workload")
    ap.add_argument("--no-sustained", action="store_true", help="skip the one-second sustained loop of the headline kernel")
    ap.add_argument("--no-reference-gpu", action="store_true", help="reference arm: do not time the reference's own GPU kernel")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        if rank == 0:
            # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every core it may run on.
            import oracle
            oracle.set_threads(len(os.sched_getaffinity(0)))
            if args.steps > 20:
                args.steps = 20       # a CPU step is seconds long: the default K of the GPU arm would take an hour
            if args.warmup > 5:
                args.warmup = 5
            print(json.dumps(run_reference(args)))
        return
    if args.gpus == 1:
        print(json.dumps(run_single(args)))
        return
    import bench_tp as tp_bench
    out = tp_bench.run(args)
    if rank == 0:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
