"""Tensor-parallel block-scaled GEMM: A row-sharded and all-gathered inside the kernel,
B and D sharded over N.  One process per GPU (``torch.distributed`` for the bootstrap only).

Plays the role of the reference's distributed all-gather GEMM
(``include/cutlass/experimental/distributed/schedules/dist_gemm_1d_schedules.hpp``,
``AllGather1D_TilingCD_RotatingA``; host orchestration in
``examples/python/CuTeDSL/cute/blackwell/kernel/distributed/distributed_all_gather_gemm_blackwell.py:2166-2273``).
There the copy engine moves the peer shards and per-stage GEMM launches are gated by flags; here a
single kernel per rank does both: one warp per CTA pushes this rank's rows into every peer's buffer
over NVLink (bulk copies staged through shared memory) and bumps per-row-block arrival counters in the
peer's memory; the tensor-core warps start on the local rows and follow the arrival order.  Two
gathered buffers are used by alternate calls, so a peer may already send the next call's rows.

The planning helpers at the top are pure Python (they restate the kernel's schedule) and are
what the CPU multi-process tests exercise.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

ROW_BLOCK = 256          # rows per readiness flag = rows of one MMA tile (two CTAs x 128)
MAX_WORLD = 8


def shard_rows(M: int, world: int, rank: int) -> tuple[int, int]:
    """Row range [begin, end) of A that ``rank`` owns."""
    if M % (world * ROW_BLOCK) != 0:
        raise ValueError(f"M={M} must be a multiple of {ROW_BLOCK} * world ({world})")
    ms = M // world
    return rank * ms, (rank + 1) * ms


def shard_cols(N: int, world: int, rank: int) -> tuple[int, int]:
    """Column range [begin, end) of B / D that ``rank`` owns."""
    if N % (world * 8) != 0:
        raise ValueError(f"N={N} must be a multiple of 8 * world ({world})")
    ns = N // world
    return rank * ns, (rank + 1) * ns


def choose_ksplit(k_atoms: int) -> int:
    """Pieces a 256-row block is cut into (each piece is one flag increment): A by rows
    (256 / ksplit each), SFA by k-atoms (k_atoms / ksplit each)."""
    ks = 32
    while ks > 1 and k_atoms % ks != 0:
        ks //= 2
    return ks


def consumption_order(world: int, rank: int) -> list[int]:
    """Shards in the order the GEMM of ``rank`` consumes them: its own first, then rank+1, ..."""
    return [(rank + j) % world for j in range(world)]


def push_order(world: int, rank: int) -> list[int]:
    """Peers in the order ``rank`` pushes its shard to them: rank-1 needs it first, then rank-2, ..."""
    return [(rank - j) % world for j in range(1, world)]


@dataclass(frozen=True)
class CopyPiece:
    dst_rank: int
    row_block: int       # global index of the 256-row block (always inside the pushing rank's shard)
    k_piece: int


def copy_schedule(world: int, rank: int, M: int, ksplit: int, cta: int, grid: int) -> list[CopyPiece]:
    """Pieces of its own shard that CTA ``cta`` of ``grid`` pushes, in order (restates the kernel loop)."""
    ms = M // world
    blocks = ms // ROW_BLOCK
    per_shard = blocks * ksplit
    out = []
    for c in range(cta, (world - 1) * per_shard, grid):
        j = c // per_shard + 1
        rem = c - (j - 1) * per_shard
        rb = rem // ksplit
        ks = (rem + rb) % ksplit          # rotated per row block: the piece that carries the scale factors moves around
        out.append(CopyPiece((rank - j) % world, rank * blocks + rb, ks))
    return out


def push_gate_open(mode: str, j: int, rem: int, per_shard: int, stage_now: int, progress: int) -> bool:
    """May a CTA send a piece for its j-th nearest consumer (piece ``rem`` of the shard's ``per_shard``)?  Restates the
    kernel's gates.  ``stage_now``: stage of the tile the CTA's producer is on (published BEFORE it waits for that
    tile's rows; a large number once the CTA has no tiles left); ``progress``: how far the CTA is through its own
    tiles, in 1/1024 of a stage.  "eager": always; "paced": from stage j - 1 on; "spread": piece by piece over the first
    three quarters of stage j - 1, a CTA that is already at a later stage counting as that far."""
    if mode == "eager":
        return True
    if mode == "paced":
        return stage_now >= j - 1
    if mode == "spread":
        need = (j - 1) * 1024 + 768 * rem // per_shard
        return max(progress, min(stage_now, 1 << 10) * 1024) >= need
    raise ValueError(mode)


def simulate_gather(world: int, blocks_per_shard: int, tiles_n: int, clusters: int, ksplit: int, mode: str,
                    gate=push_gate_open, flush_at_closed_gate: bool = True) -> bool:
    """Event-free model of one tensor-parallel call on every rank: clusters walk their tiles (tile t of the walk belongs
    to stage t // (blocks_per_shard * tiles_n) and needs one 256-row block of the shard consumed at that stage), CTAs
    push the pieces ``copy_schedule`` deals them, in order, as their gates open; a tile completes once its block has
    been ANNOUNCED complete.  As in the kernel, a piece is announced only when the CTA has moved on to its next piece
    (the announcement trails the stores), at the end of the CTA's list, or -- ``flush_at_closed_gate`` -- when the CTA
    finds its next gate closed.  Returns True when every tile of every rank completes, False when the ranks end up
    waiting for one another."""
    per_stage = blocks_per_shard * tiles_n
    total = world * per_stage
    clusters = min(clusters, total)
    grid = 2 * clusters
    M = world * blocks_per_shard * ROW_BLOCK
    pieces = [[copy_schedule(world, r, M, ksplit, c, grid) for c in range(grid)] for r in range(world)]
    sent = [[0] * grid for _ in range(world)]                       # pieces already stored, per CTA
    announced = [[0] * grid for _ in range(world)]                  # ... and announced
    arrived = [dict() for _ in range(world)]                        # rank -> {global row block: pieces announced}
    pos = [[0] * clusters for _ in range(world)]                    # tiles completed, per cluster
    own = [len(range(c, total, clusters)) for c in range(clusters)]

    def tile_block(rank: int, t: int) -> tuple[int, int]:
        """(stage, global row block) of walk position t: bands of the walk are stages, blocks cycle inside a band."""
        stage, rem = divmod(t, per_stage)
        shard = (rank + stage) % world
        return stage, shard * blocks_per_shard + rem % blocks_per_shard

    def announce_up_to(r: int, cta: int, n: int) -> bool:
        did = False
        while announced[r][cta] < n:
            pc = pieces[r][cta][announced[r][cta]]
            arrived[pc.dst_rank][pc.row_block] = arrived[pc.dst_rank].get(pc.row_block, 0) + 1
            announced[r][cta] += 1
            did = True
        return did

    changed = True
    while changed:
        changed = False
        for r in range(world):
            for c in range(clusters):
                if pos[r][c] < own[c]:
                    stage, blk = tile_block(r, c + pos[r][c] * clusters)
                    stage_now = stage
                    if stage == 0 or arrived[r].get(blk, 0) >= ksplit:
                        pos[r][c] += 1
                        changed = True
                else:
                    stage_now = 1 << 20
                progress = (1 << 30) if pos[r][c] >= own[c] else 1024 * world * pos[r][c] // own[c]
                for cta in (2 * c, 2 * c + 1):
                    mine = pieces[r][cta]
                    while sent[r][cta] < len(mine):
                        pc = mine[sent[r][cta]]
                        j = (r - pc.dst_rank) % world
                        rem = (pc.row_block - r * blocks_per_shard) * ksplit + pc.k_piece
                        if not gate(mode, j, rem, blocks_per_shard * ksplit, stage_now, progress):
                            if flush_at_closed_gate:
                                changed |= announce_up_to(r, cta, sent[r][cta])
                            break
                        changed |= announce_up_to(r, cta, sent[r][cta])       # the piece before this one
                        sent[r][cta] += 1
                        changed = True
                    if sent[r][cta] == len(mine):
                        changed |= announce_up_to(r, cta, len(mine))
    return all(pos[r][c] >= own[c] for r in range(world) for c in range(clusters))


def exchange_handles(handle: bytes, group=None) -> list[bytes]:
    """All-gather one opaque per-rank blob (the CUDA IPC handle) over ``torch.distributed``."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    out: list = [None] * world
    dist.all_gather_object(out, handle, group=group)
    return out


class _DevicePointer:
    """Exposes raw device memory through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def rs_hop_order(world: int, slice_index: int) -> list[int]:
    """Ranks in the order in which they add their partial product to the running sum of a slice of rows in the
    GEMM + reduce-scatter: the slice starts at rank slice - 1, moves left one rank per stage and ends at its owner."""
    return [(slice_index - 1 - s) % world for s in range(world)]


def rs_stage_slices(world: int, rank: int) -> list[int]:
    """Slices in the order in which ``rank`` works on them (stage 0 first); the last one is its own."""
    return [(rank + 1 + s) % world for s in range(world)]


class RsGemm:
    """Per-rank handle of the GEMM + reduce-scatter for a fixed (M, N): every rank holds the K shard of A (M x K/world)
    and of B (N x K/world); ``run`` leaves rows [rank * M / world, (rank + 1) * M / world) of alpha * A @ B^T in ``out``.
    Takes the role of the reference's reduce-scatter distributed GEMM schedules
    (``include/cutlass/experimental/distributed/schedules/dist_gemm_1d_schedules.hpp:148``)."""

    def __init__(self, M: int, N: int, group=None, all_reduce: bool = False):
        import torch
        import torch.distributed as dist
        from . import lib as L
        self._L = L
        self._lib = L.load()
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > MAX_WORLD:
            raise ValueError(f"at most {MAX_WORLD} ranks are supported")
        shard_rows(M, self.world, self.rank)      # raises when M does not split into whole 256-row blocks per rank
        self.M, self.N = M, N
        self._comm = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        self.all_reduce = all_reduce
        L.check(self._lib.bsg_rs_create(self.rank, self.world, M, N, L.RS_WITH_ALLREDUCE if all_reduce else 0, C.byref(self._comm), handle))
        if self.world > 1:
            handles = exchange_handles(bytes(handle), group)
            blob = (C.c_uint8 * (64 * self.world)).from_buffer_copy(b"".join(handles))
            L.check(self._lib.bsg_rs_connect(self._comm, blob))
            dist.barrier(group)
        self.workspace = torch.zeros(16, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))

    def build_args(self, kind: int, A, SFA, B, SFB, out, alpha: float = 1.0):
        """A: (M, K_local) packed K-major; B: (N, K_local); out: (M / world, N) bf16."""
        L = self._L
        a = L.GemmArgs()
        a.kind, a.out_kind, a.batch = kind, L.OUT_BF16, 1
        k_local = A.shape[-1] * (2 if kind == L.KIND_NVFP4 else 1)
        a.M, a.N, a.K = self.M, self.N, k_local
        a.A, a.SFA, a.B, a.SFB = A.data_ptr(), SFA.data_ptr(), B.data_ptr(), SFB.data_ptr()
        a.D = out.data_ptr() if out is not None else None
        a.alpha = alpha
        return a

    def run(self, kind: int, A, SFA, B, SFB, out, alpha: float = 1.0, stream=None, abi_args=None) -> None:
        from .operator import to_cuda_stream
        a = abi_args if abi_args is not None else self.build_args(kind, A, SFA, B, SFB, out, alpha)
        self._L.check(self._lib.bsg_rs_gemm_run(self._comm, C.byref(a), self.workspace.data_ptr(), 16, to_cuda_stream(stream)))

    def run_all_reduce(self, kind: int, A, SFA, B, SFB, alpha: float = 1.0, stream=None):
        """GEMM + all-reduce (``all_reduce=True`` at construction): every rank gets all of alpha * A @ B^T.  Returns a
        bf16 (M, N) view of the communicator's output for this call, valid until the call after the next one."""
        import torch
        from .operator import to_cuda_stream
        a = self.build_args(kind, A, SFA, B, SFB, None, alpha)
        res = C.c_void_p()
        self._L.check(self._lib.bsg_rs_allreduce_run(self._comm, C.byref(a), self.workspace.data_ptr(), 16, to_cuda_stream(stream), C.byref(res)))
        dev = torch.device("cuda", torch.cuda.current_device())
        return torch.as_tensor(_DevicePointer(res.value, self.M * self.N * 2), device=dev).view(torch.bfloat16).view(self.M, self.N)

    def check_device_status(self, stream=None) -> None:
        from .operator import to_cuda_stream
        self._L.check(self._lib.bsg_read_device_status(self.workspace.data_ptr(), to_cuda_stream(stream)))

    def close(self) -> None:
        if self._comm:
            self._lib.bsg_rs_destroy(self._comm)
            self._comm = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


class TpGemm:
    """Per-rank handle of the tensor-parallel GEMM for a fixed (kind, M, K).

    ``a_shard`` / ``sfa_shard`` are uint8 views of where this rank's rows of A and their
    interleaved scale factors live; fill them, then call ``run`` on every rank."""

    def __init__(self, kind: int, M: int, K: int, group=None, mode: str | None = None):
        import os
        import torch
        import torch.distributed as dist
        from . import lib as L
        self._L = L
        self._lib = L.load()
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > MAX_WORLD:
            raise ValueError(f"at most {MAX_WORLD} ranks are supported")
        self.kind, self.M, self.K = kind, M, K
        self.row_begin, self.row_end = shard_rows(M, self.world, self.rank)
        self._comm = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        L.check(self._lib.bsg_tp_create(self.rank, self.world, kind, M, K, C.byref(self._comm), handle))
        if self.world > 1:
            handles = exchange_handles(bytes(handle), group)
            blob = (C.c_uint8 * (64 * self.world)).from_buffer_copy(b"".join(handles))
            L.check(self._lib.bsg_tp_connect(self._comm, blob))
            dist.barrier(group)
        # "kernel" | "copy_engine", optionally with "+single" (one gathered buffer instead of two), "+release"
        # (announcements behind release fences), "+paced" / "+spread" (when the rows leave); None: the library's default
        # ("kernel+spread+release"); plain "kernel" pushes everything at the start of the call, with relaxed announcements
        mode = mode or os.environ.get("BSG_TP_MODE")
        if mode is not None:
            self.set_mode(mode)
        self.mode = mode or "kernel+spread+release"   # the library's default
        ptrs = [C.c_void_p() for _ in range(4)]
        L.check(self._lib.bsg_tp_buffers(self._comm, *[C.byref(p) for p in ptrs]))
        row_bytes = K // 2 if kind == L.KIND_NVFP4 else K
        vec = 16 if kind == L.KIND_NVFP4 else 32
        k_atoms = -(-(-(-K // vec)) // 4)
        ms = M // self.world
        dev = torch.device("cuda", torch.cuda.current_device())
        self.a_full = torch.as_tensor(_DevicePointer(ptrs[0].value, M * row_bytes), device=dev).view(M, row_bytes)
        self.sfa_full = torch.as_tensor(_DevicePointer(ptrs[1].value, (M // 128) * 512 * k_atoms), device=dev)
        self.a_shard = torch.as_tensor(_DevicePointer(ptrs[2].value, ms * row_bytes), device=dev).view(ms, row_bytes)
        self.sfa_shard = torch.as_tensor(_DevicePointer(ptrs[3].value, (ms // 128) * 512 * k_atoms), device=dev)
        self.workspace = torch.zeros(16, dtype=torch.uint8, device=dev)

    def set_mode(self, mode: str) -> None:
        """Only between calls, with every rank idle (device synchronised and a barrier passed), and the same on all ranks."""
        base, *opts = mode.split("+")
        code = {"kernel": 0, "copy_engine": 1}[base]
        for opt in opts:
            code |= {"single": 2, "release": 4, "paced": 8, "spread": 16}[opt]   # one gathered buffer; release-fenced announcements; paced / spread push
        self._L.check(self._lib.bsg_tp_set_mode(self._comm, code))
        self.mode = mode

    def build_args(self, B, SFB, out, C_=None, alpha: float = 1.0, beta: float = 0.0, tile_n: int = 0):
        """B: (N_local, K bytes) K-major uint8/e4m3 tensor; SFB its interleaved scales; out: (M, N_local) bf16."""
        L = self._L
        a = L.GemmArgs()
        a.kind, a.out_kind, a.batch = self.kind, L.OUT_BF16, 1
        a.M, a.N, a.K = self.M, out.shape[-1], self.K
        a.B, a.SFB, a.D = B.data_ptr(), SFB.data_ptr(), out.data_ptr()
        a.C = C_.data_ptr() if C_ is not None else None
        a.alpha, a.beta = alpha, beta
        a.tile_n, a.cta_group = tile_n, 2
        return a

    def run(self, B, SFB, out, C_=None, alpha: float = 1.0, beta: float = 0.0, stream=None, abi_args=None) -> None:
        from .operator import to_cuda_stream
        a = abi_args if abi_args is not None else self.build_args(B, SFB, out, C_, alpha, beta)
        self._L.check(self._lib.bsg_tp_gemm_run(self._comm, C.byref(a), self.workspace.data_ptr(), 16, to_cuda_stream(stream)))

    def check_device_status(self, stream=None) -> None:
        from .operator import to_cuda_stream
        self._L.check(self._lib.bsg_read_device_status(self.workspace.data_ptr(), to_cuda_stream(stream)))

    def close(self) -> None:
        if self._comm:
            self.a_full = self.sfa_full = self.a_shard = self.sfa_shard = None
            self._lib.bsg_tp_destroy(self._comm)
            self._comm = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
