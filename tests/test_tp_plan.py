"""Host-side logic of the tensor-parallel GEMM: shard ranges, copy schedule, and the handle
exchange over torch.distributed, run as two gloo ranks on CPU."""
import os
import socket

import pytest
import torch.multiprocessing as mp

from cutlass_b200 import tp as TP


def test_shard_ranges_cover_the_problem():
    M, N = 16384, 28672
    for world in (1, 2, 4, 8):
        rows = [TP.shard_rows(M, world, r) for r in range(world)]
        cols = [TP.shard_cols(N, world, r) for r in range(world)]
        assert rows[0][0] == 0 and rows[-1][1] == M and all(a[1] == b[0] for a, b in zip(rows, rows[1:]))
        assert cols[0][0] == 0 and cols[-1][1] == N and all(a[1] == b[0] for a, b in zip(cols, cols[1:]))
        assert all((e - b) % TP.ROW_BLOCK == 0 for b, e in rows)
    with pytest.raises(ValueError):
        TP.shard_rows(1000, 8, 0)
    with pytest.raises(ValueError):
        TP.shard_cols(100, 8, 0)


def test_ksplit_choice():
    assert TP.choose_ksplit(8192, 64) == 8        # MXFP8 K=8192
    assert TP.choose_ksplit(4096, 128) == 8       # NVFP4 K=8192
    assert TP.choose_ksplit(48, 1) == 1
    assert TP.choose_ksplit(256, 2) == 2


@pytest.mark.parametrize("world", [2, 4, 8])
def test_copy_schedule_covers_every_remote_piece_once_in_consumption_order(world):
    M, ksplit, grid = 16384, 8, 148
    blocks = M // world // TP.ROW_BLOCK
    for rank in range(world):
        seen = {}
        for cta in range(grid):
            sched = TP.copy_schedule(world, rank, M, ksplit, cta, grid)
            order = TP.consumption_order(world, rank)
            pos = [order.index(p.src_rank) for p in sched]
            assert pos == sorted(pos), "a CTA must copy shards in the order the GEMM consumes them"
            for p in sched:
                assert p.src_rank != rank
                assert p.src_rank * blocks <= p.row_block < (p.src_rank + 1) * blocks
                seen[(p.row_block, p.k_piece)] = seen.get((p.row_block, p.k_piece), 0) + 1
        assert len(seen) == (world - 1) * blocks * ksplit and set(seen.values()) == {1}


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = bytes([rank]) * 64
        got = TP.exchange_handles(mine)
        rows = TP.shard_rows(1024, world, rank)
        q.put((rank, got, rows, TP.consumption_order(world, rank)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_handle_exchange_two_gloo_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, got, rows, order in results:
        assert got == [bytes([0]) * 64, bytes([1]) * 64]          # every rank holds every handle, indexed by rank
        assert rows == (rank * 512, (rank + 1) * 512)
        assert order == [rank, 1 - rank]
