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
    assert TP.choose_ksplit(64) == 32         # MXFP8 K=8192
    assert TP.choose_ksplit(128) == 32        # NVFP4 K=8192
    assert TP.choose_ksplit(1) == 1
    assert TP.choose_ksplit(6) == 2


@pytest.mark.parametrize("world", [2, 4, 8])
def test_push_schedule_delivers_every_piece_once_and_nearest_consumer_first(world):
    M, ksplit, grid = 16384, 32, 148
    blocks = M // world // TP.ROW_BLOCK
    received = {}                                   # (dst, row_block, k_piece) -> count, over all ranks
    for rank in range(world):
        order = TP.push_order(world, rank)
        assert order[0] == (rank - 1) % world and rank not in order and len(set(order)) == world - 1
        for cta in range(grid):
            sched = TP.copy_schedule(world, rank, M, ksplit, cta, grid)
            pos = [order.index(p.dst_rank) for p in sched]
            assert pos == sorted(pos), "a CTA must serve the peers in the order they consume this shard"
            for p in sched:
                assert rank * blocks <= p.row_block < (rank + 1) * blocks
                key = (p.dst_rank, p.row_block, p.k_piece)
                received[key] = received.get(key, 0) + 1
    # every rank ends up with every remote row block, each of its ksplit pieces exactly once
    assert len(received) == world * (world - 1) * blocks * ksplit and set(received.values()) == {1}
    for dst in range(world):
        # the first shard a rank consumes after its own is rank+1's, which rank+1 pushes to it first
        assert TP.consumption_order(world, dst)[1] == (dst + 1) % world
        assert TP.push_order(world, (dst + 1) % world)[0] == dst


@pytest.mark.parametrize("grid", [2, 64, 100, 147])
def test_push_schedule_covers_every_piece_when_fewer_ctas_are_launched(grid):
    """The grid is clamped to the number of clusters that can be resident; the pieces are dealt out by CTA index
    modulo the grid, so any grid size must still deliver every piece exactly once."""
    world, M, ksplit = 4, 8192, 32
    blocks = M // world // TP.ROW_BLOCK
    seen = {}
    for cta in range(grid):
        for p in TP.copy_schedule(world, 1, M, ksplit, cta, grid):
            key = (p.dst_rank, p.row_block, p.k_piece)
            seen[key] = seen.get(key, 0) + 1
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


@pytest.mark.parametrize("grid", [128, 148])
def test_scale_factor_pieces_are_spread_over_the_ctas(grid):
    """The piece of a row block that also carries its scale factors (k_piece 0) is twice as large; the rotation of
    k_piece from block to block must keep such pieces from piling up on one CTA, whatever the grid size."""
    world, M, ksplit = 2, 16384, 32
    per_cta = [sum(1 for p in TP.copy_schedule(world, 0, M, ksplit, cta, grid) if p.k_piece == 0) for cta in range(grid)]
    blocks = M // world // TP.ROW_BLOCK
    assert sum(per_cta) == (world - 1) * blocks
    assert max(per_cta) <= 2


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_reduce_scatter_ring_schedule(world):
    """GEMM + reduce-scatter: at every stage the slice a rank works on is the one its right neighbour worked on one
    stage earlier (so the running sum it needs has been sent to it), every slice visits every rank once, and it ends
    at its owner."""
    for rank in range(world):
        mine = TP.rs_stage_slices(world, rank)
        assert sorted(mine) == list(range(world)) and mine[-1] == rank
        right = TP.rs_stage_slices(world, (rank + 1) % world)
        for s in range(1, world):
            assert mine[s] == right[s - 1]
    for j in range(world):
        order = TP.rs_hop_order(world, j)
        assert sorted(order) == list(range(world)) and order[-1] == j
        for s, r in enumerate(order):
            assert TP.rs_stage_slices(world, r)[s] == j


@pytest.mark.parametrize("mode", ["eager", "paced", "spread"])
@pytest.mark.parametrize("world,blocks,tiles_n,clusters", [(2, 8, 2, 74), (4, 4, 4, 74), (4, 4, 1, 74), (8, 8, 14, 74), (8, 1, 2, 74), (4, 2, 1, 3),
                                                           (8, 1, 1, 8)])
def test_push_gates_never_leave_the_ranks_waiting_for_one_another(mode, world, blocks, tiles_n, clusters):
    """Model of a call on every rank (clusters walking their tiles, CTAs pushing their pieces as the gates open): every
    tile completes, for the benchmark shape, for shapes with one tile per cluster and for grids smaller than the work."""
    for ksplit in (4, 32):
        assert TP.simulate_gather(world, blocks, tiles_n, clusters, ksplit, mode)


def test_spreading_by_own_pace_alone_would_deadlock_small_problems():
    """Why the spread gate also counts the stage a CTA is at: with one tile per cluster a CTA may start at a late stage
    and stand still there, and a gate that looked only at its pace would hold back the rows the others wait for."""
    def pace_only(mode, j, rem, per_shard, stage_now, progress):
        return progress >= (j - 1) * 1024 + 768 * rem // per_shard
    # 32 tiles on 32 clusters, 256 pieces over their 64 CTAs: the shape of the 2-rank NVFP4 test (M 4096, N 1024, K 4096)
    assert not TP.simulate_gather(2, 8, 2, 74, 32, "spread", gate=pace_only)
    assert TP.simulate_gather(2, 8, 2, 74, 32, "spread")


def test_announcements_must_not_wait_behind_a_closed_gate():
    """A piece is announced only when its CTA moves on to the next piece.  If the CTA then waits at a closed gate with
    the last pieces of the previous destination still unannounced, CTAs of different ranks that stand at the same stage
    wait for one another around the ring (seen on 4 GPUs: M 4096, N 1024, K 2048, spread push): the kernel announces
    what it has stored before it waits at a gate."""
    assert not TP.simulate_gather(4, 4, 1, 74, 16, "spread", flush_at_closed_gate=False)
    assert TP.simulate_gather(4, 4, 1, 74, 16, "spread")
    for mode in ("paced", "spread"):
        for shape in ((4, 4, 1, 74), (8, 8, 14, 74), (2, 8, 2, 74), (8, 1, 1, 8)):
            assert TP.simulate_gather(*shape, 16, mode)
