"""Tensor-parallel GEMM on real GPUs through the C ABI (bsg_tp_*), one process per GPU.

Every call uses a different A, so a rank that read a peer's rows before they had arrived (or rows
of the previous call) cannot pass: the operands are the exact-arithmetic fixtures and the result
must equal the oracle's bit for bit.  NVLS is switched off for the NCCL bootstrap."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem(kind, M, N, K, seed):
    from cutlass_b200 import generators as G
    rng = np.random.default_rng(seed)
    gen = G.exact_nvfp4_operand if kind == 0 else G.exact_mxfp8_operand
    A, _, sfa = gen(M, K, rng)
    B, _, sfb = gen(N, K, rng)
    return A, sfa, B, sfb


def _run_rank(tp, rank, world, kind, M, N, K, calls):
    import oracle
    vec = 16 if kind == 0 else 32
    atom_bytes = 512 * (-(-(K // vec) // 4))
    ms, ns = M // world, N // world
    for call in range(calls):
        A, sfa, B, sfb = _problem(kind, M, N, K, 100 + call)
        tp.a_shard.copy_(torch.from_numpy(A[rank * ms:(rank + 1) * ms]).cuda())
        tp.sfa_shard.copy_(torch.from_numpy(sfa[(rank * ms // 128) * atom_bytes:((rank + 1) * ms // 128) * atom_bytes]).cuda())
        Bl = np.ascontiguousarray(B[rank * ns:(rank + 1) * ns])
        sfbl = np.ascontiguousarray(sfb[(rank * ns // 128) * atom_bytes:((rank + 1) * ns // 128) * atom_bytes])
        dB, dSFB = torch.from_numpy(Bl).cuda(), torch.from_numpy(sfbl).cuda()
        out = torch.full((M, ns), 0x7FC0, dtype=torch.int16, device="cuda")          # NaN pattern: unwritten cells show up
        tp.run(dB, dSFB, out)
        tp.check_device_status()
        torch.cuda.synchronize()
        want = oracle.to_bf16(oracle.gemm_fp32(kind, A, sfa, Bl, sfbl, M, ns, K))
        got = out.cpu().numpy().view(np.uint16)
        bad = int((got != want).sum())
        assert bad == 0, f"call {call}: {bad} of {got.size} outputs differ from the oracle (rank {rank})"


def _worker(rank, world, port, kind, M, N, K, calls, q, mode=None):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist
        from cutlass_b200 import tp as TP
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        tp = TP.TpGemm(kind, M, K, mode=mode)
        try:
            _run_rank(tp, rank, world, kind, M, N, K, calls)
        finally:
            torch.cuda.synchronize()
            dist.barrier()
            tp.close()
            dist.barrier()
            dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))


@pytest.mark.parametrize("kind", [0, 1])
def test_tp_single_rank_matches_oracle(kind):
    """world = 1: the tensor-parallel kernel with every row local (no peers, no push)."""
    from cutlass_b200 import tp as TP
    tp = TP.TpGemm(kind, 512, 1024)
    try:
        _run_rank(tp, 0, 1, kind, 512, 384, 1024, calls=2)
    finally:
        tp.close()


def _spawn(world, kind, M, N, K, calls, mode=None, timeout=600):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, kind, M, N, K, calls, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=timeout) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
    assert results == [(r, "ok") for r in range(world)], results


@pytest.mark.parametrize("kind,world,M,N,K,mode", [(1, 2, 1024, 512, 2048, None), (0, 2, 1024, 512, 2048, None), (1, 2, 4096, 1024, 4096, None),
                                                   (1, 2, 4096, 1024, 4096, "kernel+release"), (1, 2, 2048, 512, 2048, "copy_engine"),
                                                   (1, 2, 4096, 1024, 4096, "kernel"), (0, 2, 4096, 1024, 4096, "kernel+paced"),
                                                   (1, 4, 2048, 1024, 2048, None), (0, 4, 4096, 1024, 4096, "kernel+release"),
                                                   (1, 4, 4096, 1024, 2048, "kernel"), (1, 4, 4096, 1024, 2048, "kernel+paced"), (1, 4, 4096, 1024, 2048, None)])
def test_tp_gathers_a_inside_the_kernel(kind, world, M, N, K, mode):
    """A different A on every call, bit-exact against the oracle; mode None is the library's default (spread push), "kernel"
    the eager push, "kernel+paced" the push paced by stages; also with the announcements behind release fences (the form
    the PTX memory model asks for) and with the copy engines moving the rows."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _spawn(world, kind, M, N, K, 3, mode)


@pytest.mark.parametrize("world", [2, 4])
def test_tp_fifty_small_calls_in_a_row(world):
    """The shape of the 8-rank case below on fewer GPUs: 2048 rows and 128 columns per rank, K 1024, 50 calls with a new A
    each, no barrier between the calls (the ranks drift apart by up to a call)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _spawn(world, 1, 2048 * world, 128 * world, 1024, 50, None, timeout=900)


def test_tp_eight_ranks_fifty_calls_at_the_benchmark_shard_size():
    """Eight ranks with 2048 rows each (the row shard of the 16384-row benchmark problem), 50 calls in a row, every
    one with a different A on every rank and every output element compared with the oracle: a rank that consumed a
    peer's rows before they had arrived, or rows left from two calls earlier in the same gathered buffer, fails."""
    world = 8
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _spawn(world, 1, 16384, 1024, 1024, 50, None, timeout=900)


def _worker_peer_absent(rank, world, port, q):
    """Rank 1 never launches its call: rank 0's kernel must come back by itself with a time-out status."""
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
        import time

        import torch.distributed as dist
        from cutlass_b200 import lib as L
        from cutlass_b200 import tp as TP
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        kind, M, N, K = 1, 1024, 512, 1024
        tp = TP.TpGemm(kind, M, K)
        verdict = "ok"
        try:
            if rank == 0:
                A, sfa, B, sfb = _problem(kind, M, N, K, 7)
                ns = N // world
                tp.a_shard.copy_(torch.from_numpy(A[:M // world]).cuda())
                tp.sfa_shard.copy_(torch.from_numpy(sfa[:tp.sfa_shard.numel()]).cuda())
                dB = torch.from_numpy(np.ascontiguousarray(B[:ns])).cuda()
                dSFB = torch.from_numpy(np.ascontiguousarray(sfb[:(ns // 128) * 512 * (K // 32 // 4)])).cuda()
                out = torch.zeros((M, ns), dtype=torch.int16, device="cuda")
                t0 = time.time()
                tp.run(dB, dSFB, out)
                torch.cuda.synchronize()                      # the bounded waits run out after about two seconds
                took = time.time() - t0
                try:
                    tp.check_device_status()
                    verdict = "no time-out was reported"
                except L.BsgError as exc:
                    if exc.code != 7:                         # BSG_ERR_TIMEOUT
                        verdict = f"unexpected status {exc}"
                if took > 30:
                    verdict = f"the kernel took {took:.1f} s to give up"
                # the context is still usable
                assert int((torch.ones(4, device="cuda") * 2).sum().item()) == 8
        finally:
            torch.cuda.synchronize()
            dist.barrier()                                    # rank 1 waits here, with nothing of its own in flight
            tp.close()
            dist.barrier()
            dist.destroy_process_group()
        q.put((rank, verdict))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))


def test_tp_rank_that_never_launches_gives_a_timeout_status_not_a_hang():
    """Failure detection without a fault: the missing peer is a host-side event (it simply does not call run); the
    surviving rank's device-side waits are bounded and the host reads BSG_ERR_TIMEOUT."""
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_peer_absent, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
    assert results == [(r, "ok") for r in range(world)], results


# --------------------------------------------------------------------------- GEMM + reduce-scatter
def _rs_worker(rank, world, port, kind, M, N, K, calls, q, all_reduce=False):
    """K is sharded; rank r must end up with rows [r * M / world, ...) of the sum over ranks, where the running sum is
    rounded to bf16 at every hop of the ring (the oracle follows the same hop order)."""
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist
        import oracle
        from cutlass_b200 import generators as G
        from cutlass_b200 import tp as TP
        torch.cuda.set_device(rank)
        if world > 1:
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        rs = TP.RsGemm(M, N, all_reduce=all_reduce)
        try:
            ms, kl = M // world, K // world
            for call in range(calls):
                rng = np.random.default_rng(300 + call)
                gen_a, gen_b = G.operand_generators(kind, True)
                shards = [(gen_a(M, kl, rng), gen_b(N, kl, rng)) for _ in range(world)]       # every rank's K shard, same on all ranks
                (A, _, sfa), (B, _, sfb) = shards[rank]
                dA, dSFA, dB, dSFB = (torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in (A, sfa, B, sfb))
                vec = 16 if kind == 0 else 32
                atom_bytes = 512 * (-(-(kl // vec) // 4))

                def slice_oracle(sl):
                    run = None
                    for hop in TP.rs_hop_order(world, sl):
                        (Ah, _, sfah), (Bh, _, sfbh) = shards[hop]
                        rows = slice(sl * ms, (sl + 1) * ms)
                        sfa_rows = sfah[(sl * ms // 128) * atom_bytes:((sl + 1) * ms // 128) * atom_bytes]
                        pre = oracle.gemm_fp32(kind, Ah[rows], sfa_rows, Bh, sfbh, ms, N, kl, run, 0.5, 1.0 if run is not None else 0.0)
                        run = oracle.to_bf16(pre)
                    return run
                if all_reduce:
                    # every rank ends up with every slice; the result lives in the communicator (two buffers, alternating)
                    full = rs.run_all_reduce(kind, dA, dSFA, dB, dSFB, alpha=0.5)
                    rs.check_device_status()
                    torch.cuda.synchronize()
                    got = full.view(torch.int16).cpu().numpy().view(np.uint16)
                    for sl in range(world):
                        bad = int((got[sl * ms:(sl + 1) * ms] != slice_oracle(sl)).sum())
                        assert bad == 0, f"call {call}: {bad} outputs of slice {sl} differ from the oracle (rank {rank})"
                    continue
                out = torch.full((ms, N), 0x7FC0, dtype=torch.int16, device="cuda")
                rs.run(kind, dA, dSFA, dB, dSFB, out, alpha=0.5)
                rs.check_device_status()
                torch.cuda.synchronize()
                run = slice_oracle(rank)
                got = out.cpu().numpy().view(np.uint16)
                bad = int((got != run).sum())
                assert bad == 0, f"call {call}: {bad} of {got.size} outputs differ from the oracle (rank {rank})"
        finally:
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            rs.close()
            if world > 1:
                dist.barrier()
                dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))


@pytest.mark.parametrize("kind,world,M,N,K", [(0, 1, 512, 384, 512), (1, 2, 1024, 512, 1024), (0, 2, 2048, 640, 2048), (1, 4, 2048, 1024, 2048),
                                              (0, 8, 4096, 512, 4096)])
def test_gemm_reduce_scatter(kind, world, M, N, K):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rs_worker, args=(r, world, port, kind, M, N, K, 4, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
    assert results == [(r, "ok") for r in range(world)], results


@pytest.mark.parametrize("kind,world,M,N,K", [(1, 1, 512, 384, 512), (0, 2, 1024, 512, 1024), (1, 2, 2048, 640, 2048), (0, 4, 2048, 1024, 2048),
                                              (1, 8, 4096, 512, 4096)])
def test_gemm_all_reduce(kind, world, M, N, K):
    """GEMM + all-reduce: the reduce-scatter ring, then every finished slice stored into every rank's output by the
    epilogue; every rank compares all M rows with the oracle's ring sums, over several calls (the outputs alternate)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rs_worker, args=(r, world, port, kind, M, N, K, 4, q, True)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
    assert results == [(r, "ok") for r in range(world)], results
