"""Multi-rank host logic on CPU: world_size 2 over gloo."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vmamba_b200 import shard


def test_shard_ranges_cover_batch():
    for gb in (0, 1, 7, 16, 128, 255, 256):
        for world in (1, 2, 3, 4, 8):
            spans = [shard.shard_range(gb, world, r) for r in range(world)]
            assert sum(c for _, c in spans) == gb
            pos = 0
            for s, c in spans:
                assert s == pos
                pos += c
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        shard.shard_range(8, 2, 2)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ms = 10.0 + 5.0 * rank
        start, count = shard.shard_range(129, world, rank)
        slowest = shard.max_over_ranks(ms)
        thr = shard.aggregate_throughput(count, ms)
        q.put((rank, start, count, slowest, thr))
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [(r[1], r[2]) for r in res] == [(0, 65), (65, 64)]
    assert all(abs(r[3] - 15.0) < 1e-9 for r in res)
    assert all(abs(r[4] - 129 / 0.015) < 1e-6 for r in res)


def _worker_with_failure(rank, world, port, q):
    """Rank 1 leaves between steps (before the bookkeeping collective); rank 0 must get a ShardFailure,
    not a hang.  No GPU is involved: the failure is made on the host."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    dist.barrier()                       # step 0 completed by everyone
    if rank == 1:
        os._exit(3)                      # the rank dies without closing the group
    try:
        shard.aggregate_throughput_or_fail(64, 10.0)
        q.put((rank, "no error"))
    except shard.ShardFailure as e:
        q.put((rank, "ShardFailure", str(e)))


def test_lost_rank_is_reported_not_hung():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_with_failure, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=120)
    assert res[0] == 0 and res[1] == "ShardFailure" and "rank 0" in res[2]
    procs[1].join(timeout=60)
    assert procs[1].exitcode == 3
    procs[0].join(timeout=60)
    if procs[0].is_alive():              # the group's destructor may wait for the dead peer: end exactly this child
        procs[0].kill()
        procs[0].join(timeout=30)
