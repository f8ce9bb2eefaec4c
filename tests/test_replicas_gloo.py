"""Replica scale-out logic on CPU with a world-size-2 gloo group."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vui_b200.replicas import aggregate_rate, shard_streams


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = shard_streams(5, rank, world)
    # rank 0 decodes 3 streams x 10 frames in 20 ms, rank 1 decodes 2 x 10 in 40 ms
    rate, ms = aggregate_rate(len(mine) * 10, 20.0 * (rank + 1))
    out.put((rank, mine, rate, ms))
    dist.barrier()
    dist.destroy_process_group()


def test_two_replicas_disjoint_streams_and_max_time():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][1] == [0, 2, 4] and res[1][1] == [1, 3]
    assert not set(res[0][1]) & set(res[1][1])
    for _, _, rate, ms in res:
        assert ms == 40.0                      # max over ranks
        assert abs(rate - 50 / 0.040) < 1e-6   # all frames of the job / slowest rank


def test_single_process_needs_no_group():
    rate, ms = aggregate_rate(100, 50.0)
    assert rate == 2000.0 and ms == 50.0
    assert shard_streams(4, 0, 1) == [0, 1, 2, 3]
