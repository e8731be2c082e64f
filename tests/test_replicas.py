"""Session partitioning over per-GPU replicas, exercised with two CPU ranks over gloo."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pega_omni_b200 import replicas


def test_round_robin_partition_is_a_partition():
    for n in (1, 7, 64, 129):
        for w in (1, 2, 4, 8):
            parts = replicas.partition(n, w)
            assert sorted(x for p in parts for x in p) == list(range(n))
            assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
            for r, p in enumerate(parts):
                assert all(replicas.owner(s, w) == r for s in p)


def _rank(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = replicas.local_sessions(10, rank, world)
    # every rank "decodes" 5 ticks of its own sessions; the timing protocol is barrier, work, max over ranks
    dist.barrier()
    seconds = torch.tensor([0.010 * (rank + 1)], dtype=torch.float64)
    frames = torch.tensor([len(mine) * 5], dtype=torch.float64)
    dist.all_reduce(seconds, op=dist.ReduceOp.MAX)
    dist.all_reduce(frames, op=dist.ReduceOp.SUM)
    dist.barrier()
    q.put((rank, mine, float(frames.item() / seconds.item())))
    dist.destroy_process_group()


def test_two_ranks_partition_and_aggregate():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0][1] == [0, 2, 4, 6, 8] and got[1][1] == [1, 3, 5, 7, 9]
    want = replicas.aggregate_frames_per_second([25, 25], [0.010, 0.020])
    assert got[0][2] == pytest.approx(want) and got[1][2] == pytest.approx(want)
