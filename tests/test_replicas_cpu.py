"""The replica layer's bookkeeping on two gloo ranks (CPU): partitioning, slowest-rank time, aggregate throughput."""
from __future__ import annotations

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG, ROOT


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, size: int, port: int, q):
    for p in (str(ROOT), str(PKG)):
        sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    from qwen3mk import replicas

    mine = replicas.partition(7)
    slow = replicas.max_over_ranks(1.0 + rank)            # rank 1 is the slow one
    agg = replicas.aggregate_throughput(len(mine) * 10.0, 1.0 + rank)
    toks = torch.tensor([100 + i for i in mine], dtype=torch.int64)
    merged = replicas.gather_tokens(toks, mine, 7)
    q.put((rank, mine, slow, agg, merged.tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_replica_bookkeeping():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, m0, s0, a0, t0), (r1, m1, s1, a1, t1) = got
    assert m0 == [0, 2, 4, 6] and m1 == [1, 3, 5]
    assert s0 == s1 == 2.0
    assert a0 == a1 == {"units": 70.0, "seconds": 2.0, "per_second": 35.0}
    assert t0 == t1 == [100, 101, 102, 103, 104, 105, 106]


def test_single_process_defaults():
    from qwen3mk import replicas

    assert replicas.world() == (0, 1)
    assert replicas.partition(5) == [0, 1, 2, 3, 4]
    assert replicas.partition(5, rank=1, size=2) == [1, 3]
    assert replicas.max_over_ranks(3.5) == 3.5
    assert replicas.aggregate_throughput(10, 2)["per_second"] == 5.0
    with pytest.raises(ValueError):
        replicas.partition(5, rank=2, size=2)
