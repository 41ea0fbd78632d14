"""Tensor-parallel bookkeeping on the CPU: the ownership rule tiles the model exactly, on every rank count, and two
gloo ranks agree on it."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


@pytest.mark.parametrize("size", [1, 2, 4, 8])
@pytest.mark.parametrize("grid", [148, 147])
def test_shares_tile_the_model(size, grid):
    from qwen3mk import tp

    vocab = 151936
    heads, kvh, rows, words, wo = [], [], [], [], {}
    for rank in range(size):
        s = tp.shard(rank, size, vocab)
        heads += list(s.q_heads); kvh += list(s.kv_heads); rows += list(s.ffn_rows); words += [s.words.start, s.words.stop]
        assert all(h // 2 in s.kv_heads for h in s.q_heads), "a query head's kv head lives on the same rank"
        shares = tp.cta_shares(grid, rank, size)
        local_qkv = sorted(r for d in shares for r in d["qkv_rows"])
        assert local_qkv == list(range(4096 // size)), "every local q/k/v row has exactly one owner"
        assert sorted(r for d in shares for r in d["ffn_rows"]) == list(s.ffn_rows)
        assert max(len(d["qkv_rows"]) for d in shares) <= 28 and max(len(d["ffn_rows"]) for d in shares) <= 21
        for d in shares[:144]:
            assert d["head"] in s.q_heads and len(d["wo_rows"]) <= 116
            wo.setdefault(d["head"], []).extend(d["wo_rows"])
        assert all(d["head"] is None for d in shares[144:])
    assert sorted(heads) == list(range(16)) and sorted(kvh) == list(range(8)) and sorted(rows) == list(range(3072))
    assert words[0] == 0 and words[-1] == vocab and all(words[i] == words[i + 1] for i in range(1, len(words) - 1, 2))
    assert all(sorted(wo[h]) == list(range(1024)) for h in range(16)), "every head's Wo rows are covered once"


def test_bad_arguments():
    from qwen3mk import tp

    with pytest.raises(ValueError):
        tp.shard(0, 3, 151936)
    with pytest.raises(ValueError):
        tp.shard(2, 2, 151936)
    with pytest.raises(ValueError):
        tp.shard(0, 8, 1001)


def _rank_main(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from qwen3mk import tp

    s = tp.shard(dist.get_rank(), dist.get_world_size(), 4096)
    mine = torch.tensor([s.q_heads.start, s.q_heads.stop, s.kv_heads.start, s.ffn_rows.start, s.words.start, s.words.stop])
    got = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(got, mine)
    q.put((rank, [g.tolist() for g in got]))
    dist.destroy_process_group()


def test_two_gloo_ranks_agree_on_the_split():
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0] == res[1] == [[0, 8, 0, 0, 0, 2048], [8, 16, 4, 1536, 2048, 4096]]
