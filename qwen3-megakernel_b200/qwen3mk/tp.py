"""Tensor parallelism over the GPUs of one node: who owns what, and the host-side hand-shake.

The reference is single-GPU (qwen3mk/kernel.py:120-131).  Here 2, 4 or 8 ranks (one process and one engine per GPU)
split one decode step Megatron-style: rank r owns query heads [r 16/T, ..), kv heads [r 8/T, ..), FFN rows [r 3072/T, ..)
and the LM-head words [r V/T, ..); every rank keeps the whole residual stream.  The two sums over ranks per layer happen
inside the persistent kernel (red instructions into every rank's accumulators over NVLink); the host only exchanges the
64-byte IPC handles of the engines' state allocations once (`attach`).  `Shard` states the ownership rule for callers
that have to slice outputs (logits of the rank's words, K/V rows of the rank's kv heads); `cta_shares` mirrors the
kernel's per-CTA split and is what the CPU tests check for gaps and overlaps.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _cabi
from .kernel import HEAD_DIM, HIDDEN, INTER, KV_HEADS, Q_HEADS

SIZES = (1, 2, 4, 8)
F_CTAS = 144


@dataclass(frozen=True)
class Shard:
    rank: int
    size: int
    q_heads: range
    kv_heads: range
    ffn_rows: range
    words: range


def shard(rank: int, size: int, vocab: int) -> Shard:
    if size not in SIZES or not 0 <= rank < size:
        raise ValueError(f"tensor parallelism: rank {rank} of {size} (sizes {SIZES})")
    if vocab % size:
        raise ValueError(f"tensor parallelism: vocabulary {vocab} does not divide over {size} ranks")
    hq, hk, il, vl = Q_HEADS // size, KV_HEADS // size, INTER // size, vocab // size
    return Shard(rank, size, range(rank * hq, (rank + 1) * hq), range(rank * hk, (rank + 1) * hk),
                 range(rank * il, (rank + 1) * il), range(rank * vl, (rank + 1) * vl))


def cta_shares(grid: int, rank: int, size: int) -> list[dict]:
    """What CTA c of `grid` owns on rank `rank` (the rule of the kernel's share_of): rows of the rank's [q; k; v] rows,
    global FFN rows, and for the first 144 CTAs a (query head, slice of Wo's 1024 rows)."""
    ql, il, hl = (Q_HEADS + 2 * KV_HEADS) * HEAD_DIM // size, INTER // size, Q_HEADS // size
    slices = F_CTAS // hl
    out = []
    for c in range(grid):
        q0, q1 = c * ql // grid, (c + 1) * ql // grid
        i0, i1 = rank * il + c * il // grid, rank * il + (c + 1) * il // grid
        d = {"qkv_rows": range(q0, q1), "ffn_rows": range(i0, i1), "head": None, "wo_rows": None}
        if c < F_CTAS:
            fs = c // hl
            d["head"] = rank * hl + c % hl
            d["wo_rows"] = range((fs * 256 // slices) * 4, ((fs + 1) * 256 // slices) * 4)
        out.append(d)
    return out


def attach(mk, group=None) -> Shard:
    """Switch engine `mk` to its share of a tensor-parallel group (default: the whole torch.distributed world): gather the
    engines' IPC handles, map the peers' state, wait until every rank has done so.  Weights handed over afterwards are the
    full tensors; the engine packs the rank's share."""
    import torch.distributed as dist

    rank, size = dist.get_rank(group), dist.get_world_size(group)
    buf = (ctypes.c_ubyte * 64)()
    _cabi.check(mk.lib, mk.handle, mk.lib.q3_tp_export(mk.handle, buf), "q3_tp_export")
    on_gpu = dist.get_backend(group) == "nccl"
    mine = torch.tensor(list(buf), dtype=torch.uint8, device=mk.device if on_gpu else "cpu")
    gathered = [torch.empty_like(mine) for _ in range(size)]
    dist.all_gather(gathered, mine, group=group)
    blob = b"".join(bytes(t.cpu().tolist()) for t in gathered)
    _cabi.check(mk.lib, mk.handle, mk.lib.q3_tp_attach(mk.handle, rank, size, blob), "q3_tp_attach")
    mk._weights_key = None
    mk.tp = shard(rank, size, mk.vocab)
    dist.barrier(group=group)
    return mk.tp


def detach(mk) -> None:
    _cabi.check(mk.lib, mk.handle, mk.lib.q3_tp_attach(mk.handle, 0, 1, None), "q3_tp_attach")
    mk._weights_key = None
    mk.tp = None
