"""Tensor-parallel decode on 2 (and 4) GPUs against the CPU oracle.  Needs at least two B200s on one node; skipped
otherwise.  One process per GPU, NCCL only for the hand-shake (NVLS off), the per-layer sums inside the kernel."""
from __future__ import annotations

import os
import socket
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _rank_main(rank, world, port, q, layers, vocab, ctx, steps):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from oracle import qwen3_oracle as O
        from qwen3mk import Megakernel, tp

        shp = O.Shape(layers=layers, vocab=vocab)
        inp = O.synthetic(11, shp, context=ctx)
        w32 = O.to_fp32(inp)
        mk = Megakernel(dev, layers=layers, vocab=vocab, path="persist")
        s = tp.attach(mk)
        devin = {k: v.to(dev) for k, v in inp.items()}
        out = mk.step(devin)
        mk.status()
        ref = O.decode_step(w32, inp["token"], inp["kcache"], inp["vcache"])
        res = {"rank": rank, "token": int(out["next_token"]), "ref_token": int(ref["next_token"])}
        words = slice(s.words.start, s.words.stop)
        res["logits_rel_l2"] = O.rel_l2(out["logits"][words], ref["logits"][words])
        kv = slice(s.kv_heads.start, s.kv_heads.stop)
        res["k_ulps"] = O.bf16_ulps(out["k_write"][:, kv], ref["k_write"][:, kv])
        res["v_ulps"] = O.bf16_ulps(out["v_write"][:, kv], ref["v_write"][:, kv])
        # chained greedy steps with a growing cache
        mk.bind(devin, chained=True, grow=steps)
        toks = []
        for _ in range(steps):
            mk.launch()
            toks.append(mk.chain_token.clone())
        mk.status()
        g = O.greedy_decode(w32, inp["token"], inp["kcache"], inp["vcache"], steps)
        res["tokens"], res["ref_tokens"] = torch.stack(toks).cpu().tolist(), g["tokens"].tolist()
        res["margins"] = [float(m) for m in g["margins"]]
        # a step after detaching is a plain single-GPU step again
        dist.barrier()
        tp.detach(mk)
        out1 = mk.step(devin)
        mk.status()
        res["single_token"] = int(out1["next_token"])
        res["single_rel_l2"] = O.rel_l2(out1["logits"], ref["logits"])
        q.put(res)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        q.put({"rank": rank, "error": traceback.format_exc()})


@pytest.mark.parametrize("world,layers,vocab,ctx", [(2, 2, 4096, 40), (2, 3, 4096, 200), (4, 2, 4096, 77), (2, 28, 151936, 128)])
def test_tensor_parallel_step_matches_the_oracle(world, layers, vocab, ctx):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    steps = 16
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    port = _free_port()
    procs = [ctxm.Process(target=_rank_main, args=(r, world, port, q, layers, vocab, ctx, steps)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
    for r in results:
        assert "error" not in r, r["error"]
    for r in results:
        assert r["token"] == r["ref_token"], r
        assert r["logits_rel_l2"] <= 1e-4 and r["k_ulps"] <= 2 and r["v_ulps"] <= 2, r
        if r["tokens"] != r["ref_tokens"]:
            i = next(k for k in range(steps) if r["tokens"][k] != r["ref_tokens"][k])
            assert r["margins"][i] < 1e-4, (i, r["tokens"][i], r["ref_tokens"][i], r["margins"][i])
        assert r["single_token"] == r["ref_token"] and r["single_rel_l2"] <= 1e-4
    assert len({tuple(r["tokens"]) for r in results}) == 1, "every rank decodes the same stream"
