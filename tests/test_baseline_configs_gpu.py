"""Parity on the configurations the benchmark itself names, at full size (28 layers, vocabulary 151936), through
the C ABI against the CPU oracle.  Needs a B200.

  1. benchmark weights (bf16 N(0, 0.02), unit gains), a cache prefilled on the GPU from 128 seeded ids, then 256
     chained greedy steps of the persistent kernel, every step gated on tokens AND logits;
  2. the full-size prefill against the fixture the reference's own prefill produced, and against the oracle;
  3. a 2048-token prompt followed by 128 greedy steps;
  4. batched decode at batch 8 / 32 / 64 with the full vocabulary (tensor-core LM head + row argmax).

Greedy runs are checked teacher-forced: the oracle replays the GPU's own token stream, so a step whose two best
logits are closer than the engine's error can flip a token without un-gating the steps after it.  Such a flip is
allowed only when the oracle's top-2 margin is below twice the largest logit error of that step, and it is printed.
Tolerances: logits rel-L2 <= 1e-4, K/V rows <= 2 bf16 ulps (decode) or 2e-2 relative (prefill, whose cached rows
are rounded to bf16 before later positions attend them)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN, gate_teacher_forced, run_chained

pytestmark = pytest.mark.gpu

GATE_LOGITS_REL_L2 = 1e-4
GATE_KV_ULPS = 2
GATE_MAX_REL = 2e-2


def to_dev(d):
    return {k: v.cuda() for k, v in d.items()}


def engine(**kw):
    from qwen3mk import Megakernel

    try:
        return Megakernel(**kw)
    except RuntimeError as e:
        pytest.fail(f"engine creation failed: {e}")


@pytest.fixture(scope="module")
def bench_weights(oracle):
    return oracle.baseline_init(0)


def test_benchmark_weights_256_greedy_steps_from_a_prefilled_cache(oracle, bench_weights):
    """The benchmark's first two configurations: position 128 after a 128-id prefill, then positions 129..383."""
    from qwen3mk import prefill

    w = bench_weights
    wdev = to_dev(w)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 151936, (128,), generator=g)
    kc, vc, last = prefill.prefill(wdev, ids, "cuda")
    tok = last.argmax().to(torch.int64).reshape(())
    w32 = oracle.to_fp32(w)
    # one step, all gates (position 128)
    mk = engine(path="persist")
    inputs = dict(wdev, token=tok, kcache=kc, vcache=vc)
    out = mk.step(inputs)
    mk.status()
    ref = oracle.decode_step(w32, int(tok), kc.cpu(), vc.cpu())
    assert oracle.rel_l2(out["logits"], ref["logits"]) <= GATE_LOGITS_REL_L2
    for n in ("k_write", "v_write"):
        assert oracle.bf16_ulps(out[n], ref[n]) <= GATE_KV_ULPS, n
    # 256 chained steps with a growing cache
    steps = 256
    mk.bind(inputs, chained=True, grow=steps)
    got, logits = run_chained(mk, steps)
    flips = gate_teacher_forced(oracle, w32, int(tok), kc.cpu(), vc.cpu(), got, logits, "benchmark weights, persist")
    assert flips <= 2, f"{flips} excused token flips in {steps} steps"
    # the layered path on the same stream: 32 steps
    mk2 = engine(path="layered")
    mk2.bind(inputs, chained=True, grow=32)
    got2, logits2 = run_chained(mk2, 32)
    gate_teacher_forced(oracle, w32, int(tok), kc.cpu(), vc.cpu(), got2, logits2, "benchmark weights, layered")


def test_full_size_prefill_against_the_reference_fixture_and_the_oracle(oracle, synth_full):
    from qwen3mk import prefill

    inp = synth_full(0)
    fx = np.load(GOLDEN / "prefill_seed0_t128.npz")
    ids = fx["ids"].tolist()
    wdev = to_dev({k: inp[k] for k in oracle.WEIGHT_NAMES})
    kc, vc, last = prefill.prefill(wdev, ids, "cuda")
    assert tuple(kc.shape) == (28, 128, 8, 128)
    # the fixture: strided samples of the reference's caches, the last rows, a logits sample and the top entries
    ks, vs = torch.from_numpy(fx["k_sample"]), torch.from_numpy(fx["v_sample"])
    assert oracle.max_rel(kc[:, ::16, :, ::4], ks) <= GATE_MAX_REL and oracle.max_rel(vc[:, ::16, :, ::4], vs) <= GATE_MAX_REL
    assert oracle.rel_l2(kc[:, ::16, :, ::4], ks) <= 1e-2 and oracle.rel_l2(vc[:, ::16, :, ::4], vs) <= 1e-2
    assert oracle.max_rel(kc[:, -1], torch.from_numpy(fx["k_last"])) <= GATE_MAX_REL
    assert oracle.max_rel(vc[:, -1], torch.from_numpy(fx["v_last"])) <= GATE_MAX_REL
    sample = torch.from_numpy(fx["logits_sample"])
    assert oracle.max_rel(last[::37], sample) <= GATE_MAX_REL
    assert oracle.rel_l2(last[::37], sample) <= 1e-2
    assert int(last.argmax()) == int(fx["logits_top_idx"][0])
    # the oracle on the same ids: every row
    rk, rv, rlast = oracle.prefill(oracle.to_fp32(inp), ids)
    assert oracle.max_rel(kc, rk) <= GATE_MAX_REL and oracle.max_rel(vc, rv) <= GATE_MAX_REL
    assert oracle.rel_l2(kc, rk) <= 1e-2 and oracle.rel_l2(vc, rv) <= 1e-2
    assert oracle.max_rel(last, rlast) <= GATE_MAX_REL
    assert int(last.argmax()) == int(rlast.argmax())


def test_prompt_of_2048_then_128_greedy_steps_full_size(oracle, bench_weights):
    """The benchmark's third configuration.  The oracle's fp32 prefill of 2048 positions runs on the host cores (tens of
    seconds); the decode steps are checked against the oracle on the GPU's own bf16 cache."""
    from qwen3mk import prefill

    w = bench_weights
    wdev = to_dev(w)
    w32 = oracle.to_fp32(w)
    T, steps = 2048, 128
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 151936, (T,), generator=g)
    kc, vc, last = prefill.prefill(wdev, ids, "cuda")
    rk, rv, rlast = oracle.prefill(w32, ids.tolist())
    assert oracle.max_rel(kc, rk) <= GATE_MAX_REL and oracle.max_rel(vc, rv) <= GATE_MAX_REL
    assert oracle.rel_l2(kc, rk) <= 1e-2 and oracle.rel_l2(vc, rv) <= 1e-2
    assert oracle.max_rel(last, rlast) <= GATE_MAX_REL
    err = float((last.cpu() - rlast).abs().max())
    top2 = torch.topk(rlast, 2)
    assert int(last.argmax()) == int(top2.indices[0]) or float(top2.values[0] - top2.values[1]) <= 2 * err
    tok = last.argmax().to(torch.int64).reshape(())
    mk = engine(path="auto", max_positions=4096)
    mk.bind(dict(wdev, token=tok, kcache=kc, vcache=vc), chained=True, grow=steps)
    got, logits = run_chained(mk, steps)
    flips = gate_teacher_forced(oracle, w32, int(tok), kc.cpu(), vc.cpu(), got, logits, "2048-token prompt, then decode")
    assert flips <= 2


@pytest.mark.parametrize("batch", [8, 32, 64])
def test_full_vocabulary_batched_decode(oracle, synth_full, batch):
    """The benchmark's fourth configuration at full size: the tensor-core LM head over 151936 words and the row argmax.
    Short ragged caches keep the memory small; every sequence is checked at batch 8 and 32, every fourth at batch 64."""
    from qwen3mk.kernel import SeqTable

    inp = synth_full(0)
    w32 = oracle.to_fp32(inp)
    g = torch.Generator().manual_seed(100 + batch)
    lens = torch.randint(1, 400, (batch,), generator=g).tolist()
    toks = torch.randint(0, 151936, (batch,), generator=g)
    kcs = [(torch.randn(28, n, 8, 128, generator=g) * 0.1).to(torch.bfloat16) for n in lens]
    vcs = [(torch.randn(28, n, 8, 128, generator=g) * 0.1).to(torch.bfloat16) for n in lens]
    mk = engine(path="auto", max_batch=batch)
    seqs = SeqTable([k.cuda() for k in kcs], [v.cuda() for v in vcs])
    wdev = to_dev({k: inp[k] for k in oracle.WEIGHT_NAMES})
    out = mk.bind_sequences(wdev, toks.cuda(), seqs)
    mk.launch()
    mk.status()
    pick = range(batch) if batch <= 32 else range(0, batch, 4)
    for b in pick:
        ref = oracle.decode_step(w32, int(toks[b]), kcs[b], vcs[b])
        e = oracle.rel_l2(out["logits"][b], ref["logits"])
        assert e <= GATE_LOGITS_REL_L2, f"seq {b} len {lens[b]}: logits rel-L2 {e:.3e}"
        assert int(out["next_token"][b]) == int(ref["next_token"]), f"seq {b}"
        for n in ("k_write", "v_write"):
            assert oracle.bf16_ulps(out[n][b], ref[n]) <= GATE_KV_ULPS, (b, n)
    # every row's argmax agrees with its own logits (ties -> lowest index)
    assert torch.equal(out["next_token"].cpu(), out["logits"].argmax(dim=1).cpu())
