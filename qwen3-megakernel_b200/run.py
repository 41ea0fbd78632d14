#!/usr/bin/env python3
"""Command line for the B200 Qwen3-0.6B decode engine (same sub-commands as the reference's run.py:1-158).

  run.py check [--weights hf|synthetic] [--seed N] [--context N]
  run.py bench [--weights hf|synthetic] [--iters N] [--context N] [--grow] [--chains N]
  run.py trace [--context N]            per-phase timing of the persistent kernel (device time stamps)
  run.py compare [--context N]          the engine next to cuBLAS-through-PyTorch under a CUDA graph, same inputs
  run.py batch [--batch B] [--context N] [--steps K] [--plain]   one batched decode step of the layered path
  run.py prefill [--tokens T] [--reps N]                         causal forward over T random ids
  run.py demo --prompt "..."

`check` verifies what can be verified without a second implementation: the persistent kernel and the
layered path (two independent kernel sets) agree within the reference's gates, inputs are not mutated, and
200 re-launches reproduce the first result.  The comparison with the fp32 CPU oracle lives in tests/.
Set HF_HOME to the Hugging Face cache; HF_HUB_OFFLINE=1 forbids downloads.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

import torch  # noqa: E402

from qwen3mk import Megakernel, bench as bench_mod, prefill as prefill_mod, weights  # noqa: E402

DEFAULT_PROMPT = ("The capital of France is Paris. The capital of Germany is Berlin. The capital of Italy is Rome. " * 8
                  + "The capital of Spain is")
GATE_LOGITS_REL_L2 = 1e-4
GATE_KV_ULPS = 2
SYNC_LOGITS_REL_L2 = 1e-5


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float((a - b).norm() / b.norm())


def bf16_ulps(a: torch.Tensor, ref: torch.Tensor) -> float:
    """Largest |a - ref| in bf16 ulps of max(|ref|, rms(ref)) (the unit the reference's gate uses, run.py:42-50)."""
    r = ref.float().abs().clamp_min(float(ref.float().pow(2).mean().sqrt()))
    ulp = torch.exp2(torch.floor(torch.log2(r)) - 7)
    return float(((a.float() - ref.float()).abs() / ulp).max())


def get_inputs(kind: str, seed: int, context: int, prompt: str = DEFAULT_PROMPT, device="cuda") -> tuple[dict, dict]:
    if kind == "synthetic":
        return weights.synthetic(seed, device, context=context), {"weights": "synthetic", "seed": seed, "context": context}
    w = weights.load_hf(device=device)
    tok = prefill_mod.load_tokenizer()
    inputs, info = prefill_mod.prefix_state(w, tok, prompt, device)
    info["weights"] = "hf"
    return inputs, info


def cmd_check(args) -> int:
    inputs, info = get_inputs(args.weights, args.seed, args.context)
    print(f"inputs: {info}")
    ok = True

    def gate(name, value, limit, good):
        nonlocal ok
        ok &= bool(good)
        print(f"  {name:<34} {value}  (limit {limit})  {'ok' if good else 'FAIL'}")

    snap = {k: v.clone() for k, v in inputs.items()}
    fast = Megakernel(path="auto")
    slow = Megakernel(path="layered")
    out = fast.step(inputs)
    lay = slow.step(inputs)
    fast.status()
    slow.status()
    # the checker: the same step in fp32 PyTorch on the GPU, which shares no code with the kernels (the reference's own
    # check compares its kernel with an fp32 PyTorch step: run.py:57-104)
    from qwen3mk import baselines

    chk = baselines.TorchGraphDecoder(inputs, products="fp32")
    with torch.no_grad():
        chk._step()
    ref = {"logits": chk.logits, "next_token": chk.next_token, "k_write": chk.k_write, "v_write": chk.v_write}
    for label, got in ((f"persistent kernel (grid {fast.grid} x {fast.threads} threads)", out), ("layered kernels", lay)):
        print(f"{label} vs fp32 PyTorch")
        gate("next_token equal", f"{int(got['next_token'])} / {int(ref['next_token'])}", "equal", int(got["next_token"]) == int(ref["next_token"]))
        e = rel_l2(got["logits"], ref["logits"])
        gate("logits rel-L2", f"{e:.3e}", GATE_LOGITS_REL_L2, e <= GATE_LOGITS_REL_L2)
        for n in ("k_write", "v_write"):
            u = bf16_ulps(got[n], ref[n])
            gate(f"{n} max bf16 ulps", f"{u:.0f}", GATE_KV_ULPS, u <= GATE_KV_ULPS)
    changed = [k for k in inputs if not torch.equal(inputs[k], snap[k])]
    gate("inputs not mutated", changed or "none changed", "none", not changed)
    first = {k: v.clone() for k, v in out.items()}
    bound = fast.bind(inputs)
    for _ in range(200):
        fast.launch()
    fast.status()
    gate("200 launches: next_token", int(bound["next_token"]), "equal", int(bound["next_token"]) == int(first["next_token"]))
    e = rel_l2(bound["logits"], first["logits"])
    gate("200 launches: logits rel-L2", f"{e:.3e}", SYNC_LOGITS_REL_L2, e <= SYNC_LOGITS_REL_L2)
    for n in ("k_write", "v_write"):
        u = bf16_ulps(bound[n], first[n])
        gate(f"200 launches: {n} bf16 ulps", f"{u:.0f}", GATE_KV_ULPS, u <= GATE_KV_ULPS)
    print("PASS" if ok else "FAIL")
    return 0 if ok else 1


def cmd_bench(args) -> int:
    inputs, info = get_inputs(args.weights, args.seed, args.context)
    mk = Megakernel()
    g = bench_mod.gpu_info(mk.device)
    print(f"gpu: {g['name']}  SMs: {g['sm_count']}  SM clock: {g['sm_clock_mhz']} MHz  inputs: {info}")
    iso = bench_mod.isolated(mk, inputs, iters=args.iters)
    print(f"isolated: median {iso['event_us_median']:.1f} us (events), {iso['wall_us_median']:.1f} us (wall); "
          f"event min {iso['event_us_min']:.1f} max {iso['event_us_max']:.1f}; iters {iso['iters']}")
    st = bench_mod.steady(mk, inputs, grow=args.grow, reps=args.chains)
    print(f"steady:   median {st['us_per_step_median']:.1f} us/step; min {st['us_per_step_min']:.1f} max {st['us_per_step_max']:.1f}; "
          f"{st['reps']} chains of {st['steps']} steps{' (cache grows)' if args.grow else ''}")
    mk.status()
    return 0


PHASE_EVENTS = ["Q stage", "Q done", "K/V prefetch", "F q/k/v exchange", "F partial", "F group", "F done", "wait attn delta",
                "GD stage", "GD hid", "GD done", "wait FFN delta"]


def cmd_trace(args) -> int:
    """Median duration of every traced segment of a layer, plus the skew and the hop of the two delta waits (skew: how
    long the last CTA's contribution trails the median CTA's; hop: from that last contribution to the median CTA having
    the complete delta in registers)."""
    import numpy as np

    inputs, info = get_inputs("synthetic", args.seed, args.context)
    mk = Megakernel(path="persist")
    tr = mk.enable_trace()
    mk.bind(inputs)
    for _ in range(4):
        mk.launch()
    mk.status()
    t = tr.cpu().numpy().astype(np.int64)
    t = t - t[:, 0].min()
    L, ev = mk.layers, 12
    med = np.median(t, axis=0)
    seg = np.zeros((L, ev))
    for layer in range(L):
        b = 1 + ev * layer
        for k in range(ev):
            seg[layer, k] = med[b + k] - (med[b + k - 1] if (k or layer) else med[0])
    m = np.median(seg[1:], axis=0) if L > 1 else seg[0]
    print(f"context {args.context}: kernel span {t[:, 2 + ev * L].max() / 1e3:.1f} us, layers {med[ev * L] / 1e3:.1f} us, "
          f"LM head {(t[:, 1 + ev * L].max() - med[ev * L]) / 1e3:.1f} us, layer median {m.sum() / 1e3:.2f} us")
    for n, v in zip(PHASE_EVENTS, m):
        print(f"  {n:<16} {v:7.0f} ns")
    for name, d in (("F", 6), ("GD", 10)):
        skew = np.median([t[:, 1 + ev * l + d].max() - np.median(t[:, 1 + ev * l + d]) for l in range(1, L)])
        hop = np.median([np.median(t[:, 2 + ev * l + d]) - t[:, 1 + ev * l + d].max() for l in range(1, L)])
        print(f"  delta after {name:<3} skew {skew:6.0f} ns  hop {hop:6.0f} ns")
    return 0


def cmd_compare(args) -> int:
    """The measured-comparator table (the reference's README.md:12-18 rows that need no extra package)."""
    from qwen3mk import baselines

    inputs, info = get_inputs(args.weights, args.seed, args.context)
    g = bench_mod.gpu_info("cuda")
    print(f"gpu: {g['name']}  SM clock: {g['sm_clock_mhz']} MHz  inputs: {info}")
    for r in baselines.compare(inputs):
        print(f"  {r['name']:<40} {r['us_per_step_median']:9.1f} us/step (min {r['us_per_step_min']:.1f})   {r['note']}")
    return 0


def cmd_batch(args) -> int:
    """One batched decode step (layered tensor-core path): `--batch` sequences of `--context` cached positions."""
    from qwen3mk.kernel import SeqTable, LAYERS, KV_HEADS, HEAD_DIM, VOCAB

    # under torchrun every rank runs its own replica of the batch on its own GPU; the time is the slowest rank's
    import os
    import torch.distributed as dist
    from qwen3mk import replicas

    world, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, ctx = args.batch, args.context
    w = weights.baseline_init(args.seed, dev)
    lens = None
    if args.ragged:   # cache lengths uniform in [128, context], seeded
        lens = torch.randint(128, ctx + 1, (B,), generator=torch.Generator().manual_seed(args.seed)).tolist()
    if world > 1:
        dist.barrier()
    res = bench_mod.batched(dev, w, B, ctx, steps=args.steps, seed=args.seed, lens=lens, graph=not args.plain, path=args.path)
    us = res["us_per_step"]
    if world > 1:
        us = replicas.max_over_ranks(us, dev)
        dist.barrier()
        if dist.get_rank() == 0:
            print(f"{world} replicas of batch {B}: {us:.1f} us/step on the slowest, {world * B * 1e6 / us:.0f} tokens/s over the job")
        dist.destroy_process_group()
        return 0
    shape = f"{B} sequences of {res['lens_min']}..{res['lens_max']} (mean {res['lens_mean']:.0f})" if args.ragged else f"{B} x {ctx}"
    print(f"batch {shape} cached positions: {us:.1f} us/step, {B * 1e6 / us:.0f} tokens/s, "
          f"{res['algorithmic_bytes'] / us / 1e6:.2f} TB/s of algorithmic bytes, {res['kernels_per_step']:.0f} kernels per step"
          f"{' (plain launches)' if args.plain else ' (graph replay)'}")
    return 0


def cmd_prefill(args) -> int:
    """Causal forward over `--tokens` uniform-random ids (tcgen05 GEMMs + tiled attention), timed with CUDA events."""
    from qwen3mk.kernel import VOCAB

    dev = torch.device("cuda", torch.cuda.current_device())
    T = args.tokens
    w = weights.baseline_init(args.seed, dev)
    g = torch.Generator().manual_seed(args.seed)
    ids = torch.randint(0, VOCAB, (T,), generator=g)
    mk = Megakernel(dev, max_tokens=T, max_positions=max(T + 1, 256))
    times = []
    for i in range(args.reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        prefill_mod.prefill(w, ids, dev, engine=mk)
        e1.record()
        torch.cuda.synchronize(dev)
        if i:   # the first call packs the weights and builds the tensor maps
            times.append(e0.elapsed_time(e1))
    mk.status()
    ms = sorted(times)[len(times) // 2]
    flop = 2.0 * T * 15_728_640 * 28 + 4.0 * 28 * 16 * 128 * (T * (T + 1) / 2)   # projections + causal QK^T and PV
    print(f"prefill of {T} tokens: {ms:.2f} ms (median of {len(times)}; includes the cache allocation and one synchronisation), "
          f"{T / ms:.0f} tokens/ms, {flop / ms / 1e9:.0f} TFLOP/s of algorithmic flops")
    return 0


def cmd_demo(args) -> int:
    try:
        tok = prefill_mod.load_tokenizer()
        prefill_mod.build_prefix(tok, args.prompt)
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    w = weights.load_hf(device="cuda")
    inputs, info = prefill_mod.prefix_state(w, tok, args.prompt, "cuda")
    print(f"prompt tokens: {info['prompt_tokens']}  cut: {info['cut']}  input id ({info['input_id_source']}): "
          f"{info['input_id']} {tok.decode([info['input_id']])!r}")
    mk = Megakernel()
    out = mk.step(inputs)
    ref = Megakernel(path="layered").step(inputs)
    got, want = int(out["next_token"]), int(ref["next_token"])
    print(f"persistent kernel next token: {got} {tok.decode([got])!r}")
    print(f"layered kernels  next token: {want} {tok.decode([want])!r}")
    print(f"match: {got == want}")
    return 0 if got == want else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("check", "bench", "trace", "compare"):
        p = sub.add_parser(name)
        p.add_argument("--weights", choices=["hf", "synthetic"], default="synthetic")
        p.add_argument("--seed", type=int, default=0)
        p.add_argument("--context", type=int, default=128)
        if name == "bench":
            p.add_argument("--iters", type=int, default=200)
            p.add_argument("--grow", action="store_true")
            p.add_argument("--chains", type=int, default=20, help="chains of 50 steps in the steady measurement")
    p = sub.add_parser("batch")
    p.add_argument("--batch", type=int, default=64)
    p.add_argument("--context", type=int, default=1024)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--plain", action="store_true", help="plain launches instead of CUDA-graph replay")
    p.add_argument("--ragged", action="store_true", help="cache lengths drawn uniformly from [128, --context]")
    p.add_argument("--path", default="auto", choices=["auto", "layered", "fused"],
                   help="fused: the persistent layer kernel between the attention launches instead of one launch per phase")
    p = sub.add_parser("prefill")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--reps", type=int, default=5)
    p.add_argument("--seed", type=int, default=0)
    p = sub.add_parser("demo")
    p.add_argument("--prompt", default=DEFAULT_PROMPT)
    args = ap.parse_args(argv)
    return {"check": cmd_check, "bench": cmd_bench, "trace": cmd_trace, "compare": cmd_compare, "batch": cmd_batch, "prefill": cmd_prefill, "demo": cmd_demo}[args.cmd](args)


if __name__ == "__main__":
    sys.exit(main())
