#!/usr/bin/env python3
"""Benchmark of the Qwen3-0.6B decode path on B200: microseconds per decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (`config.workload`): batch-1 greedy decode with the benchmark's weights (bf16 N(0, 0.02)
matrices, unit RMSNorm gains, seeded), a KV cache built by prefilling 128 uniform-random token ids,
then K consecutive steps starting at position 128; the cache grows on the device and each step's
argmax feeds the next.  One "step" = one decode step.  With N GPUs every rank runs its own replica of
that stream (no inter-GPU traffic), the time is the maximum over ranks and `value` is that time per step
divided by N (the job finishes N steps in it); `per_replica_us_per_step` keeps the undivided figure.

One JSON line is printed by rank 0.  `value` is the device-timed figure with everything resident in
HBM; `e2e` is the same stream driven from host memory (token in from pinned memory, token out to the
host, one synchronisation per step).  `--impl reference` times the CPU restatement of the reference's
fp32 decode step (oracle/) on the host cores for the same workload, a bounded number of steps.

Extra records in the line: `reference_kernel` (the reference project's own CUDA kernel timed on this GPU through its
own launcher and timing code, from baseline/_ref, in a child process; `unavailable` with the reason otherwise),
`batch64_ctx1024` (the replicated batched-decode configuration: 64 sequences of 1024 cached positions per GPU),
`prefill_t2048` (a causal forward over 2048 tokens, single-GPU runs) and
`static_ctx128` (position 128 held fixed, the case the reference's published figure is quoted on).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (str(ROOT), str(ROOT / "qwen3-megakernel_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

CTX0 = 128
TRAFFIC_PROFILE = ROOT / "profiles" / "persist_decode_bs1_ctx128.md"   # the ncu summary that holds the kernel's DRAM traffic per launch
PUBLISHED_US = 373.6        # the reference kernel's steady microseconds per step on one B200 (its README)
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def algorithmic_bytes(ctx: int, layers: int = 28, vocab: int = 151936) -> int:
    """HBM bytes one batch-1 decode step must move at cache length `ctx`: every weight once, the norm
    gains, the cached K/V rows, the embedding row, the logits and the new K/V rows."""
    per_layer_w = (2048 * 1024 + 2 * 1024 * 1024 + 1024 * 2048 + 2 * 3072 * 1024 + 1024 * 3072) * 2
    weights = layers * per_layer_w + vocab * 1024 * 2
    gains = layers * (1024 * 2 + 128 * 2) * 2 + 1024 * 2
    kv_read = layers * ctx * 8 * 128 * 2 * 2
    per_seq = 1024 * 2 + vocab * 4 + layers * 8 * 128 * 2 * 2
    return weights + gains + kv_read + per_seq


def ncu_traffic() -> dict | None:
    """DRAM bytes per launch of the persistent kernel at cache length 128, read from the committed ncu summary (a line
    `traffic_bytes_per_launch: <bytes> (commit <hash>)`), with the commit the capture was made on."""
    try:
        m = re.search(r"traffic_bytes_per_launch:\s*(\d+)\s*\(commit\s+(\w+)\)", TRAFFIC_PROFILE.read_text())
        return {"bytes": int(m.group(1)), "commit": m.group(2)} if m else None
    except OSError:
        return None


def reference_kernel_record(timeout_s: int = 240) -> dict:
    """The reference project's own kernel on this GPU (baseline/time_ref_kernel.py, a child process that imports nothing
    of this repository's engine).  Never raises: a failure is reported as {"unavailable": reason}."""
    script = ROOT / "baseline" / "time_ref_kernel.py"
    if not (ROOT / "baseline" / "_ref" / "qwen3mk" / "kernel.py").exists():
        return {"unavailable": "baseline/_ref is not installed (python baseline/install_ref.py)"}
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS"):
        env.pop(k, None)
    try:
        r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=timeout_s, env=env)
        lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        return json.loads(lines[-1]) if lines else {"unavailable": f"no output (exit {r.returncode}): {r.stderr.strip()[-200:]}"}
    except subprocess.TimeoutExpired:
        return {"unavailable": f"no answer within {timeout_s} s"}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"}


def prefill_record(dev, w: dict, tokens: int = 2048, reps: int = 3) -> dict:
    """Milliseconds of a causal forward over `tokens` seeded random ids through `prefill.prefill` (CUDA events, median of
    `reps` after one untimed call; includes allocating the cache), with the algorithmic flops of the projections and of the
    causal QK^T and PV products."""
    from qwen3mk import Megakernel, prefill as prefill_mod

    ids = torch.randint(0, w["embed"].shape[0], (tokens,), generator=torch.Generator().manual_seed(0))
    mk = Megakernel(dev, max_tokens=tokens, max_positions=max(tokens + 1, 256))
    times = []
    for i in range(reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        prefill_mod.prefill(w, ids, dev, engine=mk)
        e1.record()
        torch.cuda.synchronize(dev)
        if i:
            times.append(e0.elapsed_time(e1))
    mk.status()
    ms = sorted(times)[len(times) // 2]
    flop = 2.0 * tokens * 15_728_640 * 28 + 4.0 * 28 * 16 * 128 * (tokens * (tokens + 1) / 2)
    return {"ms": ms, "tokens_per_s": tokens / ms * 1e3, "algorithmic_tflops": flop / ms / 1e9, "tokens": tokens, "activation_planes": 1}


def measured_peak_gbs() -> tuple[float, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Polls NVML for the SM clock and the throttle reasons while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None
        self._period = period_s

    def _run(self):
        nv = self._nv
        names = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80, "sw_power_cap": 0x4}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for n, b in names.items():
                    if bits & b:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(self._period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def build_workload(device, seed: int = 0):
    """Weights on `device` and the 128-position cache prefilled on the GPU from seeded random ids."""
    from qwen3mk import prefill, weights

    w = weights.baseline_init(seed, device)
    g = torch.Generator().manual_seed(seed + 1)
    ids = torch.randint(0, 151936, (CTX0,), generator=g)
    kc, vc, last = prefill.prefill(w, ids, device)
    inputs = dict(w)
    inputs.update(token=last.argmax().to(torch.int64).reshape(()), kcache=kc, vcache=vc)
    return inputs, ids


def cpu_workload(O, seed: int = 0):
    """The GPU arm's workload rebuilt on the host: the same seeded weights, the cache of the same 128 seeded ids (through the
    oracle's fp32 prefill, rounded to bf16) and the prompt's greedy token."""
    w32 = O.to_fp32(O.baseline_init(seed))
    g = torch.Generator().manual_seed(seed + 1)
    ids = torch.randint(0, 151936, (CTX0,), generator=g)
    kc, vc, last = O.prefill(w32, ids.tolist())
    return w32, int(last.argmax()), kc, vc


def cpu_baseline(seconds: float = 12.0, seed: int = 0) -> dict:
    """The oracle's decode step on the host cores: same weights and cache length, a bounded number of steps."""
    from oracle import qwen3_oracle as O

    w32, tok, kc, vc = cpu_workload(O, seed)
    O.decode_step(w32, tok, kc, vc)  # warm-up
    times = []
    t_end = time.perf_counter() + seconds
    while time.perf_counter() < t_end and len(times) < 200:
        t0 = time.perf_counter()
        out = O.decode_step(w32, tok, kc, vc)
        times.append(time.perf_counter() - t0)
        tok = int(out["next_token"])
    return {"value": statistics.median(times) * 1e6, "unit": "us/step", "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": "port",
            "sample": f"{len(times)} decode steps at position {CTX0} (fp32 torch on the host, median)"}


def run_reference_arm(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    steps = max(1, min(args.steps, 64))
    # every host core: a launcher such as torchrun sets OMP_NUM_THREADS=1 for its ranks, which would slow this arm fivefold
    torch.set_num_threads(os.cpu_count() or 1)
    from oracle import qwen3_oracle as O

    w32, tok, kc, vc = cpu_workload(O, 0)
    for _ in range(max(1, min(args.warmup, 3))):
        O.decode_step(w32, tok, kc, vc)
    t0 = time.perf_counter()
    res = O.greedy_decode(w32, tok, kc, vc, steps)
    dt = time.perf_counter() - t0
    us = dt / steps * 1e6
    assert res["tokens"].numel() == steps
    line = {"impl": "reference", "metric": "us_per_step_qwen3_0.6b_bs1_ctx128", "value": us, "unit": "us/step",
            "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": us / 1e3,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"Qwen3-0.6B bs1 greedy decode, {args.steps} consecutive steps from position {CTX0} "
                                   f"(cache {CTX0 + 1}->{CTX0 + args.steps} positions)",
                       "sample": f"the first {steps} of those steps on the host cores (fp32 restatement of the reference's CPU path)",
                       "weights": "bf16 N(0,0.02), RMSNorm gains 1, seed 0", "cache": "prefill of 128 uniform-random ids (fp32 on the host)"},
            "cpu_baseline": {"value": us, "unit": "us/step", "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(),
                             "kind": "port", "sample": f"{steps} greedy steps from position {CTX0}"},
            "e2e": {"value": us, "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "tokens_per_s": 1e6 / us, "gpu_launches": 0}
    print(json.dumps(line))


def tensor_parallel_record(dev, inputs: dict, world: int, barrier) -> dict:
    """Batch-1 decode split over all `world` GPUs (heads, FFN rows and vocabulary sharded; the per-layer sums run inside the
    kernel over NVLink).  Tokens of 64 growing steps are compared with the single-GPU engine's on the same inputs; the time
    is the steady figure at position 128 and the mean of the 64 growing steps, the slowest rank's."""
    from qwen3mk import Megakernel, bench as bench_mod, replicas, tp

    n_tok = 64

    def stream(mk):
        mk.bind(inputs, chained=True, grow=n_tok)
        toks = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n_tok):
            mk.launch()
            toks.append(mk.chain_token.clone())
        e1.record()
        torch.cuda.synchronize(dev)
        mk.status()
        return torch.stack(toks).cpu().tolist(), e0.elapsed_time(e1) * 1e3 / n_tok

    single = Megakernel(dev, path="persist", max_positions=8192)
    want, _ = stream(single)
    del single
    mk = Megakernel(dev, path="persist", max_positions=8192, wait_limit_us=2_000_000)
    shard = tp.attach(mk)
    got, grow_us = stream(mk)
    barrier()
    static_us = bench_mod.steady(mk, inputs, steps=50, reps=5, warmup=50)["us_per_step_median"]
    mk.status()
    barrier()
    same = sum(int(a == b) for a, b in zip(got, want))
    return {"ranks": world, "us_per_step_ctx128": replicas.max_over_ranks(static_us, dev),
            "us_per_step_growing_64": replicas.max_over_ranks(grow_us, dev), "tokens_equal_to_single_gpu": f"{same}/{n_tok}",
            "tokens_per_s": 1e6 / replicas.max_over_ranks(static_us, dev),
            "shard": {"q_heads": len(shard.q_heads), "kv_heads": len(shard.kv_heads), "ffn_rows": len(shard.ffn_rows), "words": len(shard.words)},
            "note": "one decode stream over all GPUs; sums over ranks by red instructions into every rank's accumulators over NVLink"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--path", choices=["auto", "layered", "persist"], default="auto")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-extras", action="store_true", help="leave out the batch64_ctx1024 and reference_kernel records (profiling runs)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return 0

    import torch.distributed as dist

    from qwen3mk import Megakernel, replicas

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    K, W = args.steps, max(args.warmup, 3)

    inputs, _ = build_workload(dev)
    mk = Megakernel(dev, path=args.path, max_positions=max(8192, CTX0 + K + W + 8))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident: W warm-up steps, then exactly K chained steps on a fresh cache ------------
    mk.bind(inputs, chained=True, grow=W)
    for _ in range(W):
        mk.launch()
    torch.cuda.synchronize(dev)
    mk.bind(inputs, chained=True, grow=K)
    n0 = mk.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local) as clk:
        e0.record()
        for _ in range(K):
            mk.launch()
        e1.record()
        barrier()
    launches = mk.launch_count - n0
    mk.status()
    ms = e0.elapsed_time(e1)
    last_token = int(mk.chain_token)
    ms = replicas.max_over_ranks(ms, dev)          # the job is as slow as its slowest replica
    us_step = ms * 1e3 / K

    # ---- end to end from host memory: token H2D, step, token D2H, every step -------------------------
    Ke = min(K, 128)
    e2e_inputs = dict(inputs, token=inputs["token"].clone())   # the token buffer below is rewritten every step
    mk.bind(e2e_inputs, chained=False, grow=Ke + 3)
    tok_host = torch.empty(1, dtype=torch.int64).pin_memory()
    out_host = torch.empty(1, dtype=torch.int64).pin_memory()
    tok_dev = mk._tok[0]
    bound = mk._out
    tok_host[0] = int(inputs["token"])
    t0 = time.perf_counter()
    for i in range(3 + Ke):
        if i == 3:
            barrier()
            t0 = time.perf_counter()
        tok_dev.copy_(tok_host, non_blocking=True)
        mk.launch()
        out_host.copy_(bound[1].reshape(1), non_blocking=True)
        torch.cuda.synchronize(dev)
        tok_host[0] = out_host[0]
    e2e_s = time.perf_counter() - t0
    e2e_s = replicas.max_over_ranks(e2e_s, dev)
    e2e_us = e2e_s / Ke * 1e6

    # ---- the published figure's own case, for reference: position 128 held fixed (the cache does not grow) ----
    from qwen3mk import bench as bench_mod
    static_us = bench_mod.steady(mk, inputs, steps=50, reps=5, warmup=50)["us_per_step_median"]
    mk.status()

    # ---- the replicated batched configuration: 64 sequences of 1024 cached positions on every GPU ----------------
    b64 = None
    if not args.skip_extras:
        barrier()
        weights_only = {k: inputs[k] for k in inputs if k not in ("token", "kcache", "vcache")}
        b64 = bench_mod.batched(dev, weights_only, 64, 1024, steps=20)
        b64_us = replicas.max_over_ranks(b64["us_per_step"], dev)
        barrier()

    # ---- the prompt configuration: causal forward over 2048 tokens (rank 0 of a single-GPU run) ----------------------
    prefill_rec = None
    if not args.skip_extras and world == 1:
        try:
            prefill_rec = prefill_record(dev, weights_only)
        except Exception as e:  # noqa: BLE001
            prefill_rec = {"unavailable": f"{type(e).__name__}: {e}"}

    # ---- tensor parallelism over all N GPUs: the same stream as one job instead of N replicas ------------------------
    tp_rec = None
    if world in (2, 4, 8):
        try:
            tp_rec = tensor_parallel_record(dev, inputs, world, barrier)
        except Exception as e:  # noqa: BLE001  (the replica figures above stand on their own)
            tp_rec = {"ranks": world, "error": f"{type(e).__name__}: {e}"[:300]}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    traffic = ncu_traffic()
    mean_ctx = CTX0 + (K - 1) / 2.0
    bytes_step = algorithmic_bytes(int(round(mean_ctx)))
    peak, peak_kind = measured_peak_gbs()
    achieved = bytes_step / (us_step * 1e-6) / 1e9
    launches_per_step = launches / K
    grid = mk.grid
    line = {
        # whole-job figure: the N replicas together finish N decode steps in the time of one
        "metric": "us_per_step_qwen3_0.6b_bs1_ctx128", "value": us_step / world, "unit": "us/step", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": us_step / 1e3, "higher_is_better": False, "scaling": "weak",
        "per_replica_us_per_step": us_step,
        "vs_baseline": us_step / world / PUBLISHED_US, "dtype": "bf16 weights, fp32 activations and accumulation",
        "data": "synthetic",
        "config": {"workload": f"Qwen3-0.6B bs1 greedy decode, {K} consecutive steps from position {CTX0} "
                               f"(cache {CTX0 + 1}->{CTX0 + K} positions, grows on the device)",
                   "weights": "bf16 N(0,0.02), RMSNorm gains 1, seed 0", "cache": "prefill of 128 uniform-random ids on the GPU",
                   "replicas": world, "path": args.path, "launches_per_step": launches_per_step,
                   "persistent_grid": grid, "l2": "inputs larger than L2: 1.19 GB of weights streamed every step"},
        "tokens_per_s": world * 1e6 / us_step,
        "hbm_frac_of_8tbs": bytes_step / (us_step * 1e-6) / 1e9 / NOMINAL_HBM_GBS,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "traffic": traffic["bytes"] if traffic else None,
                     "traffic_source": (f"ncu capture of one launch at cache length 128 on commit {traffic['commit']} "
                                        f"({TRAFFIC_PROFILE.name})") if traffic else None,
                     "algorithmic_bytes_per_step": bytes_step,
                     "kernel": "q3_persist_decode (one launch per step)" if launches_per_step <= 1.5 else
                               f"whole step ({launches_per_step:.0f} launches)"},
        "e2e": {"value": e2e_us / world, "unit": "us/step", "h2d_bytes_per_step": 8 * world, "d2h_bytes_per_step": 8 * world, "steps": Ke,
                "per_replica_us_per_step": e2e_us},
        "gpu_launches": launches, "clocks": clk.summary(), "last_token": last_token,
        "static_ctx128": {"us_per_step": static_us, "vs_published": static_us / PUBLISHED_US,
                          "note": "position 128 held fixed: the case the reference's 373.6 us is quoted on"},
    }
    if tp_rec is not None:
        line["tp"] = tp_rec
    if prefill_rec is not None:
        line["prefill_t2048"] = prefill_rec
    if b64 is not None:
        line["batch64_ctx1024"] = {"us_per_step_slowest": b64_us, "tokens_per_s_job": world * 64 * 1e6 / b64_us,
                                   "tokens_per_s_per_gpu": 64 * 1e6 / b64_us, "kernels_per_step": b64["kernels_per_step"],
                                   "hbm_gbs": b64["algorithmic_bytes"] / (b64_us * 1e-6) / 1e9,
                                   "hbm_frac": b64["algorithmic_bytes"] / (b64_us * 1e-6) / 1e9 / peak,
                                   "note": "one replica per GPU, 64 sequences x 1024 cached positions each, no inter-GPU traffic"}
        ref_k = reference_kernel_record()
        if "steady_us" in ref_k:
            ref_k["ours_static_over_reference_steady"] = static_us / ref_k["steady_us"]
        line["reference_kernel"] = ref_k
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
