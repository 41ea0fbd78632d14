"""Timing of the decode engine: isolated launches and a steady chain.

`isolated`, `steady` and `gpu_info` restate the reference's functions of the same names (qwen3mk/bench.py:22-89): the
signatures, the result keys and the two-clock method are the contract a caller of that module relies on, so they follow
it step for step.  `grow` and `batched` are additions.
isolated: one launch on an idle GPU between two synchronisations, timed by CUDA events and by the host clock.
steady:   back-to-back chained launches (each launch's argmax is the next launch's token, no host sync);
          the value is the event time of a chain divided by its length.  `grow=True` lets the cache
          advance one position per launch instead of re-decoding the same position.
Every number is a median over repeats.
"""
from __future__ import annotations

import statistics
import time

import torch

from .kernel import Megakernel


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def isolated(mk: Megakernel, inputs: dict, iters: int = 200, warmup: int = 20, flush_l2: bool = False) -> dict:
    """Median microseconds of one isolated launch (event clock and wall clock)."""
    mk.bind(inputs)
    dev = mk.device
    scrub = None
    if flush_l2:
        scrub = torch.empty(2 * torch.cuda.get_device_properties(dev).L2_cache_size, dtype=torch.uint8, device=dev)
    for _ in range(warmup):
        mk.launch()
    torch.cuda.synchronize(dev)
    by_event, by_wall = [], []
    for _ in range(iters):
        if scrub is not None:
            scrub.zero_()
        torch.cuda.synchronize(dev)
        t0, t1 = _events()
        w0 = time.perf_counter()
        t0.record()
        mk.launch()
        t1.record()
        torch.cuda.synchronize(dev)
        by_wall.append((time.perf_counter() - w0) * 1e6)
        by_event.append(t0.elapsed_time(t1) * 1e3)
    return {"event_us_median": statistics.median(by_event), "wall_us_median": statistics.median(by_wall),
            "event_us_min": min(by_event), "event_us_max": max(by_event), "iters": iters}


def steady(mk: Megakernel, inputs: dict, steps: int = 50, reps: int = 20, warmup: int = 200, grow: bool = False) -> dict:
    """Median microseconds per step over `reps` chains of `steps` chained launches."""
    dev = mk.device
    per_step = []
    if not grow:
        mk.bind(inputs, chained=True)
        for _ in range(warmup):
            mk.launch()
        torch.cuda.synchronize(dev)
    for _ in range(reps):
        if grow:   # a fresh cache per chain, so every chain walks the same positions
            mk.bind(inputs, chained=True, grow=steps + 3)
            for _ in range(3):
                mk.launch()
            torch.cuda.synchronize(dev)
        t0, t1 = _events()
        t0.record()
        for _ in range(steps):
            mk.launch()
        t1.record()
        torch.cuda.synchronize(dev)
        per_step.append(t0.elapsed_time(t1) * 1e3 / steps)
    return {"us_per_step_median": statistics.median(per_step), "us_per_step_min": min(per_step),
            "us_per_step_max": max(per_step), "steps": steps, "reps": reps}


def gpu_info(device) -> dict:
    """GPU name, SM count and the current SM clock in MHz (None when neither NVML nor nvidia-smi answers)."""
    dev = torch.device(device)
    props = torch.cuda.get_device_properties(dev)
    info = {"name": props.name, "sm_count": props.multi_processor_count, "sm_clock_mhz": None}
    try:
        import pynvml

        pynvml.nvmlInit()
        info["sm_clock_mhz"] = pynvml.nvmlDeviceGetClockInfo(pynvml.nvmlDeviceGetHandleByIndex(dev.index or 0), pynvml.NVML_CLOCK_SM)
    except Exception:
        try:
            import subprocess

            txt = subprocess.run(["nvidia-smi", f"--id={dev.index or 0}", "--query-gpu=clocks.sm", "--format=csv,noheader,nounits"],
                                 capture_output=True, text=True, check=True).stdout
            info["sm_clock_mhz"] = int(txt.split()[0])
        except Exception:
            pass
    return info


def batched(device, w: dict, batch: int = 64, context: int = 1024, steps: int = 20, warmup: int = 3, seed: int = 0,
            lens: list[int] | None = None, graph: bool = True, path: str = "auto") -> dict:
    """Microseconds per decode step of `batch` sequences with `context` cached positions each (or the given `lens`):
    seeded random caches and tokens, one engine on `device`, CUDA-event time of `steps` back-to-back launches.
    Also returns the kernels launched per step and the algorithmic HBM bytes of a step (every weight once, the norm
    gains, and per sequence its K/V rows, embedding row, logits and new K/V rows)."""
    from .kernel import HEAD_DIM, KV_HEADS, SeqTable

    dev = torch.device(device)
    layers, vocab = w["wq"].shape[0], w["embed"].shape[0]
    lens = [context] * batch if lens is None else [int(n) for n in lens]
    g = torch.Generator(device=dev).manual_seed(seed)
    cache = lambda n: (torch.randn(layers, n, KV_HEADS, HEAD_DIM, device=dev, generator=g) * 0.1).to(torch.bfloat16)
    kcs, vcs = [cache(n) for n in lens], [cache(n) for n in lens]
    mk = Megakernel(dev, max_batch=batch, layers=layers, vocab=vocab, max_positions=max(8192, max(lens) + 8), path=path)
    toks = torch.randint(0, vocab, (batch,), device=dev, generator=g)
    mk.bind_sequences(w, toks, SeqTable(kcs, vcs), graph=graph)
    for _ in range(warmup):
        mk.launch()
    torch.cuda.synchronize(dev)
    n0 = mk.launch_count
    t0, t1 = _events()
    t0.record()
    for _ in range(steps):
        mk.launch()
    t1.record()
    torch.cuda.synchronize(dev)
    mk.status()
    us = t0.elapsed_time(t1) * 1e3 / steps
    per_layer_w = (2048 * 1024 + 2 * 1024 * 1024 + 1024 * 2048 + 2 * 3072 * 1024 + 1024 * 3072) * 2
    nbytes = layers * per_layer_w + vocab * 1024 * 2 + layers * (1024 * 2 + 128 * 2) * 2 + 1024 * 2
    nbytes += sum(layers * n * 8 * 128 * 2 * 2 + 1024 * 2 + vocab * 4 + layers * 8 * 128 * 2 * 2 for n in lens)
    return {"us_per_step": us, "tokens_per_s": batch * 1e6 / us, "kernels_per_step": (mk.launch_count - n0) / steps,
            "algorithmic_bytes": nbytes, "batch": batch, "lens_min": min(lens), "lens_max": max(lens), "lens_mean": sum(lens) / batch}
