"""Time the reference project's own decode kernel on this GPU, through its own launcher and timing code.

    python baseline/time_ref_kernel.py [--steps 50] [--reps 20] [--iters 200]

Runs in its own process with ONLY baseline/_ref on the import path: the reference's `qwen3mk.Megakernel`
(NVRTC-compiles csrc/qwen3_step.cu, cooperative launch), its `weights.synthetic(0)` inputs, its
`bench.steady` and `bench.isolated` (qwen3mk/bench.py:22-66), and its CPU oracle for one sanity step.  Nothing
of this repository's engine is imported.  Prints one JSON line; on any failure the line is
{"unavailable": "<error>"} and the exit code is still 0, so the caller can quote the reason."""
from __future__ import annotations

import argparse
import json
import sys
import traceback
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=200)
    args = ap.parse_args()
    try:
        if not (REF / "qwen3mk" / "kernel.py").exists():
            raise RuntimeError("baseline/_ref is missing: run `python baseline/install_ref.py` where the reference tree is mounted")
        sys.path.insert(0, str(REF))
        import torch
        from cuda.bindings import nvrtc

        import qwen3mk
        from qwen3mk import bench, reference, weights

        assert Path(qwen3mk.__file__).resolve().is_relative_to(REF), qwen3mk.__file__
        dev = torch.device("cuda", 0)
        mk = qwen3mk.Megakernel(dev)
        inputs = weights.synthetic(0, dev)
        out = mk.step(inputs)
        torch.cuda.synchronize(dev)
        cpu = {k: v.cpu() for k, v in inputs.items()}
        ref = reference.decode_step(reference.to_fp32(cpu), cpu["token"], cpu["kcache"], cpu["vcache"])
        token_ok = bool(int(out["next_token"]) == int(ref["next_token"]))
        st = bench.steady(mk, inputs, steps=args.steps, reps=args.reps, warmup=args.warmup)
        iso = bench.isolated(mk, inputs, iters=args.iters, warmup=20)
        info = bench.gpu_info(dev)
        _, major, minor = nvrtc.nvrtcVersion()
        line = {"steady_us": st["us_per_step_median"], "steady_us_min": st["us_per_step_min"], "steady_us_max": st["us_per_step_max"],
                "isolated_us": iso["event_us_median"], "isolated_wall_us": iso["wall_us_median"],
                "nvrtc": f"{major}.{minor}", "grid": mk.grid, "arch": mk.arch, "clocks": {"sm_mhz": info.get("sm_clock_mhz")},
                "gpu": info.get("name"), "token_matches_its_cpu_reference": token_ok,
                "what": "the reference's csrc/qwen3_step.cu through its own Megakernel and bench.steady / isolated, "
                        "weights.synthetic(0), batch 1, position 128 held fixed"}
    except BaseException as e:  # noqa: BLE001  (the caller wants the reason, whatever it is)
        msg = f"{type(e).__name__}: {e}".strip().splitlines()
        line = {"unavailable": (msg[0] if msg else "error")[:300], "trace_tail": traceback.format_exc().strip().splitlines()[-3:]}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
