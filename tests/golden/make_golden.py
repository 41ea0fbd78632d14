"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own Python code.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/qwen3-megakernel

The reference's modules (`qwen3mk.reference`, `qwen3mk.prefill`, `qwen3mk.weights`) are imported
from that checkout and executed on the CPU.  Inputs are never stored: they are seeded
(`weights.synthetic(seed, "cpu")` of the reference == `oracle.qwen3_oracle.synthetic(seed)`), and
each fixture carries checksums of the inputs it was made from, so a consumer can tell whether its
regenerated inputs are the same tensors.  Outputs are stored in full where small (k_write, v_write,
next_token) and as a strided sample plus the top-16 entries where large (logits, prefill caches).
"""

from __future__ import annotations

import hashlib
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
LOGIT_STRIDE = 37
KV_POS_STRIDE, KV_DIM_STRIDE = 16, 4


def load_reference(root: Path):
    """Import the reference's qwen3mk package without importing its kernel launcher's CUDA deps."""
    pkg = types.ModuleType("qwen3mk")
    pkg.__path__ = [str(root / "qwen3mk")]
    sys.modules["qwen3mk"] = pkg
    mods = {}
    for name in ("kernel", "reference", "weights", "prefill"):
        spec = importlib.util.spec_from_file_location(f"qwen3mk.{name}", root / "qwen3mk" / f"{name}.py")
        m = importlib.util.module_from_spec(spec)
        sys.modules[f"qwen3mk.{name}"] = m
        spec.loader.exec_module(m)
        setattr(pkg, name, m)
        mods[name] = m
    return mods


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def input_marks(inputs: dict) -> dict:
    """Cheap identity marks of the seeded inputs: exact for the small tensors, fp64 sums for the big ones."""
    return {
        "in_token": np.int64(int(inputs["token"])),
        "in_sha_kcache": np.array(digest(inputs["kcache"])),
        "in_sha_ln1": np.array(digest(inputs["ln1"])),
        "in_sum_wq": np.float64(inputs["wq"].double().sum().item()),
        "in_sum_wd": np.float64(inputs["wd"].double().sum().item()),
        "in_sum_embed": np.float64(inputs["embed"].double().sum().item()),
    }


def summarize_step(out: dict) -> dict:
    logits = out["logits"].float()
    top = torch.topk(logits, 16)
    return {
        "next_token": np.int64(int(out["next_token"])),
        "logits_sample": logits[::LOGIT_STRIDE].numpy().copy(),
        "logits_top_idx": top.indices.numpy().copy(),
        "logits_top_val": top.values.numpy().copy(),
        "logits_norm": np.float64(logits.double().norm().item()),
        "k_write": out["k_write"].float().numpy().copy(),
        "v_write": out["v_write"].float().numpy().copy(),
    }


def main(ref_root: str) -> None:
    torch.manual_seed(0)
    ref = load_reference(Path(ref_root))
    R, W, P = ref["reference"], ref["weights"], ref["prefill"]

    # --- full-size decode at the reference's own configuration (position 128), seeds 0 and 1,
    #     plus position 129 on seed 0 (cache extended by the bf16-rounded rows of the first step).
    for seed in (0, 1):
        inputs = W.synthetic(seed, "cpu")
        w32 = R.to_fp32(inputs)
        out = R.decode_step(w32, inputs["token"], inputs["kcache"], inputs["vcache"])
        fx = {**input_marks(inputs), **summarize_step(out)}
        np.savez_compressed(HERE / f"decode_seed{seed}_pos128.npz", **fx)
        print(f"seed {seed}: next_token {int(out['next_token'])}")
        if seed == 0:
            kc = torch.cat([inputs["kcache"], out["k_write"].to(torch.bfloat16)[:, None]], dim=1)
            vc = torch.cat([inputs["vcache"], out["v_write"].to(torch.bfloat16)[:, None]], dim=1)
            out2 = R.decode_step(w32, out["next_token"], kc, vc, pos=129)
            fx2 = {**input_marks(inputs), **summarize_step(out2), "in_step_token": np.int64(int(out["next_token"]))}
            np.savez_compressed(HERE / "decode_seed0_pos129.npz", **fx2)
            print(f"seed 0 pos 129: next_token {int(out2['next_token'])}")

            # --- prefill over 128 seeded ids with the reference's fp32 prefill
            g = torch.Generator().manual_seed(1234)
            ids = torch.randint(0, 151936, (128,), generator=g).tolist()
            kc_p, vc_p, last = P.prefill(w32, ids, "cpu")
            top = torch.topk(last, 16)
            np.savez_compressed(
                HERE / "prefill_seed0_t128.npz", **input_marks(inputs), ids=np.array(ids, dtype=np.int64),
                k_sample=kc_p[:, ::KV_POS_STRIDE, :, ::KV_DIM_STRIDE].float().numpy(),
                v_sample=vc_p[:, ::KV_POS_STRIDE, :, ::KV_DIM_STRIDE].float().numpy(),
                k_last=kc_p[:, -1].float().numpy(), v_last=vc_p[:, -1].float().numpy(),
                logits_sample=last[::LOGIT_STRIDE].numpy(), logits_top_idx=top.indices.numpy(),
                logits_top_val=top.values.numpy(), logits_norm=np.float64(last.double().norm().item()))
            print(f"prefill: argmax {int(last.argmax())}")
        del inputs, w32

    # --- a 2-layer, 4096-word model through the reference's decode_step (its layer count is a module
    #     constant, patched for this call only; every other line of the reference runs unchanged).
    sys.path.insert(0, str(HERE.parent.parent))
    from oracle import qwen3_oracle as O

    small = O.synthetic(7, O.Shape(layers=2, vocab=4096), context=40)
    R.LAYERS = 2
    try:
        out = R.decode_step(O.to_fp32(small), small["token"], small["kcache"], small["vcache"], pos=40)
    finally:
        R.LAYERS = 28
    np.savez_compressed(HERE / "decode_small_seed7_pos40.npz", in_token=np.int64(int(small["token"])),
                        in_sha_kcache=np.array(digest(small["kcache"])),
                        in_sum_wq=np.float64(small["wq"].double().sum().item()),
                        next_token=np.int64(int(out["next_token"])), logits=out["logits"].numpy(),
                        k_write=out["k_write"].numpy(), v_write=out["v_write"].numpy())
    print(f"small: next_token {int(out['next_token'])}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of a checkout of garv901/qwen3-megakernel>")
    main(sys.argv[1])
