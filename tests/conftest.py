"""Shared pytest setup: the `gpu` marker, import paths, and session-cached seeded inputs."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "qwen3-megakernel_b200"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); deselected by -m 'not gpu'")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import qwen3_oracle

    return qwen3_oracle


_SYNTH_CACHE: dict = {}


@pytest.fixture(scope="session")
def synth_full(oracle):
    """Seeded full-size inputs, generated once per seed per session (about 8 s each)."""
    def get(seed: int):
        if seed not in _SYNTH_CACHE:
            _SYNTH_CACHE.clear()          # hold one 1.2 GB set at a time
            _SYNTH_CACHE[seed] = oracle.synthetic(seed)
        return _SYNTH_CACHE[seed]
    return get


# ---- helpers of the greedy-decode parity tests ---------------------------------------------------------

def run_chained(mk, steps):
    """`steps` chained launches on the bound inputs; returns the tokens and a copy of every step's logits."""
    toks, logits = [], []
    out = mk._out
    for _ in range(steps):
        mk.launch()
        toks.append(mk.chain_token.clone())
        logits.append(out[0].clone())
    mk.status()
    return torch.stack(toks).cpu(), logits


def gate_teacher_forced(oracle, w32, token, kc, vc, got_tokens, got_logits, what):
    """Replay the GPU's token stream through the oracle and gate every step.  Returns the number of excused flips."""
    flips = []

    def on_step(i, out):
        g = got_logits[i].cpu()
        e = oracle.rel_l2(g, out["logits"])
        assert e <= 1e-4, f"{what}: step {i}: logits rel-L2 {e:.3e}"
        want, got = int(out["next_token"]), int(got_tokens[i])
        if got != want:
            err = float((g - out["logits"]).abs().max())
            top2 = torch.topk(out["logits"], 2).values
            margin = float(top2[0] - top2[1])
            assert margin <= 2 * err + 1e-7, f"{what}: step {i}: token {got}, oracle {want}, top-2 margin {margin:.3e}, max logit error {err:.3e}"
            flips.append((i, got, want, margin, err))

    oracle.greedy_decode(w32, token, kc, vc, len(got_tokens), forced_tokens=got_tokens.tolist(), on_step=on_step)
    for i, got, want, margin, err in flips:
        print(f"{what}: step {i}: token {got} instead of {want} excused: top-2 margin {margin:.3e} <= 2 x logit error {err:.3e}")
    return len(flips)
