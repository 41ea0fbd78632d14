"""Shared pytest setup: the `gpu` marker, import paths, and session-cached seeded inputs."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

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
