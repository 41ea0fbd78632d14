"""Qwen3-0.6B decode on one B200 through the q3mk C-ABI library (hand-written sm_100a CUDA).

Drop-in surface of the reference package (qwen3mk/__init__.py:3-5): `Megakernel`, `INPUT_ORDER`,
and the submodules `kernel`, `weights`, `prefill`, `bench`.
"""
from .kernel import INPUT_ORDER, Megakernel

__all__ = ["INPUT_ORDER", "Megakernel"]
