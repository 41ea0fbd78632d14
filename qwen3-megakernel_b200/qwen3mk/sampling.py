"""Temperature / top-k sampling on the GPU over the fp32 logits of a decode step.

The reference decodes greedily and returns the fp32 logits "for the caller" (qwen3mk/kernel.py:44-50); this module is
the step after that: `sample` picks one token per row through the C ABI (`q3_sample`), with the uniform numbers drawn
from a seeded generator so that a run can be repeated, and can write straight into the token buffer the next launch
reads.  `sample_reference` states the same rule in plain PyTorch on whatever device the logits are on; it is the
documentation of the rule, not a fallback (`sample` fails without the CUDA library).
"""
from __future__ import annotations

import torch

from . import _cabi


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, *, generator: torch.Generator | None = None,
           u: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of `logits` (CUDA fp32 [vocab] or [batch, vocab]).  top_k = 0 keeps the whole vocabulary;
    temperature <= 0 or top_k = 1 is the arg-max.  `u` (CUDA fp32 [batch], values in [0, 1)) overrides the generator.
    Enqueues on the current stream and returns the int64 tensor of tokens (`out` when given) without synchronising."""
    if not logits.is_cuda or logits.dtype != torch.float32 or not logits.is_contiguous():
        raise ValueError("sample: logits must be a contiguous CUDA float32 tensor")
    rows = logits.reshape(-1, logits.shape[-1])
    batch, vocab = rows.shape
    if u is None:
        u = torch.rand(batch, device=logits.device, dtype=torch.float32, generator=generator)
    if u.dtype != torch.float32 or u.numel() != batch or not u.is_cuda:
        raise ValueError(f"sample: u must be a CUDA float32 tensor of {batch} numbers")
    if out is None:
        out = torch.empty(logits.shape[:-1], dtype=torch.int64, device=logits.device)
    elif out.dtype != torch.int64 or out.numel() != batch or not out.is_cuda:
        raise ValueError(f"sample: out must be a CUDA int64 tensor of {batch} elements")
    lib = _cabi.load()
    rc = lib.q3_sample(rows.data_ptr(), batch, vocab, float(temperature), int(top_k), u.data_ptr(), out.data_ptr(),
                       torch.cuda.current_stream(logits.device).cuda_stream)
    _cabi.check(lib, None, rc, "q3_sample")
    return out


def sample_reference(logits: torch.Tensor, temperature: float, top_k: int, u: torch.Tensor) -> torch.Tensor:
    """The sampling rule in PyTorch (fp64): keep logits >= the k-th largest, weigh by exp((l - max) / T), return the first
    index whose cumulative weight exceeds u * total."""
    rows = logits.reshape(-1, logits.shape[-1]).double()
    if temperature <= 0 or top_k == 1:
        return rows.argmax(dim=-1).reshape(logits.shape[:-1])
    keep = torch.ones_like(rows, dtype=torch.bool)
    if 0 < top_k < rows.shape[-1]:
        kth = rows.topk(top_k, dim=-1).values[:, -1:]
        keep = rows >= kth
    w = torch.where(keep, torch.exp((rows - rows.max(dim=-1, keepdim=True).values) / temperature), torch.zeros_like(rows))
    cdf = w.cumsum(dim=-1)
    target = u.reshape(-1, 1).double().to(rows.device) * cdf[:, -1:]
    return (cdf > target).double().argmax(dim=-1).reshape(logits.shape[:-1])
