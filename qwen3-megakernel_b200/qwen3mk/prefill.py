"""Build the KV cache of a prompt on the GPU.

Same surface as the reference's module (qwen3mk/prefill.py:22-99): `load_tokenizer`, `build_prefix`,
`prefill`, `prefix_state`, `PREFIX`.  The reference runs an fp32 PyTorch forward over exactly 128
positions; here `prefill` runs the engine's own kernels over any prompt length through the C ABI
(`q3_prefill`) and writes the bf16 caches directly.

Rules kept for the reference's 128-token case (`build_prefix`): a longer prompt is cut to its first
128 tokens and token 129 becomes the decode input; a prompt of exactly 128 tokens decodes its greedy
continuation; a shorter prompt is an error because the fixed-shape path has no padding mask.
"""
from __future__ import annotations

import ctypes

import torch

from . import _cabi
from .kernel import CONTEXT, HEAD_DIM, KV_HEADS, Megakernel
from .weights import WEIGHT_NAMES

PREFIX = CONTEXT


def load_tokenizer(model_id_or_path: str = "Qwen/Qwen3-0.6B"):
    from transformers import AutoTokenizer

    from .weights import resolve_model_dir

    return AutoTokenizer.from_pretrained(str(resolve_model_dir(model_id_or_path)))


def build_prefix(tokenizer, prompt: str, prefix: int = PREFIX) -> tuple[list[int], int | None, dict]:
    """(prefix ids, input id of the next position or None, info).  None means: take the greedy token."""
    ids = tokenizer(prompt, add_special_tokens=False)["input_ids"]
    n = len(ids)
    info = {"prompt_tokens": n, "cut": max(0, n - prefix - 1)}
    if n < prefix:
        raise ValueError(f"the prompt has {n} tokens. The kernel decodes position {prefix} and has no attention mask, "
                         f"so the prompt must have at least {prefix} tokens (padding would be attended)")
    return ids[:prefix], (ids[prefix] if n > prefix else None), info


@torch.no_grad()
def prefill(w: dict, ids, device="cuda", *, capacity: int | None = None, engine: Megakernel | None = None):
    """Causal forward over `ids` on the GPU.  w: the weight dict (bf16; fp32 copies of bf16 weights are
    cast back, which is exact).  Returns kcache, vcache (bf16 [layers, capacity, 8, 128], slots
    [0, len(ids)) filled; capacity defaults to len(ids)) and the fp32 logits [vocab] of the last position."""
    dev = torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    ids_t = torch.as_tensor(ids, dtype=torch.int64).to(dev).contiguous()
    n = ids_t.numel()
    cap = n if capacity is None else int(capacity)
    wb = {k: (w[k] if w[k].dtype == torch.bfloat16 else w[k].to(torch.bfloat16)).to(dev).contiguous() for k in WEIGHT_NAMES}
    layers, vocab = wb["wq"].shape[0], wb["embed"].shape[0]
    mk = engine if engine is not None else Megakernel(dev, layers=layers, vocab=vocab, max_tokens=n, max_positions=max(cap + 1, 256))
    mk._set_weights(wb)
    # every slot below n is written by the launch; only the spare slots are cleared (235 MB of memset at 2048 tokens otherwise)
    kc = torch.empty((layers, cap, KV_HEADS, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    vc = torch.empty_like(kc)
    if cap > n:
        kc[:, n:].zero_()
        vc[:, n:].zero_()
    logits = torch.empty(vocab, dtype=torch.float32, device=dev)
    nxt = torch.empty((), dtype=torch.int64, device=dev)
    a = _cabi.PrefillArgs(n, cap, ids_t.data_ptr(), kc.data_ptr(), vc.data_ptr(), logits.data_ptr(), nxt.data_ptr())
    rc = mk.lib.q3_prefill(mk.handle, ctypes.byref(a), torch.cuda.current_stream(dev).cuda_stream)
    _cabi.check(mk.lib, mk.handle, rc, "q3_prefill")
    torch.cuda.synchronize(dev)   # wb / ids_t may be temporaries: finish before they are released
    return kc, vc, logits


def prefix_state(w_bf16: dict, tokenizer, prompt: str, device="cuda") -> tuple[dict, dict]:
    """Engine inputs (weights plus token, kcache, vcache) for a prompt, and an info dict."""
    ids, next_id, info = build_prefix(tokenizer, prompt)
    kc, vc, last_logits = prefill(w_bf16, ids, device)
    if next_id is None:
        next_id = int(last_logits.argmax())
        info["input_id_source"] = "greedy token after the prefix"
    else:
        info["input_id_source"] = "token 129 of the prompt"
    info["input_id"] = next_id
    inputs = dict(w_bf16)
    inputs.update(token=torch.tensor(next_id, dtype=torch.int64, device=device), kcache=kc, vcache=vc)
    return inputs, info
