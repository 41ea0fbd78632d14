"""CPU oracle for the Qwen3-0.6B decode / prefill path.  TEST INFRASTRUCTURE ONLY.

This module is the checker the parity tests, the smoke test and the CPU-baseline leg
of the benchmark compare the CUDA engine against.  Nothing in the shipped package may
import it: the product path is the CUDA library and fails loudly without it.

It restates, in plain fp32 PyTorch on the host, the algorithm of the reference
project (garv901/qwen3-megakernel):

  * one decode step            qwen3mk/reference.py:44-87  (`decode_step`)
  * RMSNorm                    qwen3mk/reference.py:20-23
  * RoPE tables (fp64 angles)  qwen3mk/reference.py:26-31, qwen3mk/kernel.py:102-106
  * rotate-half                qwen3mk/reference.py:34-36
  * masked softmax attention   qwen3mk/reference.py:90-97
  * causal prefill             qwen3mk/prefill.py:46-81   (reference asserts T == 128; here T is free)
  * seeded synthetic inputs    qwen3mk/weights.py:101-124

Conventions kept from the reference: all activations fp32; weights are bf16 values
widened to fp32; the new token's K and V enter attention UNROUNDED while cached K/V
are whatever the (bf16) cache holds; K is stored after head-norm and RoPE; ties in
argmax resolve to the lowest index (torch.argmax on CPU).

Parity pin: `tests/golden/*.npz` were produced by importing the reference's own
Python modules (see tests/golden/make_golden.py) and `tests/test_oracle_golden.py`
checks this restatement against them.

Differences in form (not in result): the reference materialises a zero-padded fp32
cache of pos+1 slots and masks; here the new K/V row is concatenated to the cached
rows, which is the same set of attended positions.  The layer count, vocabulary and
batch are taken from the tensors so small models can be checked quickly.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

HIDDEN = 1024
Q_HEADS = 16
KV_HEADS = 8
HEAD_DIM = 128
INTER = 3072
VOCAB = 151936
LAYERS = 28
EPS = 1e-6
ROPE_THETA = 1e6

WEIGHT_NAMES = ("ln1", "wq", "wk", "wv", "qn", "kn", "wo", "ln2", "wg", "wu", "wd", "fnorm", "embed")


@dataclass(frozen=True)
class Shape:
    """Model extents that may be shrunk for quick tests; the per-head geometry is fixed."""
    layers: int = LAYERS
    vocab: int = VOCAB


def weight_shapes(shape: Shape = Shape()) -> dict:
    L, V = shape.layers, shape.vocab
    return {
        "ln1": (L, HIDDEN), "wq": (L, Q_HEADS * HEAD_DIM, HIDDEN), "wk": (L, KV_HEADS * HEAD_DIM, HIDDEN),
        "wv": (L, KV_HEADS * HEAD_DIM, HIDDEN), "qn": (L, HEAD_DIM), "kn": (L, HEAD_DIM),
        "wo": (L, HIDDEN, Q_HEADS * HEAD_DIM), "ln2": (L, HIDDEN), "wg": (L, INTER, HIDDEN),
        "wu": (L, INTER, HIDDEN), "wd": (L, HIDDEN, INTER), "fnorm": (HIDDEN,), "embed": (V, HIDDEN),
    }


# ----------------------------------------------------------------------------- inputs

def synthetic(seed: int = 0, shape: Shape = Shape(), context: int = 128) -> dict:
    """Seeded inputs with the distribution of the reference's `weights.synthetic`
    (qwen3mk/weights.py:101-124), drawn in the same order from one CPU generator, so that
    with the default shape the tensors equal the reference's bit for bit."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    shp = weight_shapes(shape)

    def randn(*s):
        return torch.randn(s, generator=gen)

    def mat(name, fan_in):
        return (randn(*shp[name]) * fan_in ** -0.5).to(torch.bfloat16)

    def gain(name):
        return (1 + 0.1 * randn(*shp[name])).to(torch.bfloat16)

    out = {"token": torch.randint(shape.vocab, (), generator=gen, dtype=torch.int64)}
    out["ln1"] = gain("ln1")
    out["wq"] = mat("wq", 1024)
    out["wk"] = mat("wk", 1024)
    out["wv"] = mat("wv", 1024)
    out["qn"] = gain("qn")
    out["kn"] = gain("kn")
    out["wo"] = mat("wo", 2048)
    out["ln2"] = gain("ln2")
    out["wg"] = mat("wg", 1024)
    out["wu"] = mat("wu", 1024)
    out["wd"] = mat("wd", 3072)
    out["fnorm"] = gain("fnorm")
    out["embed"] = (randn(shape.vocab, HIDDEN) * 0.02).to(torch.bfloat16)
    out["kcache"] = (randn(shape.layers, context, KV_HEADS, HEAD_DIM) * 0.1).to(torch.bfloat16)
    out["vcache"] = (randn(shape.layers, context, KV_HEADS, HEAD_DIM) * 0.1).to(torch.bfloat16)
    return out


def baseline_init(seed: int = 0, shape: Shape = Shape()) -> dict:
    """The benchmark's weight distribution: every matrix (embedding included) bf16 N(0, 0.02),
    every RMSNorm gain exactly 1.  Returns the 13 weights only; the KV cache comes from prefill."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    out = {}
    for name, s in weight_shapes(shape).items():
        if name in ("ln1", "ln2", "qn", "kn", "fnorm"):
            out[name] = torch.ones(s, dtype=torch.bfloat16)
        else:
            out[name] = (torch.randn(s, generator=gen) * 0.02).to(torch.bfloat16)
    return out


def to_fp32(inputs: dict) -> dict:
    """The 13 weights widened to fp32 (qwen3mk/reference.py:39-41)."""
    return {n: inputs[n].float() for n in WEIGHT_NAMES}


# ----------------------------------------------------------------------------- pieces

def rms_norm(x: torch.Tensor, gain: torch.Tensor) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps), then * gain; fp32 throughout (reference.py:20-23)."""
    x = x.float()
    return (x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + EPS)) * gain.float()


def rope_cos_sin(positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """cos, sin [n, 128] fp32 for integer positions; angles in fp64, the 64 frequencies repeated
    twice along the last axis (Hugging Face layout; reference.py:26-31)."""
    inv_freq = ROPE_THETA ** (-torch.arange(0, HEAD_DIM, 2, dtype=torch.float64) / HEAD_DIM)
    ang = positions.to(torch.float64)[:, None] * inv_freq[None, :]
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos().float(), ang.sin().float()


def rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin with rotate_half(x) = [-x[64:], x[:64]] (reference.py:34-36,69-70)."""
    half = HEAD_DIM // 2
    swapped = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + swapped * sin


def _attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """q [QH, D]; k, v [S, KVH, D] -> [QH, D].  GQA: q-head h reads kv-head h // 2 (reference.py:90-97)."""
    groups = Q_HEADS // KV_HEADS
    kk = k.repeat_interleave(groups, dim=1).permute(1, 0, 2)   # [QH, S, D]
    vv = v.repeat_interleave(groups, dim=1).permute(1, 0, 2)
    scores = torch.einsum("hd,hsd->hs", q, kk) * HEAD_DIM ** -0.5
    probs = torch.softmax(scores, dim=-1, dtype=torch.float32)
    return torch.einsum("hs,hsd->hd", probs, vv)


# ----------------------------------------------------------------------------- decode

@torch.no_grad()
def decode_step(w: dict, token, kcache: torch.Tensor, vcache: torch.Tensor, pos: int | None = None,
                trace: dict | None = None) -> dict:
    """One batch-1 decode step at position `pos` (default: the cache length).

    w: fp32 weights.  kcache, vcache: [L, >=pos, 8, 128], any float dtype; slots [0, pos) are attended.
    Returns logits [V] fp32, next_token (int64 scalar), k_write and v_write [L, 8, 128] fp32
    (reference.py:44-87).  `trace`, when given, receives per-layer intermediates for debugging."""
    L = w["wq"].shape[0]
    if pos is None:
        pos = kcache.shape[1]
    cos, sin = rope_cos_sin(torch.tensor([pos]))
    x = w["embed"][int(token)].float().clone()                 # [H]
    ks, vs = [], []
    for l in range(L):
        xn = rms_norm(x, w["ln1"][l])
        q = (w["wq"][l] @ xn).view(Q_HEADS, HEAD_DIM)
        k = (w["wk"][l] @ xn).view(KV_HEADS, HEAD_DIM)
        v = (w["wv"][l] @ xn).view(KV_HEADS, HEAD_DIM)
        q = rotate(rms_norm(q, w["qn"][l]), cos, sin)
        k = rotate(rms_norm(k, w["kn"][l]), cos, sin)
        ks.append(k)
        vs.append(v)
        k_all = torch.cat([kcache[l, :pos].float(), k[None]], dim=0)   # the new row enters unrounded
        v_all = torch.cat([vcache[l, :pos].float(), v[None]], dim=0)
        o = _attend(q, k_all, v_all).reshape(Q_HEADS * HEAD_DIM)
        x = x + w["wo"][l] @ o
        if trace is not None:
            trace.setdefault("x_attn", []).append(x.clone())
        xn = rms_norm(x, w["ln2"][l])
        h = torch.nn.functional.silu(w["wg"][l] @ xn) * (w["wu"][l] @ xn)
        x = x + w["wd"][l] @ h
        if trace is not None:
            trace.setdefault("x_mlp", []).append(x.clone())
    logits = w["embed"] @ rms_norm(x, w["fnorm"])
    return {"logits": logits, "next_token": logits.argmax(), "k_write": torch.stack(ks), "v_write": torch.stack(vs)}


@torch.no_grad()
def greedy_decode(w: dict, token, kcache: torch.Tensor, vcache: torch.Tensor, steps: int,
                  forced_tokens=None, on_step=None, forced_rows=None) -> dict:
    """`steps` consecutive decode steps.  After each step the new K/V rows are appended to the cache
    ROUNDED TO bf16 (what a cache of the kernel's output dtype holds; qwen3mk/kernel.py:48-49), and the
    argmax token (or `forced_tokens[i]` when teacher-forcing) feeds the next step.

    `on_step(i, out)` is called with every step's full output (logits, k_write, v_write), so that a checker
    can gate each step without this loop keeping all logits.  `forced_rows[i] = (k_row, v_row)` (bf16
    [L, 8, 128]) replaces the rows this loop would append after step i: a checker replaying another
    implementation's stream hands over that implementation's rows, so that both see the same cache at every
    step (two correct implementations may round a row to different neighbouring bf16 values, after which
    their caches, and with them all later logits, differ at the 2^-8 level).  Returns tokens [steps] (the argmax of every
    step), margins [steps] (top-1 minus top-2 logit), the final caches (bf16) and the last step's logits."""
    kc = kcache.to(torch.bfloat16).clone()
    vc = vcache.to(torch.bfloat16).clone()
    toks, margins = [], []
    tok = int(token)
    out = None
    for i in range(steps):
        out = decode_step(w, tok, kc, vc)
        top2 = torch.topk(out["logits"], 2).values
        margins.append(float(top2[0] - top2[1]))
        toks.append(int(out["next_token"]))
        if on_step is not None:
            on_step(i, out)
        k_row, v_row = (out["k_write"], out["v_write"]) if forced_rows is None else forced_rows[i]
        kc = torch.cat([kc, k_row.to(torch.bfloat16)[:, None]], dim=1)
        vc = torch.cat([vc, v_row.to(torch.bfloat16)[:, None]], dim=1)
        tok = toks[-1] if forced_tokens is None else int(forced_tokens[i])
    return {"tokens": torch.tensor(toks, dtype=torch.int64), "margins": torch.tensor(margins),
            "kcache": kc, "vcache": vc, "logits": out["logits"] if out else None}


@torch.no_grad()
def decode_batch(w: dict, tokens, kcaches: list, vcaches: list) -> list:
    """Batched decode = one independent `decode_step` per sequence, each at its own position
    (the reference is batch 1: reference.py:52,57-58,63)."""
    return [decode_step(w, int(t), kc, vc) for t, kc, vc in zip(tokens, kcaches, vcaches)]


# ----------------------------------------------------------------------------- prefill

@torch.no_grad()
def prefill(w: dict, ids, return_all_logits: bool = False):
    """Causal fp32 forward over T = len(ids) positions (qwen3mk/prefill.py:46-81 with T free).

    Returns kcache, vcache (bf16 [L, T, 8, 128]; K after head-norm and RoPE) and the fp32 logits
    of the last position [V] (or of every position [T, V] when `return_all_logits`)."""
    L = w["wq"].shape[0]
    ids = torch.as_tensor(ids, dtype=torch.int64)
    T = ids.numel()
    cos, sin = rope_cos_sin(torch.arange(T))
    cos, sin = cos[:, None, :], sin[:, None, :]
    allowed = torch.ones(T, T, dtype=torch.bool).tril()
    groups = Q_HEADS // KV_HEADS
    x = w["embed"][ids].float()
    kout, vout = [], []
    for l in range(L):
        xn = rms_norm(x, w["ln1"][l])
        q = (xn @ w["wq"][l].T).view(T, Q_HEADS, HEAD_DIM)
        k = (xn @ w["wk"][l].T).view(T, KV_HEADS, HEAD_DIM)
        v = (xn @ w["wv"][l].T).view(T, KV_HEADS, HEAD_DIM)
        q = rotate(rms_norm(q, w["qn"][l]), cos, sin)
        k = rotate(rms_norm(k, w["kn"][l]), cos, sin)
        kout.append(k)
        vout.append(v)
        kk = k.repeat_interleave(groups, dim=1).permute(1, 0, 2)      # [QH, T, D]
        vv = v.repeat_interleave(groups, dim=1).permute(1, 0, 2)
        s = (q.permute(1, 0, 2) @ kk.transpose(-1, -2)) * HEAD_DIM ** -0.5
        s = s.masked_fill(~allowed[None], -math.inf)
        o = torch.softmax(s, dim=-1) @ vv                              # [QH, T, D]
        x = x + o.permute(1, 0, 2).reshape(T, Q_HEADS * HEAD_DIM) @ w["wo"][l].T
        xn = rms_norm(x, w["ln2"][l])
        x = x + (torch.nn.functional.silu(xn @ w["wg"][l].T) * (xn @ w["wu"][l].T)) @ w["wd"][l].T
    last = x if return_all_logits else x[-1:]
    logits = rms_norm(last, w["fnorm"]) @ w["embed"].T
    kc = torch.stack(kout).to(torch.bfloat16).contiguous()
    vc = torch.stack(vout).to(torch.bfloat16).contiguous()
    return kc, vc, (logits if return_all_logits else logits[0])


# ----------------------------------------------------------------------------- gates (run.py:37-54)

def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten().cpu(), b.double().flatten().cpu()
    return float((a - b).norm() / b.norm())


def bf16_ulps(a: torch.Tensor, ref: torch.Tensor) -> float:
    """Largest |a - ref| in bf16 ulps, the unit being the ulp of max(|ref|, rms(ref)) (run.py:42-50)."""
    a, ref = a.float().cpu(), ref.float().cpu()
    r = ref.abs().clamp_min(float(ref.pow(2).mean().sqrt()))
    ulp = torch.exp2(torch.floor(torch.log2(r)) - 7)
    return float(((a - ref).abs() / ulp).max())


def max_rel(a: torch.Tensor, ref: torch.Tensor) -> float:
    """max |a - ref| / max |ref|: the "within 2e-2 relative" bound of the benchmark spec."""
    a, ref = a.double().cpu(), ref.double().cpu()
    return float((a - ref).abs().max() / ref.abs().max())
