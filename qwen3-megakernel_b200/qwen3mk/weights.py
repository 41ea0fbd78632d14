"""Engine inputs: real Qwen3-0.6B weights from a Hugging Face checkpoint, or seeded random ones.

Same surface as the reference's module (qwen3mk/weights.py:34-124): `load_hf`, `synthetic`,
`resolve_model_dir`, `WEIGHT_NAMES`, `STATE_NAMES`, `MODEL_ID`; every function returns a dict keyed by
the kernel input names.  `baseline_init` adds the benchmark's distribution (N(0, 0.02) matrices,
unit RMSNorm gains).

Checkpoint tensor -> input name (i = layer, stacked over the layers):
    model.embed_tokens.weight                          embed  (tied LM head)
    model.layers.i.input_layernorm.weight              ln1
    model.layers.i.self_attn.{q,k,v,o}_proj.weight     wq wk wv wo
    model.layers.i.self_attn.{q,k}_norm.weight         qn kn
    model.layers.i.post_attention_layernorm.weight     ln2
    model.layers.i.mlp.{gate,up,down}_proj.weight      wg wu wd
    model.norm.weight                                  fnorm
"""
from __future__ import annotations

import json
import os
from pathlib import Path

import torch

from .kernel import CONTEXT, HEAD_DIM, HIDDEN, INTER, KV_HEADS, LAYERS, Q_HEADS, VOCAB, input_specs

MODEL_ID = "Qwen/Qwen3-0.6B"
WEIGHT_NAMES = ("ln1", "wq", "wk", "wv", "qn", "kn", "wo", "ln2", "wg", "wu", "wd", "fnorm", "embed")
STATE_NAMES = ("token", "kcache", "vcache")

_PER_LAYER = (
    ("ln1", "input_layernorm.weight"), ("wq", "self_attn.q_proj.weight"), ("wk", "self_attn.k_proj.weight"),
    ("wv", "self_attn.v_proj.weight"), ("qn", "self_attn.q_norm.weight"), ("kn", "self_attn.k_norm.weight"),
    ("wo", "self_attn.o_proj.weight"), ("ln2", "post_attention_layernorm.weight"),
    ("wg", "mlp.gate_proj.weight"), ("wu", "mlp.up_proj.weight"), ("wd", "mlp.down_proj.weight"),
)
_REQUIRED_CONFIG = (("hidden_size", HIDDEN), ("num_hidden_layers", LAYERS), ("num_attention_heads", Q_HEADS),
                    ("num_key_value_heads", KV_HEADS), ("head_dim", HEAD_DIM), ("intermediate_size", INTER),
                    ("vocab_size", VOCAB), ("rope_theta", 1e6))


def resolve_model_dir(model_id_or_path: str = MODEL_ID) -> Path:
    """A local directory as is; otherwise the Hugging Face cache snapshot of a model id (honours HF_HOME and
    HF_HUB_OFFLINE)."""
    if os.path.isdir(model_id_or_path):
        return Path(model_id_or_path)
    from huggingface_hub import snapshot_download

    return Path(snapshot_download(model_id_or_path, allow_patterns=["*.safetensors", "*.json", "merges.txt", "vocab.json"]))


def load_hf(model_id_or_path: str = MODEL_ID, device="cpu", *, layers: int | None = None, vocab: int | None = None) -> dict:
    """The 13 weight tensors of a Qwen3-0.6B checkpoint: bf16, [out, in] layout, stacked over layers, on `device`.
    Raises ValueError when config.json does not describe the architecture the kernels are built for.  `layers` and
    `vocab` override the two extents the engine takes at run time (a cut-down checkpoint for tests); the per-head
    geometry always has to match."""
    from safetensors import safe_open

    root = resolve_model_dir(model_id_or_path)
    config = json.loads((root / "config.json").read_text())
    want_layers, want_vocab = LAYERS if layers is None else int(layers), VOCAB if vocab is None else int(vocab)
    for key, want in _REQUIRED_CONFIG:
        want = {"num_hidden_layers": want_layers, "vocab_size": want_vocab}.get(key, want)
        if config.get(key) != want:
            raise ValueError(f"config.json {key}={config.get(key)!r}, the kernel needs {want!r}")
    shards = sorted(root.glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no .safetensors file in {root}")
    where = {}
    for shard in shards:
        f = safe_open(str(shard), framework="pt", device="cpu")
        where.update({k: f for k in f.keys()})

    def tensor(key: str) -> torch.Tensor:
        if key not in where:
            raise KeyError(f"{key} is in none of the {len(shards)} .safetensors files of {root}")
        return where[key].get_tensor(key)

    specs = input_specs(want_layers, want_vocab)
    raw = {name: torch.stack([tensor(f"model.layers.{i}.{suffix}") for i in range(want_layers)]) for name, suffix in _PER_LAYER}
    raw["fnorm"] = tensor("model.norm.weight")
    raw["embed"] = tensor("model.embed_tokens.weight")
    out = {}
    for name in WEIGHT_NAMES:
        shape, dtype = specs[name]
        if tuple(raw[name].shape) != shape:
            raise ValueError(f"{name}: shape {tuple(raw[name].shape)}, expected {shape}")
        out[name] = raw[name].to(device=device, dtype=dtype).contiguous()
    return out


def synthetic(seed: int = 0, device="cuda", *, layers: int = LAYERS, vocab: int = VOCAB, context: int = CONTEXT) -> dict:
    """All 16 inputs, random: matrices N(0,1) * fan_in^-0.5, norm gains 1 + 0.1 N(0,1), embedding 0.02 N(0,1),
    KV cache 0.1 N(0,1), a random token; one generator on `device`, drawn in input order
    (the distribution of qwen3mk/weights.py:101-124)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    specs = input_specs(layers, vocab, context)
    fan_in = {"wq": HIDDEN, "wk": HIDDEN, "wv": HIDDEN, "wo": Q_HEADS * HEAD_DIM, "wg": HIDDEN, "wu": HIDDEN, "wd": INTER}
    out = {"token": torch.randint(vocab, (), generator=gen, device=device, dtype=torch.int64)}
    for name in WEIGHT_NAMES + ("kcache", "vcache"):
        z = torch.randn(specs[name][0], generator=gen, device=device)
        if name in fan_in:
            z = z * fan_in[name] ** -0.5
        elif name == "embed":
            z = z * 0.02
        elif name in ("kcache", "vcache"):
            z = z * 0.1
        else:
            z = 1 + 0.1 * z
        out[name] = z.to(torch.bfloat16)
    return out


def baseline_init(seed: int = 0, device="cuda", *, layers: int = LAYERS, vocab: int = VOCAB) -> dict:
    """The 13 weights with the benchmark's distribution: every matrix (embedding included) bf16 N(0, 0.02),
    every RMSNorm gain 1.  Drawn on the CPU so that a CPU checker can rebuild the same tensors."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    specs = input_specs(layers, vocab)
    out = {}
    for name in WEIGHT_NAMES:
        shape = specs[name][0]
        if name in ("ln1", "ln2", "qn", "kn", "fnorm"):
            out[name] = torch.ones(shape, dtype=torch.bfloat16, device=device)
        else:
            out[name] = (torch.randn(shape, generator=gen) * 0.02).to(torch.bfloat16).to(device)
    return out
