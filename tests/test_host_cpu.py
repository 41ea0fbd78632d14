"""Host-side logic and the C-ABI library's surface.  No GPU, no compute calls."""
from __future__ import annotations

import ctypes
import json
import re

import pytest
import torch

from conftest import ROOT


def test_library_exports_every_declared_symbol():
    from qwen3mk import _cabi

    header = (ROOT / "include" / "q3mk.h").read_text()
    declared = set(re.findall(r"\b(q3_[a-z_0-9]+)\s*\(", header))
    assert declared, "no declarations found in include/q3mk.h"
    lib = _cabi.load()
    for name in sorted(declared):
        assert hasattr(lib, name), f"libq3mk.so does not export {name}"
    assert declared == set(_cabi.SYMBOLS)
    assert lib.q3_version().decode().endswith("sm_100a")


def test_struct_layouts_match_header():
    from qwen3mk import _cabi

    assert ctypes.sizeof(_cabi.Config) == 24
    assert ctypes.sizeof(_cabi.Weights) == 13 * 8
    assert ctypes.sizeof(_cabi.DecodeArgs) == 16 + 9 * 8
    assert _cabi.DecodeArgs.token.offset == 16
    assert ctypes.sizeof(_cabi.PrefillArgs) == 8 + 5 * 8


def test_create_rejects_bad_config_before_touching_cuda():
    from qwen3mk import _cabi

    lib = _cabi.load()
    h = ctypes.c_void_p()
    for bad in (_cabi.Config(0, 100, 1, 0, 0, 0), _cabi.Config(2, 0, 1, 0, 0, 0), _cabi.Config(2, 100, 0, 0, 0, 0)):
        rc = lib.q3_create(0, ctypes.byref(bad), ctypes.byref(h))
        assert rc == _cabi.ERR_INVALID and not h.value
        assert b"out of range" in lib.q3_last_error(None)
    with pytest.raises(ValueError):
        _cabi.check(lib, None, _cabi.ERR_INVALID, "q3_create")
    # null handles are rejected, not dereferenced
    assert lib.q3_decode(None, None, None) == _cabi.ERR_INVALID
    assert lib.q3_prefill(None, None, None) == _cabi.ERR_INVALID
    assert lib.q3_set_weights(None, None) == _cabi.ERR_INVALID
    lib.q3_destroy(None)


@pytest.mark.skipif(torch.cuda.is_available(), reason="only meaningful without a GPU")
def test_engine_fails_loudly_without_gpu():
    from qwen3mk import Megakernel

    with pytest.raises(RuntimeError, match="no CPU path"):
        Megakernel()


def test_rope_tables_match_oracle(oracle):
    from qwen3mk import kernel

    t = kernel.rope_table("cpu")
    assert tuple(t.shape) == (128,) and t.dtype == torch.float32
    rows = kernel.rope_rows(300, "cpu")
    assert torch.equal(rows[128], t)
    cos, sin = oracle.rope_cos_sin(torch.arange(300))
    assert torch.equal(rows[:, :64], cos[:, :64]) and torch.equal(rows[:, 64:], sin[:, :64])
    assert torch.equal(cos[:, :64], cos[:, 64:])


def test_specs_and_input_order():
    from qwen3mk import INPUT_ORDER, kernel

    assert INPUT_ORDER == ("token", "ln1", "wq", "wk", "wv", "qn", "kn", "wo", "ln2", "wg", "wu", "wd", "fnorm",
                           "embed", "kcache", "vcache")
    assert kernel.INPUT_SPECS["kcache"] == ((28, 128, 8, 128), torch.bfloat16)
    assert kernel.OUTPUT_SPECS["logits"] == ((151936,), torch.float32)
    assert kernel.input_specs(2, 512, 9)["vcache"][0] == (2, 9, 8, 128)


def test_seqtable_validation():
    from qwen3mk.kernel import SeqTable

    k = torch.zeros(2, 10, 8, 128, dtype=torch.bfloat16)
    s = SeqTable([k, k.clone()], [k.clone(), k.clone()], [3, 10])
    assert s.batch == 2 and s.max_len == 10 and s.len.tolist() == [3, 10]
    assert s.stride.tolist() == [10 * 1024] * 2 and s.seq_k[0].item() == k.data_ptr()
    with pytest.raises(ValueError):
        SeqTable([k], [k.float()])
    with pytest.raises(ValueError):
        SeqTable([k], [k], [11])
    with pytest.raises(ValueError):
        SeqTable([k.transpose(0, 1)], [k.transpose(0, 1)])
    with pytest.raises(ValueError):
        SeqTable([], [])


class FakeTokenizer:
    def __call__(self, prompt, add_special_tokens=False):
        return {"input_ids": [int(x) for x in prompt.split()]}


def test_build_prefix_rules():
    from qwen3mk import prefill

    tok = FakeTokenizer()
    ids, nxt, info = prefill.build_prefix(tok, " ".join(str(i) for i in range(173)))
    assert ids == list(range(128)) and nxt == 128 and info == {"prompt_tokens": 173, "cut": 44}
    ids, nxt, info = prefill.build_prefix(tok, " ".join(str(i) for i in range(128)))
    assert len(ids) == 128 and nxt is None and info["cut"] == 0
    with pytest.raises(ValueError, match="at least 128 tokens"):
        prefill.build_prefix(tok, "1 2 3")


def test_load_hf_rejects_other_architectures(tmp_path):
    from qwen3mk import weights

    cfg = {"hidden_size": 1024, "num_hidden_layers": 12, "num_attention_heads": 16, "num_key_value_heads": 8,
           "head_dim": 128, "intermediate_size": 3072, "vocab_size": 151936, "rope_theta": 1e6}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(ValueError, match="num_hidden_layers"):
        weights.load_hf(str(tmp_path))
    cfg["num_hidden_layers"] = 28
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(FileNotFoundError):
        weights.load_hf(str(tmp_path))
    assert weights.resolve_model_dir(str(tmp_path)) == tmp_path


def test_synthetic_generators_match_oracle(oracle):
    from qwen3mk import weights

    a = weights.synthetic(5, "cpu", layers=1, vocab=300, context=6)
    b = oracle.synthetic(5, oracle.Shape(1, 300), context=6)
    assert all(torch.equal(a[k], b[k]) for k in a)
    a = weights.baseline_init(5, "cpu", layers=1, vocab=300)
    b = oracle.baseline_init(5, oracle.Shape(1, 300))
    assert set(a) == set(weights.WEIGHT_NAMES) and all(torch.equal(a[k], b[k]) for k in a)
    assert float(a["ln1"].float().min()) == 1.0 and abs(float(a["wq"].float().std()) - 0.02) < 2e-3


def test_oracle_batch_and_greedy_consistency(oracle):
    """decode_batch == independent steps; greedy_decode step i == decode_step on the grown cache."""
    shp = oracle.Shape(layers=1, vocab=256)
    inp = oracle.synthetic(11, shp, context=5)
    w = oracle.to_fp32(inp)
    g = oracle.greedy_decode(w, inp["token"], inp["kcache"], inp["vcache"], steps=3)
    assert g["kcache"].shape[1] == 8 and g["tokens"].shape == (3,)
    again = oracle.decode_step(w, int(g["tokens"][1]), g["kcache"][:, :7], g["vcache"][:, :7])
    assert int(again["next_token"]) == int(g["tokens"][2])
    outs = oracle.decode_batch(w, [3, 4], [inp["kcache"], inp["kcache"][:, :2]], [inp["vcache"], inp["vcache"][:, :2]])
    solo = oracle.decode_step(w, 4, inp["kcache"][:, :2], inp["vcache"][:, :2])
    assert torch.equal(outs[1]["logits"], solo["logits"])
    # prefill's last-position logits == decoding the last token against the fp32 cache of the rest
    ids = [5, 9, 200, 31]
    kc, vc, last = oracle.prefill(w, ids)
    assert tuple(kc.shape) == (1, 4, 8, 128)
    alll = oracle.prefill(w, ids, return_all_logits=True)[2]
    assert torch.allclose(alll[-1], last, rtol=1e-5, atol=1e-6)


def test_load_hf_reads_a_sharded_checkpoint_end_to_end(tmp_path):
    """A 2-layer, 512-word checkpoint in the Hugging Face layout, split over two .safetensors files and stored as
    fp32: names, stacking over layers, dtype and shapes must come out as the engine's 13 inputs."""
    import json

    import torch
    from safetensors.torch import save_file

    from qwen3mk import weights
    from qwen3mk.kernel import input_specs

    L, V = 2, 512
    g = torch.Generator().manual_seed(0)
    specs = input_specs(L, V)
    want = {n: torch.randn(specs[n][0], generator=g).to(torch.bfloat16) for n in weights.WEIGHT_NAMES}
    shard0, shard1 = {}, {}
    for name, suffix in weights._PER_LAYER:
        for i in range(L):
            (shard0 if i == 0 else shard1)[f"model.layers.{i}.{suffix}"] = want[name][i].float().contiguous()
    shard1["model.norm.weight"] = want["fnorm"].float()
    shard0["model.embed_tokens.weight"] = want["embed"].float()
    shard1["lm_head.weight"] = want["embed"].float()           # tied head stored twice, as some exports do: ignored
    save_file(shard0, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file(shard1, str(tmp_path / "model-00002-of-00002.safetensors"))
    cfg = {"hidden_size": 1024, "num_hidden_layers": L, "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128,
           "intermediate_size": 3072, "vocab_size": V, "rope_theta": 1e6}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    got = weights.load_hf(str(tmp_path), layers=L, vocab=V)
    assert tuple(got) == weights.WEIGHT_NAMES
    for n in weights.WEIGHT_NAMES:
        assert got[n].dtype == torch.bfloat16 and got[n].is_contiguous() and tuple(got[n].shape) == specs[n][0], n
        assert torch.equal(got[n], want[n]), n
    # the full-size extents are still the default
    import pytest
    with pytest.raises(ValueError, match="num_hidden_layers"):
        weights.load_hf(str(tmp_path))
    # a missing tensor is named
    (tmp_path / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(KeyError, match="model.layers.1"):
        weights.load_hf(str(tmp_path), layers=L, vocab=V)
