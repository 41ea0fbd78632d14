"""The CPU oracle against golden vectors produced by the reference's own Python code
(tests/golden/make_golden.py).  No GPU.  These tests are what pins the oracle."""
from __future__ import annotations

import hashlib

import numpy as np
import pytest
import torch

from conftest import GOLDEN

LOGIT_STRIDE = 37
TOL = 2e-5  # fp32 restatement vs fp32 reference: same math, different op order


def sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def check_inputs(fx, inputs):
    assert int(fx["in_token"]) == int(inputs["token"])
    assert str(fx["in_sha_kcache"]) == sha(inputs["kcache"])
    if "in_sha_ln1" in fx:
        assert str(fx["in_sha_ln1"]) == sha(inputs["ln1"])
    assert float(fx["in_sum_wq"]) == inputs["wq"].double().sum().item()


def close(a, b, tol=TOL):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return np.abs(a - b).max() <= tol * max(np.abs(b).max(), 1e-30)


def check_step(fx, out):
    assert int(out["next_token"]) == int(fx["next_token"])
    logits = out["logits"]
    assert close(logits[::LOGIT_STRIDE].numpy(), fx["logits_sample"])
    assert close(logits[torch.as_tensor(fx["logits_top_idx"])].numpy(), fx["logits_top_val"])
    assert abs(float(logits.double().norm()) - float(fx["logits_norm"])) <= TOL * float(fx["logits_norm"])
    assert close(out["k_write"].numpy(), fx["k_write"])
    assert close(out["v_write"].numpy(), fx["v_write"])


def test_small_model_matches_reference(oracle):
    fx = np.load(GOLDEN / "decode_small_seed7_pos40.npz")
    inp = oracle.synthetic(7, oracle.Shape(layers=2, vocab=4096), context=40)
    check_inputs(fx, inp)
    out = oracle.decode_step(oracle.to_fp32(inp), inp["token"], inp["kcache"], inp["vcache"])
    assert int(out["next_token"]) == int(fx["next_token"])
    assert close(out["logits"].numpy(), fx["logits"])
    assert close(out["k_write"].numpy(), fx["k_write"])
    assert close(out["v_write"].numpy(), fx["v_write"])


@pytest.mark.parametrize("seed", [0, 1])
def test_full_decode_pos128_matches_reference(oracle, synth_full, seed):
    fx = np.load(GOLDEN / f"decode_seed{seed}_pos128.npz")
    inp = synth_full(seed)
    check_inputs(fx, inp)
    out = oracle.decode_step(oracle.to_fp32(inp), inp["token"], inp["kcache"], inp["vcache"])
    check_step(fx, out)


def test_full_decode_pos129_and_prefill_match_reference(oracle, synth_full):
    inp = synth_full(0)
    w = oracle.to_fp32(inp)
    # position 129: the greedy loop's second step (cache extended with bf16-rounded rows)
    fx = np.load(GOLDEN / "decode_seed0_pos129.npz")
    check_inputs(fx, inp)
    g = oracle.greedy_decode(w, inp["token"], inp["kcache"], inp["vcache"], steps=2)
    assert int(g["tokens"][0]) == int(fx["in_step_token"])
    assert g["kcache"].shape[1] == 130
    out = oracle.decode_step(w, int(g["tokens"][0]), g["kcache"][:, :129], g["vcache"][:, :129])
    check_step(fx, out)
    assert int(g["tokens"][1]) == int(fx["next_token"])
    # prefill over 128 ids
    fp = np.load(GOLDEN / "prefill_seed0_t128.npz")
    kc, vc, last = oracle.prefill(w, fp["ids"].tolist())
    assert kc.dtype == torch.bfloat16 and tuple(kc.shape) == (28, 128, 8, 128)
    # bf16 outputs: allow one bf16 ulp where fp32 rounding noise straddles a rounding boundary
    for got, name in ((kc, "k"), (vc, "v")):
        ref_s = fp[f"{name}_sample"]
        got_s = got[:, ::16, :, ::4].float().numpy()
        assert np.abs(got_s - ref_s).max() <= 2 ** -7 * np.abs(ref_s).max()
        assert (got_s != ref_s).mean() < 1e-2
        assert np.abs(got[:, -1].float().numpy() - fp[f"{name}_last"]).max() <= 2 ** -7 * np.abs(fp[f"{name}_last"]).max()
    assert close(last[::LOGIT_STRIDE].numpy(), fp["logits_sample"], 1e-4)
    assert int(last.argmax()) == int(fp["logits_top_idx"][0])
