"""The tensor-core linear op (tcgen05 / TMEM / TMA GEMM) against a plain fp32 PyTorch product of the same
bf16 weights.  Tolerances: one bf16 plane rounds the activations to bf16 (relative 2^-8 per element, about
4e-3 on the result), three planes are exact to fp32 up to summation order (3e-5)."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def linear_tc(w, x, nsplit, resid=None):
    from qwen3mk import _cabi

    lib = _cabi.load()
    n_rows, K = w.shape
    n_tok = x.shape[0]
    tile = 32 if n_tok <= 32 else (64 if n_tok <= 64 else 128)
    rows = (n_tok + tile - 1) // tile * tile
    planes = torch.empty(nsplit * rows * K, dtype=torch.bfloat16, device="cuda")
    out = torch.full((n_tok, n_rows), float("nan"), dtype=torch.float32, device="cuda") if resid is None else resid.clone()
    rc = lib.q3_linear_tc(w.data_ptr(), x.data_ptr(), out.data_ptr(), None if resid is None else out.data_ptr(), n_rows, n_tok, K, nsplit,
                          planes.data_ptr(), planes.numel() * 2, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.q3_last_error(None)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("n_tok,n_rows,K", [(32, 128, 128), (17, 256, 1024), (64, 1024, 3072), (100, 2048, 1024), (384, 1024, 2048), (2048, 4096, 1024)])
@pytest.mark.parametrize("nsplit", [1, 3])
def test_linear_tc_matches_fp32_product(n_tok, n_rows, K, nsplit):
    g = torch.Generator(device="cuda").manual_seed(n_tok + n_rows + K)
    w = (torch.randn(n_rows, K, generator=g, device="cuda") * K ** -0.5).to(torch.bfloat16)
    x = torch.randn(n_tok, K, generator=g, device="cuda")
    ref = x.double() @ w.double().T
    out = linear_tc(w, x, nsplit)
    err = float((out.double() - ref).norm() / ref.norm())
    assert err <= (3e-5 if nsplit == 3 else 6e-3), err
    assert torch.isfinite(out).all()


def test_linear_tc_residual_and_rejections():
    from qwen3mk import _cabi

    g = torch.Generator(device="cuda").manual_seed(1)
    w = (torch.randn(1024, 2048, generator=g, device="cuda") / 45).to(torch.bfloat16)
    x = torch.randn(40, 2048, generator=g, device="cuda")
    r = torch.randn(40, 1024, generator=g, device="cuda")
    out = linear_tc(w, x, 3, resid=r)
    ref = r.double() + x.double() @ w.double().T
    assert float((out.double() - ref).norm() / ref.norm()) <= 1e-5
    lib = _cabi.load()
    assert lib.q3_linear_tc(1, 1, 1, None, 100, 4, 128, 1, 1, 1 << 30, None) == _cabi.ERR_INVALID     # rows not a multiple of 128
    assert lib.q3_linear_tc(1, 1, 1, None, 128, 4, 128, 4, 1, 1 << 30, None) == _cabi.ERR_INVALID     # too many planes
    assert lib.q3_linear_tc(1, 1, 1, None, 128, 4, 128, 1, 1, 16, None) == _cabi.ERR_INVALID          # planes buffer too small
