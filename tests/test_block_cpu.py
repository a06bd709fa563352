"""The oracle of the block-level steps (RMSNorm, residual) against the reference's own class and its frozen outputs."""
import os
import sys

import pytest
import torch

from oracle import block_ref, ref_shim
from conftest import golden_path


def _inputs(fx):
    g = torch.Generator().manual_seed(fx["seed"])
    x = torch.randn(fx["T"], fx["D"], generator=g)
    w = 1.0 + 0.1 * torch.randn(fx["D"], generator=g)
    dy = torch.randn(fx["T"], fx["D"], generator=g)
    return x, w, dy


def test_rmsnorm_oracle_matches_reference_fixture():
    fx = torch.load(golden_path("rmsnorm"), weights_only=False)
    x, w, dy = _inputs(fx)
    assert abs(x.double().pow(2).sum().sqrt().item() - fx["x_l2"]) < 1e-9          # seeded inputs reproduce
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y = block_ref.rmsnorm(xr, wr, fx["eps"])
    (y * dy).sum().backward()
    torch.testing.assert_close(y.detach(), fx["y"], rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(xr.grad, fx["dx"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(wr.grad, fx["dw"], rtol=1e-5, atol=1e-5)


@pytest.mark.skipif(not ref_shim.available(), reason="reference source tree not present")
def test_rmsnorm_oracle_matches_live_reference_class():
    models_dir = os.path.join(ref_shim.REFERENCE_ROOT, "models")
    if models_dir not in sys.path:
        sys.path.insert(0, models_dir)
    from normalization import RMSNorm
    g = torch.Generator().manual_seed(5)
    x = torch.randn(3, 19, 128, generator=g)
    norm = RMSNorm(128, eps=1e-5)
    with torch.no_grad():
        norm.weight.copy_(torch.rand(128, generator=g) + 0.5)
    torch.testing.assert_close(block_ref.rmsnorm(x, norm.weight.detach(), 1e-5), norm(x).detach(), rtol=1e-6, atol=1e-6)


def test_residual_block_oracle_composes_norm_ffn_and_add():
    g = torch.Generator().manual_seed(6)
    x, w = torch.randn(2, 5, 64, generator=g), torch.rand(64, generator=g)
    lin = torch.randn(64, 64, generator=g)
    out = block_ref.ffn_block_residual(x, w, 1e-6, lambda t: t @ lin)
    torch.testing.assert_close(out, x + block_ref.rmsnorm(x, w) @ lin)
