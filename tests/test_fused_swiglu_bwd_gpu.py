"""The SwiGLU adjoint inside the dgrad GEMM epilogue (EPI_SWIGLU_BWD) against the GEMM + streaming-kernel path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fused_swiglu_adjoint_matches_unfused_path():
    from oracle import inputs
    from swamla_b200 import functional
    from swamla_b200.layer import LatentMoELayer
    w = inputs.WORKLOADS["tiny_ragged"]
    params, buffers, x, dy = inputs.make_inputs(w)
    results = []
    for fused in (False, True):
        layer = LatentMoELayer(w.config())
        layer.load_state_dict({**params, **buffers}, strict=True)
        layer = layer.to("cuda:0").to(torch.bfloat16).train()
        xg = x.to("cuda:0").to(torch.bfloat16).requires_grad_(True)
        old = functional.FUSE_SWIGLU_BWD
        functional.FUSE_SWIGLU_BWD = fused
        try:
            y = layer(xg)
            y.backward(dy.to("cuda:0").to(torch.bfloat16))
            torch.cuda.synchronize()
        finally:
            functional.FUSE_SWIGLU_BWD = old
        results.append({"x": xg.grad, **{k: p.grad for k, p in layer.named_parameters()}})
    a, b = results
    for k in a:
        # same bf16 rounding points; only the approximate exp / reciprocal of the sigmoid differ
        err = (a[k].float() - b[k].float()).abs().max().item()
        scale = a[k].float().abs().max().item()
        assert err <= 2e-2 * scale, (k, err, scale)
        rel = ((a[k].float() - b[k].float()).norm() / a[k].float().norm()).item()
        assert rel <= 2e-3, (k, rel)
