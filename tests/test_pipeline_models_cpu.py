"""The CPU models of the bf16 / e4m3 pipelines (oracle/bf16_pipeline.py) against the fp32 oracle: the models are what the
GPU results are compared with to about one ulp, so they must themselves sit inside the tolerance of the path."""
import pytest
import torch

from oracle import bf16_pipeline, inputs, latent_moe_ref as R


def _oracle(w, params, buffers, x, dy, aux_grad, sel=None):
    rb = inputs.round_to_bf16
    pr = {k: rb(v) for k, v in params.items()}
    return R.layer_forward_backward(pr, buffers, rb(x), rb(dy), w.K, z_loss_coef=w.router_z_loss_coef, aux_grad=aux_grad,
                                    sel_override=sel)


@pytest.mark.parametrize("name", ["tiny", "tiny_ragged", "tiny_moe", "tiny_moe_ragged"])
@pytest.mark.parametrize("aux_grad", [0.0, 2.0])
def test_bf16_pipeline_model_is_within_tolerance_of_fp32_oracle(name, aux_grad):
    w = inputs.WORKLOADS[name]
    params, buffers, x, dy = inputs.make_inputs(w)
    out, grads = _oracle(w, params, buffers, x, dy, aux_grad)
    model, model_grads = bf16_pipeline.forward_backward(params, buffers, x, dy, w.K, w.router_z_loss_coef, aux_grad=aux_grad,
                                                        sel_override=out["sel"])
    assert torch.equal(model["sel"], out["sel"]) and torch.equal(model["perm"], out["perm"])
    for k in ("y", "x_latent", "h1", "hidden", "y_sorted", "routed", "h1_s", "hidden_s"):
        ok, rep = R.within_tolerance(model[k].reshape(out[k].shape), out[k], 2e-2)
        assert ok, (k, rep)
    for k, ref in grads.items():
        ok, rep = R.within_tolerance(model_grads[k], ref, 2e-2)
        assert ok, (k, rep)


def test_e4m3_pipeline_model_is_within_fp8_tolerance_for_outputs():
    w = inputs.WORKLOADS["tiny_fp8"]
    params, buffers, x, dy = inputs.make_inputs(w)
    out, grads = _oracle(w, params, buffers, x, dy, 0.0)
    model, model_grads = bf16_pipeline.forward_backward(params, buffers, x, dy, w.K, w.router_z_loss_coef,
                                                        sel_override=out["sel"], fp8=True)
    for name, a, b in (("y", model["y"], out["y"]), ("dx", model_grads["x"], grads["x"])):
        ok, rep = R.within_tolerance(a, b, 6e-2)
        assert ok, (name, rep)
    # quantisation really happens: the e4m3 model differs from the bf16 model
    bf, _ = bf16_pipeline.forward_backward(params, buffers, x, dy, w.K, w.router_z_loss_coef, sel_override=out["sel"])
    assert (bf["y_sorted"] - model["y_sorted"]).abs().max().item() > 0


def test_fake_quantisation_matches_the_recipe():
    g = torch.Generator().manual_seed(0)
    t = torch.randn(64, 64, generator=g) * 3
    q = bf16_pipeline.fq(t)
    amax = t.abs().max()
    ref = ((t * (448.0 / amax)).clamp(-448, 448).to(torch.float8_e4m3fn).float()) * (amax / 448.0)
    assert torch.equal(q, ref)
    assert torch.equal(bf16_pipeline.fq(torch.zeros(4, 4)), torch.zeros(4, 4))          # amax = 0: unchanged
    assert (q - t).abs().max().item() <= amax.item() * 2.0 ** -4                         # e4m3: 3 mantissa bits
