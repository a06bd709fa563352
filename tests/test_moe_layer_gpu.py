"""The non-latent MoELayer (models/moe.py:294-559) on the GPU against the CPU oracle and against golden fixtures
generated from the reference class itself."""
import pytest
import torch

from oracle import inputs, latent_moe_ref as R
from conftest import golden_path

pytestmark = pytest.mark.gpu
RTOL_BF16 = 2e-2      # outputs and gradients vs the fp32 reference


def build_layer(w, params, buffers, dtype):
    from swamla_b200.layer import create_moe_layer
    layer = create_moe_layer(w.config())                 # use_latent_moe=False -> MoELayer
    assert type(layer).__name__ == "MoELayer"
    state = dict(params)
    state.update(buffers)
    layer.load_state_dict(state, strict=True)
    return layer.to("cuda:0").to(dtype) if dtype != torch.float32 else layer.to("cuda:0")


def assert_close(name, test, ref, rtol=RTOL_BF16):
    ok, rep = R.within_tolerance(test.detach().float().cpu(), ref, rtol)
    assert ok, f"{name} vs fp32 oracle (rtol {rtol}): {rep}"


def near_ties_only(sel, ref_sel, scores, limit):
    rows = (sel != ref_sel).any(dim=1)
    for t in rows.nonzero().flatten().tolist():
        diff = sorted(set(sel[t].tolist()) ^ set(ref_sel[t].tolist()))
        if diff:
            vals = scores[t, diff]
            assert (vals.max() - vals.min()).item() < limit, f"row {t}: selection differs beyond a near-tie"
    return rows.float().mean().item()


@pytest.mark.parametrize("name", ["tiny_moe", "tiny_moe_ragged", "tiny_moe_shared2", "moe_1b"])
@pytest.mark.parametrize("aux_grad", [0.0, 3.0])
def test_moe_layer_fwd_bwd_matches_oracle(name, aux_grad):
    if name == "moe_1b" and aux_grad != 0.0:
        pytest.skip("one aux-loss case per size is enough for the big shape")
    from swamla_b200 import functional
    w = inputs.WORKLOADS[name]
    tokens = 1024 if name == "moe_1b" else None           # the oracle's per-expert loop stays in seconds
    params, buffers, x, dy = inputs.make_inputs(w, tokens=tokens)
    layer = build_layer(w, params, buffers, torch.bfloat16)
    layer.train()

    def run(force=None):
        for p_ in layer.parameters():
            p_.grad = None
        xg = x.to("cuda:0").to(torch.bfloat16).requires_grad_(True)
        functional._testing.FORCE_SEL = force
        try:
            y = layer(xg)
            loss = (y.float() * dy.to("cuda:0").to(torch.bfloat16).float()).sum() + aux_grad * layer.get_aux_loss()
            loss.backward()
            torch.cuda.synchronize()
        finally:
            functional._testing.FORCE_SEL = None
        return y, xg

    def oracle(sel_override=None):
        pr = {k: inputs.round_to_bf16(v) for k, v in params.items()}
        return R.layer_forward_backward(pr, buffers, inputs.round_to_bf16(x), inputs.round_to_bf16(dy), w.K,
                                        z_loss_coef=w.router_z_loss_coef, aux_grad=aux_grad, sel_override=sel_override)

    y, xg = run()
    assert y.dtype == torch.bfloat16 and y.shape == x.shape
    sel = layer.router._last_selected_experts.cpu().long()
    out, grads = oracle()
    if not torch.equal(sel, out["sel"]):
        scores = torch.sigmoid(out["logits"]) + buffers["router.expert_bias"]
        assert near_ties_only(sel, out["sel"], scores, 1e-4) < 0.01
        out, grads = oracle(sel_override=sel)
    assert torch.equal(layer.router._last_counts.cpu().long(), out["counts"])
    assert_close("y", y, out["y"])
    assert abs(layer.get_aux_loss().item() - out["aux_loss"].item()) <= 1e-4 * abs(out["aux_loss"].item())
    assert_close("grad x", xg.grad, grads["x"])
    named = dict(layer.named_parameters())
    assert set(named) == set(params)
    for k, ref in grads.items():
        if k == "x":
            continue
        assert named[k].grad is not None and named[k].grad.dtype == named[k].dtype, k
        assert_close(f"grad {k}", named[k].grad, ref)
    # deterministic
    y2, xg2 = run()
    assert torch.equal(y, y2) and torch.equal(xg.grad, xg2.grad)


@pytest.mark.parametrize("name", ["tiny_moe", "tiny_moe_ragged"])
def test_moe_layer_fp32_against_golden_fixture(name):
    """fp32 parameters and x -> fp32 out and fp32 gradients, compared with the frozen outputs of the reference MoELayer."""
    from swamla_b200 import functional
    fx = torch.load(golden_path(name), weights_only=False)
    w = inputs.WORKLOADS[name]
    params, buffers, x, dy = inputs.make_inputs(w)
    layer = build_layer(w, params, buffers, torch.float32)
    layer.train()
    xg = x.to("cuda:0").requires_grad_(True)
    y = layer(xg)
    assert y.dtype == torch.float32
    sel = layer.router._last_selected_experts.cpu().long()
    ref_sel = fx["sel"].long()
    scores = torch.sigmoid(x.reshape(-1, w.D) @ params["router.gate.weight"].t()) + buffers["router.expert_bias"]
    assert near_ties_only(sel, ref_sel, scores, 8e-3) < 0.3       # bf16-rounded logits against fp32 ones

    def check(what, t, d):
        flat = t.detach().float().cpu().reshape(-1)[::d["step"]]
        ok, rep = R.within_tolerance(flat, d["sample"], RTOL_BF16)
        assert ok, f"{what} vs reference fixture: {rep}"

    functional._testing.FORCE_SEL = ref_sel                          # the float path on the reference's own selection
    try:
        y = layer(xg)
        check("y", y, fx["y"])
        assert abs(layer.get_aux_loss().item() - fx["aux_loss"]) <= 2e-3 * abs(fx["aux_loss"])
        ((y * dy.to("cuda:0")).sum() + fx["aux_grad"] * layer.get_aux_loss()).backward()
    finally:
        functional._testing.FORCE_SEL = None
    named = dict(layer.named_parameters())
    assert set(fx["grads"]) - {"x"} == set(named)
    for k, d in fx["grads"].items():
        g = xg.grad if k == "x" else named[k].grad
        assert g.dtype == torch.float32
        check(f"grad {k}", g, d)
    layer.router.update_bias_from_last_forward()
    torch.testing.assert_close(layer.router.expert_bias.cpu(), fx["expert_bias_after_update"], rtol=0, atol=0)
    torch.testing.assert_close(layer.router.load_history.cpu(), fx["load_history_after_update"], rtol=1e-6, atol=1e-7)


def test_moe_layer_contract():
    from swamla_b200 import _cabi
    from swamla_b200.layer import LatentMoELayer, MoELayer, create_moe_layer
    w = inputs.WORKLOADS["tiny_moe"]
    params, buffers, _, _ = inputs.make_inputs(w)
    layer = create_moe_layer(w.config())
    assert isinstance(layer, MoELayer)
    assert isinstance(create_moe_layer(inputs.WORKLOADS["tiny"].config(), use_latent=True), LatentMoELayer)
    assert set(layer.state_dict()) == set(params) | set(buffers)
    assert [k for k, _ in layer.named_parameters()] == list(params)      # registration order of the reference class
    assert (layer.n_experts, layer.n_activated, layer.d_model, layer.expert_dim) == (w.E, w.K, w.D, w.Fs)
    assert layer.experts.gate_up_weight.shape == (w.E, w.D, 2 * w.F)
    with pytest.raises(_cabi.LmoeError):
        layer(torch.randn(1, 4, w.D))
