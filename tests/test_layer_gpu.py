"""The drop-in layer on the GPU against the CPU oracle (fp32 on the same bf16-rounded inputs)
and against the golden fixtures generated from the reference module."""
import pytest
import torch

from oracle import inputs, latent_moe_ref as R
from conftest import golden_path

pytestmark = pytest.mark.gpu
RTOL_BF16 = 2e-2      # outputs and gradients vs the fp32 reference


def build_layer(w, params, buffers, dtype):
    from swamla_b200.layer import LatentMoELayer
    layer = LatentMoELayer(w.config())
    state = dict(params)
    state.update(buffers)
    layer.load_state_dict(state, strict=True)
    return layer.to("cuda:0").to(dtype) if dtype != torch.float32 else layer.to("cuda:0")


def oracle_on_rounded(w, params, buffers, x, dy, aux_grad, sel_override=None):
    pr = {k: inputs.round_to_bf16(v) for k, v in params.items()}
    return R.layer_forward_backward(pr, buffers, inputs.round_to_bf16(x), inputs.round_to_bf16(dy), w.K,
                                    z_loss_coef=w.router_z_loss_coef, aux_grad=aux_grad, sel_override=sel_override)


def assert_close(name, test, ref, rtol=RTOL_BF16):
    """Within `rtol` of the fp32 oracle (criterion: oracle.latent_moe_ref.within_tolerance)."""
    ok, rep = R.within_tolerance(test.detach().float().cpu(), ref, rtol)
    assert ok, f"{name} vs fp32 oracle (rtol {rtol}): {rep}"


BF16_ULP = 2.0 ** -7


def assert_matches_bf16_model(name, test, model):
    """About one bf16 ulp from the CPU model of the bf16 pipeline: every element within 2 ulp
    (plus a small floor for values near zero) and a relative Frobenius error <= 2.5e-3 (one-ulp flips
    accumulate along the backward chain; the fp32 comparison sits at 3.5e-3 .. 5e-3).  The router
    adjoint subtracts nearly equal terms (d_w_k - sum_j d_w_j w_j), which amplifies the last-bit
    differences of its inputs: 4 ulp there and for what is computed from it."""
    ulps = 4 if any(s in name for s in ("d_logits", "router.gate")) else 2
    rep = R.closeness(test.detach().float().cpu(), model, ulps * BF16_ULP)
    assert rep["rel_fro"] <= 2.5e-3 and rep["max_ratio"] <= 1.5 and rep["frac_out"] <= 1e-5, f"{name} vs bf16 pipeline model: {rep}"


@pytest.mark.parametrize("name", ["tiny", "tiny_ragged", "cfg1", "cfg5_2k"])
@pytest.mark.parametrize("aux_grad", [0.0, 3.0])
def test_layer_fwd_bwd_matches_oracle(name, aux_grad):
    if name in ("cfg1", "cfg5_2k") and aux_grad != 0.0:
        pytest.skip("one aux-loss case per size is enough for the big shape")
    from oracle import bf16_pipeline
    from swamla_b200 import functional
    w = inputs.WORKLOADS[name]
    params, buffers, x, dy = inputs.make_inputs(w)
    layer = build_layer(w, params, buffers, torch.bfloat16)
    layer.train()
    xg = x.to("cuda:0").to(torch.bfloat16).requires_grad_(True)
    sink = {}
    functional._testing.SINK = sink
    try:
        y = layer(xg)
        loss = (y.float() * dy.to("cuda:0").to(torch.bfloat16).float()).sum() + aux_grad * layer.get_aux_loss()
        loss.backward()
        torch.cuda.synchronize()
    finally:
        functional._testing.SINK = None
    assert sink["status"].item() == 0
    assert y.dtype == torch.bfloat16 and y.shape == x.shape

    sel = sink["sel"].cpu().long()
    out, grads = oracle_on_rounded(w, params, buffers, x, dy, aux_grad)
    mismatch = (sel != out["sel"]).any(dim=1)
    if mismatch.any():
        # same inputs, different fp32 accumulation order: a flipped selection must be a near-tie
        scores = torch.sigmoid(out["logits"]) + buffers["router.expert_bias"]
        for t in mismatch.nonzero().flatten().tolist():
            diff = sorted(set(sel[t].tolist()) ^ set(out["sel"][t].tolist()))
            vals = scores[t, diff] if diff else scores[t, sel[t]]
            assert (vals.max() - vals.min()).item() < 1e-4, f"row {t}: selection differs beyond a near-tie"
        assert mismatch.float().mean().item() < 0.01
        out, grads = oracle_on_rounded(w, params, buffers, x, dy, aux_grad, sel_override=sel)
    model, model_grads = bf16_pipeline.forward_backward(params, buffers, x, dy, w.K, w.router_z_loss_coef,
                                                        aux_grad=aux_grad, sel_override=sel)

    # integer results, bit-exact against the oracle run on the same selection
    route = sink["route"]
    assert torch.equal(route.counts.cpu().long(), out["counts"])
    assert torch.equal(route.offsets.cpu().long(), out["offsets"])
    assert torch.equal(route.perm.cpu().long(), out["perm"])

    # every intermediate: within the bf16 tolerance of the fp32 oracle, and ~1 ulp from the bf16 model
    rows = route.pos.cpu().long()[out["perm"]]      # padded layout -> canonical sorted order
    sorted_keys = {"x_sorted", "h1", "hidden", "y_sorted", "d_y_sorted", "d_h1", "d_x_sorted"}
    for k in ("logits", "weights", "x_latent", "x_sorted", "h1", "hidden", "y_sorted", "routed", "h1_s", "hidden_s"):
        got = sink[k].cpu()[rows] if k in sorted_keys else sink[k]
        assert_close(k, got, out[k], 1e-3 if k in ("logits", "weights") else RTOL_BF16)
        assert_matches_bf16_model(k, got, model[k])
    # (d_hidden and d_hidden_s never reach memory: the SwiGLU adjoint runs in the epilogue of their GEMMs)
    for k in ("d_routed", "d_h1_s", "d_y_sorted", "d_weights", "d_h1", "d_x_sorted", "d_x_latent", "d_logits"):
        got = sink[k].cpu()[rows] if k in sorted_keys else sink[k]
        assert_matches_bf16_model(k, got, model[k])
    assert_close("y", y, out["y"])
    assert_matches_bf16_model("y", y, model["y"])
    assert abs(layer.get_aux_loss().item() - out["aux_loss"].item()) <= 1e-4 * abs(out["aux_loss"].item())
    # pad rows of the expert layout are zero
    used = route.n_tiles.item() * 128
    pad = route.row_src[:used] < 0
    if pad.any():
        for k in ("x_sorted", "h1", "hidden", "y_sorted", "d_y_sorted", "d_h1", "d_x_sorted"):
            assert sink[k][:used][pad].float().abs().max().item() == 0, k

    # gradients: outputs of the path, the 2e-2 criterion applies
    assert_close("grad x", xg.grad, grads["x"])
    assert_matches_bf16_model("grad x", xg.grad, model_grads["x"])
    named = dict(layer.named_parameters())
    for k, ref in grads.items():
        if k == "x":
            continue
        assert named[k].grad is not None, k
        assert named[k].grad.dtype == named[k].dtype
        assert_close(f"grad {k}", named[k].grad, ref)
        assert_matches_bf16_model(f"grad {k}", named[k].grad, model_grads[k])


@pytest.mark.parametrize("aux_grad", [0.0, 2.0])
def test_layer_with_two_shared_experts_matches_oracle(aux_grad):
    """``models/moe.py:671-674, 713-715``: the outputs of all shared experts are summed.  The layer runs them as one
    expert of twice the width; output and every gradient (each shared expert's own parameters included) against the fp32
    oracle on the rounded inputs (the oracle itself is pinned on ``tests/golden/tiny_shared2.pt``, frozen from the
    reference module)."""
    w = inputs.WORKLOADS["tiny_shared2"]
    params, buffers, x, dy = inputs.make_inputs(w)
    layer = build_layer(w, params, buffers, torch.bfloat16)
    assert len(layer.shared_experts) == 2
    layer.train()
    xg = x.to("cuda:0").to(torch.bfloat16).requires_grad_(True)
    y = layer(xg)
    loss = (y.float() * dy.to("cuda:0").to(torch.bfloat16).float()).sum() + aux_grad * layer.get_aux_loss()
    loss.backward()
    layer.check_status()
    sel = layer.router._last_selected_experts.cpu().long()
    out, grads = oracle_on_rounded(w, params, buffers, x, dy, aux_grad, sel_override=sel)
    assert (sel != oracle_on_rounded(w, params, buffers, x, dy, aux_grad)[0]["sel"]).any(dim=1).float().mean().item() < 0.01
    assert_close("y", y, out["y"])
    assert_close("grad x", xg.grad, grads["x"])
    named = dict(layer.named_parameters())
    for k, ref in grads.items():
        if k == "x":
            continue
        assert named[k].grad is not None, k
        assert_close(f"grad {k}", named[k].grad, ref)
    assert {k for k in grads if k.startswith("shared_experts.1.")} == {"shared_experts.1.gate_up_proj.weight",
                                                                        "shared_experts.1.down_proj.weight"}


def test_layer_state_dict_and_attributes_match_reference_contract():
    fx = torch.load(golden_path("tiny"), weights_only=False)
    w = inputs.WORKLOADS["tiny"]
    params, buffers, _, _ = inputs.make_inputs(w)
    layer = build_layer(w, params, buffers, torch.float32)
    assert type(layer).__name__ == "LatentMoELayer"
    assert list(layer.state_dict().keys()) == list(params.keys())[:-1] + ["router.expert_bias", "router.load_history",
                                                                         "router.update_count", "router.gate.weight"] \
        or set(layer.state_dict().keys()) == set(params) | set(buffers)
    assert [k for k, _ in layer.named_parameters()] == list(params.keys())
    assert (layer.n_experts, layer.n_activated, layer.latent_dim, layer.latent_expert_dim) == (w.E, w.K, w.L, w.F)
    assert hasattr(layer.experts, "gate_up_weight") and hasattr(layer.experts, "down_weight")
    assert len(list(layer.shared_experts)) == 1 and layer.down_proj.weight.shape == (w.L, w.D)
    assert set(fx["grads"].keys()) - {"x"} == set(params.keys())


@pytest.mark.parametrize("name", ["tiny", "tiny_ragged", "cfg1"])
def test_layer_fp32_master_weights_against_golden_fixture(name):
    """fp32 parameters and fp32 x (the reference's CPU-runnable case): fp32 in -> fp32 out, grads fp32;
    compared with the frozen outputs of the reference module itself."""
    fx = torch.load(golden_path(name), weights_only=False)
    w = inputs.WORKLOADS[name]
    params, buffers, x, dy = inputs.make_inputs(w)
    layer = build_layer(w, params, buffers, torch.float32)
    layer.train()
    xg = x.to("cuda:0").requires_grad_("grads" in fx)
    y = layer(xg)
    assert y.dtype == torch.float32
    sel = layer.router._last_selected_experts.cpu()
    # The kernels compute the gate logits from bf16-rounded x and weights, the reference fixture from
    # fp32 ones: the k-th and (k+1)-th expert of a row swap when their fp32 scores are within the bf16
    # rounding of the logits.  Every differing row must be such a near-tie in the reference's own scores.
    ref_sel = fx["sel"].long()
    mism_rows = (sel.long() != ref_sel).any(dim=1)
    mismatch = mism_rows.float().mean().item()
    if mism_rows.any():
        logits = x.reshape(-1, w.D) @ params["router.gate.weight"].t()
        scores = torch.sigmoid(logits) + buffers["router.expert_bias"]
        for t in mism_rows.nonzero().flatten().tolist():
            diff = sorted(set(sel[t].tolist()) ^ set(ref_sel[t].tolist()))
            if diff:
                vals = scores[t, diff]
                assert (vals.max() - vals.min()).item() < 8e-3, f"row {t}: flip is not a bf16-level near-tie"

    def check(name, t, d):
        flat = t.detach().float().cpu().reshape(-1)[::d["step"]]
        ok, rep = R.within_tolerance(flat, d["sample"], RTOL_BF16)
        assert ok, f"{name} vs reference fixture: {rep}"

    check("y", y, fx["y"])
    assert abs(layer.get_aux_loss().item() - fx["aux_loss"]) <= 2e-3 * abs(fx["aux_loss"])

    # Second pass on the reference's own selection (test hook): the float path and every gradient
    # against the fixture, and the bias update bit-exact.
    from swamla_b200 import functional
    functional._testing.FORCE_SEL = ref_sel
    try:
        y = layer(xg)
        check("y (reference selection)", y, fx["y"])
        if "grads" in fx:
            loss = (y * dy.to("cuda:0")).sum() + fx["aux_grad"] * layer.get_aux_loss()
            loss.backward()
            named = dict(layer.named_parameters())
            for k, d in fx["grads"].items():
                g = xg.grad if k == "x" else named[k].grad
                assert g.dtype == torch.float32
                check(f"grad {k}", g, d)
    finally:
        functional._testing.FORCE_SEL = None
    layer.router.update_bias_from_last_forward()
    torch.testing.assert_close(layer.router.expert_bias.cpu(), fx["expert_bias_after_update"], rtol=0, atol=0)
    torch.testing.assert_close(layer.router.load_history.cpu(), fx["load_history_after_update"], rtol=1e-6, atol=1e-7)
    assert layer.router.update_count.item() == 1
    assert mismatch < 0.3


def test_layer_is_deterministic_and_checkpoint_safe():
    w = inputs.WORKLOADS["tiny_ragged"]
    params, buffers, x, dy = inputs.make_inputs(w)
    layer = build_layer(w, params, buffers, torch.bfloat16)
    xg = x.to("cuda:0").to(torch.bfloat16)
    y1 = layer(xg)
    y2 = layer(xg)
    assert torch.equal(y1, y2)
    xr = xg.clone().requires_grad_(True)
    y3 = torch.utils.checkpoint.checkpoint(layer, xr, use_reentrant=False)
    y3.float().sum().backward()
    assert torch.equal(y3, y1) and xr.grad is not None


def test_layer_refuses_cpu_tensors():
    from swamla_b200 import _cabi
    w = inputs.WORKLOADS["tiny"]
    from swamla_b200.layer import LatentMoELayer
    layer = LatentMoELayer(w.config())
    with pytest.raises(_cabi.LmoeError):
        layer(torch.randn(1, 4, w.D))


def test_layer_under_torch_compile_matches_eager():
    """The reference trains with torch.compile(model) (train.py:936-942): the layer's custom operators (fake +
    autograd registrations, swamla_b200/compiled_ops.py) keep ONE graph across it (fullgraph=True raises on any graph
    break) and must give the same bits and gradients as the eager call, over several steps with the bias update."""
    import torch.nn as nn
    w = inputs.WORKLOADS["tiny_ragged"]
    params, buffers, x, dy = inputs.make_inputs(w)
    layer = build_layer(w, params, buffers, torch.bfloat16).train()

    class Wrapped(nn.Module):                      # some compilable work either side of the layer
        def __init__(self, ffn):
            super().__init__()
            self.ffn = ffn

        def forward(self, t):
            return self.ffn(t * 1.5) + t

    model = Wrapped(layer)
    compiled = torch.compile(model, backend="aot_eager", fullgraph=True)   # dynamo + AOT autograd, no code generation
    outs = []
    for fn in (model, compiled):
        layer.router.expert_bias.zero_()
        per_step = []
        for it in range(2):
            for p_ in layer.parameters():
                p_.grad = None
            xg = (x * (1 + 0.25 * it)).to("cuda:0").to(torch.bfloat16).requires_grad_(True)
            y = fn(xg)
            ((y.float() * dy.to("cuda:0").to(torch.bfloat16).float()).sum() + 2.0 * layer.get_aux_loss()).backward()
            counts = layer.router._last_counts.clone()
            layer.router.update_bias_from_last_forward()
            per_step.append((y.detach(), xg.grad, layer.get_aux_loss().detach().clone(), counts,
                             layer.router.expert_bias.clone(), *[p_.grad.clone() for p_ in layer.parameters()]))
        outs.append(per_step)
    layer.check_status()
    for step_a, step_b in zip(outs[0], outs[1]):
        for i, (a, b) in enumerate(zip(step_a, step_b)):
            assert torch.equal(a, b), i            # the same kernels on the same inputs: the same bits
