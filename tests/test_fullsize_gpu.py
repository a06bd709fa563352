"""BASELINE-size workloads (cfg2, cfg3, cfg4).  Two kinds of checks: (1) size-independent properties (token independence
of the forward, structural invariants of routing, linearity of the backward, run-to-run determinism), and (2) the fp32
oracle itself, which is plain torch and therefore also runs on the GPU (fp32 matmuls, TF32 off) in seconds at full
size: y, dx and every parameter gradient of cfg2 and cfg3 are compared with it at the bf16 tolerance.  That covers what
only exists at size: per-expert weight gradients contracting over many k-blocks, the split-K of the dense weight
gradients at K = T, the skewed expert loads of cfg3, multi-wave tile schedules."""
import pytest
import torch

from oracle import inputs, latent_moe_ref as R

pytestmark = pytest.mark.gpu


def _build(w, fp8=False):
    from swamla_b200.layer import LatentMoELayer
    params, buffers, x, dy = inputs.make_inputs(w)
    cfg = w.config()
    if fp8:
        cfg.moe_fp8 = True
    layer = LatentMoELayer(cfg)
    layer.load_state_dict({**params, **buffers}, strict=True)
    return layer.to("cuda:0").to(torch.bfloat16).train(), params, buffers, x, dy


def _routing_invariants(layer, w, sink):
    route, sel = sink["route"], sink["sel"]
    T, K, E = w.T, w.K, w.E
    n = T * K
    counts = route.counts.long()
    assert counts.sum().item() == n and route.offsets[-1].item() == n
    assert torch.equal(route.offsets.long()[1:], counts.cumsum(0))
    flat = sel.reshape(-1).long()
    perm = route.perm.long()
    assert torch.equal(torch.sort(perm).values, torch.arange(n, device=perm.device))          # a permutation
    sorted_e = flat[perm]
    assert torch.all(sorted_e[1:] >= sorted_e[:-1])                                            # grouped by expert
    same = sorted_e[1:] == sorted_e[:-1]
    assert torch.all(perm[1:][same] > perm[:-1][same])                                         # stable inside an expert
    assert torch.equal(torch.bincount(flat, minlength=E), counts)
    # top-k property on the device's own fp32 logits: every selected score >= every unselected one, slots descending
    scores = torch.sigmoid(sink["logits"]) + layer.router.expert_bias.float()
    picked = scores.gather(1, sel.long())
    assert torch.all(picked[:, :-1] >= picked[:, 1:])
    masked = scores.scatter(1, sel.long(), float("-inf"))
    assert torch.all(picked[:, -1] >= masked.max(dim=1).values)
    assert torch.all(torch.sort(sel.long(), 1).values[:, 1:] != torch.sort(sel.long(), 1).values[:, :-1])   # distinct
    torch.testing.assert_close(sink["weights"].sum(1), torch.ones(T, device=sel.device), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", ["cfg2", "cfg3"])
def test_full_size_forward_backward_properties(name):
    from swamla_b200 import functional
    w = inputs.WORKLOADS[name]
    layer, params, buffers, x, dy = _build(w)
    xg = x.to("cuda:0").to(torch.bfloat16).requires_grad_(True)
    dyg = dy.to("cuda:0").to(torch.bfloat16)
    sink = {}
    functional._testing.SINK = sink
    try:
        y = layer(xg)
        y.backward(dyg)
        torch.cuda.synchronize()
    finally:
        functional._testing.SINK = None
    assert sink["status"].item() == 0
    assert torch.isfinite(y.float()).all() and torch.isfinite(xg.grad.float()).all()
    _routing_invariants(layer, w, sink)
    if name == "cfg3":      # the Zipf-skewed bias must actually skew the load
        load = sink["route"].counts.float()
        assert (load.max() / load.mean()).item() > 3.0
    g1 = {"x": xg.grad.clone(), **{k: p.grad.clone() for k, p in layer.named_parameters()}}

    # token independence: the first 1024 tokens alone give bit-identical outputs (a row's result does not depend on
    # its place in an expert's segment); that small case is what the CPU oracle checks
    sub = x.reshape(-1, w.D)[:1024].reshape(1, 1024, w.D)
    y_sub = layer(sub.to("cuda:0").to(torch.bfloat16))
    assert torch.equal(y_sub.reshape(-1, w.D), y.detach().reshape(-1, w.D)[:1024])
    pr = {k: inputs.round_to_bf16(v) for k, v in params.items()}
    sel_sub = layer.router._last_selected_experts.cpu().long()
    with torch.no_grad():
        ref = R.layer_forward(pr, buffers, inputs.round_to_bf16(sub), w.K, sel_override=sel_sub)
    ok, rep = R.within_tolerance(y_sub.float().cpu(), ref["y"], 2e-2)
    assert ok, rep

    # linearity of the backward: doubling dy doubles every gradient exactly (a power of two in bf16 / fp32)
    for p in layer.parameters():
        p.grad = None
    x2 = x.to("cuda:0").to(torch.bfloat16).requires_grad_(True)
    layer(x2).backward(dyg * 2)
    torch.cuda.synchronize()
    g2 = {"x": x2.grad, **{k: p.grad for k, p in layer.named_parameters()}}
    for k in g1:
        assert torch.equal(g2[k].float(), g1[k].float() * 2), k

    # determinism: the same step again gives the same bits
    for p in layer.parameters():
        p.grad = None
    x3 = x.to("cuda:0").to(torch.bfloat16).requires_grad_(True)
    y3 = layer(x3)
    y3.backward(dyg)
    assert torch.equal(y3, y) and torch.equal(x3.grad, g1["x"])
    for k, p in layer.named_parameters():
        assert torch.equal(p.grad, g1[k]), k


@pytest.mark.parametrize("name", ["cfg2", "cfg3"])
def test_full_size_outputs_and_gradients_match_fp32_oracle(name):
    dev = torch.device("cuda:0")
    torch.backends.cuda.matmul.allow_tf32 = False           # the oracle's matmuls stay true fp32 on the GPU
    w = inputs.WORKLOADS[name]
    layer, params, buffers, x, dy = _build(w)
    xg = x.to(dev).to(torch.bfloat16).requires_grad_(True)
    y = layer(xg)
    y.backward(dy.to(dev).to(torch.bfloat16))
    layer.check_status()
    sel = layer.router._last_selected_experts.long()
    counts = layer.router._last_counts.long()

    pr = {k: inputs.round_to_bf16(v).to(dev) for k, v in params.items()}
    bufs = {k: v.to(dev) for k, v in buffers.items()}
    xr, dyr = inputs.round_to_bf16(x).to(dev), inputs.round_to_bf16(dy).to(dev)
    with torch.no_grad():
        free = R.layer_forward(pr, bufs, xr, w.K, z_loss_coef=w.router_z_loss_coef)
    # same inputs, different accumulation order of the gate GEMM: selections may differ on near-ties only
    differ = (torch.sort(sel, 1).values != torch.sort(free["sel"], 1).values).any(1)
    assert differ.float().mean().item() < 0.01
    if differ.any():
        scores = torch.sigmoid(free["logits"]) + bufs["router.expert_bias"]
        rows = differ.nonzero().flatten()
        kth = scores[rows].gather(1, free["sel"][rows])[:, -1]                    # the oracle's K-th score
        ours = scores[rows].gather(1, sel[rows]).min(1).values                    # our lowest selected score
        # (logits contract over 1,024 products in another order and on the tensor cores' fp32 accumulators)
        assert (kth - ours).abs().max().item() < 5e-4
    del free
    out, grads = R.layer_forward_backward(pr, bufs, xr, dyr, w.K, z_loss_coef=w.router_z_loss_coef, sel_override=sel)
    assert torch.equal(counts, out["counts"])
    ok, rep = R.within_tolerance(y.detach().float(), out["y"], 2e-2)
    assert ok, ("y", rep)
    ok, rep = R.within_tolerance(xg.grad.float(), grads["x"], 2e-2)
    assert ok, ("grad x", rep)
    named = dict(layer.named_parameters())
    for k, ref in grads.items():
        if k == "x":
            continue
        ok, rep = R.within_tolerance(named[k].grad.float(), ref, 2e-2)
        assert ok, (f"grad {k}", rep)


def test_full_size_fp8_runs_and_keeps_invariants():
    from swamla_b200 import functional
    w = inputs.WORKLOADS["cfg4"]
    layer, params, buffers, x, dy = _build(w, fp8=True)
    xg = x.to("cuda:0").to(torch.bfloat16).requires_grad_(True)
    sink = {}
    functional._testing.SINK = sink
    try:
        y = layer(xg)
        y.backward(dy.to("cuda:0").to(torch.bfloat16))
        torch.cuda.synchronize()
    finally:
        functional._testing.SINK = None
    assert sink["status"].item() == 0
    _routing_invariants(layer, w, sink)
    for name, t in [("y", y), ("dx", xg.grad)] + [(k, p.grad) for k, p in layer.named_parameters()]:
        assert torch.isfinite(t.float()).all(), name
    # the bf16 layer with the same weights agrees within the FP8 band on y (shared path dominates y)
    layer16, *_ = _build(inputs.WORKLOADS["cfg4"])
    y16 = layer16(x.to("cuda:0").to(torch.bfloat16))
    rel = ((y.float() - y16.float()).norm() / y16.float().norm()).item()
    assert rel <= 6e-2, rel
