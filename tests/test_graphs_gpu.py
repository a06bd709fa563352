"""CUDA-graph replay of the layer (forward and backward) against eager execution."""
import pytest
import torch

from oracle import inputs

pytestmark = pytest.mark.gpu


def test_graph_replay_matches_eager_bit_for_bit():
    from swamla_b200.graphs import GraphedLatentMoE
    from swamla_b200.layer import LatentMoELayer
    w = inputs.WORKLOADS["tiny_ragged"]
    params, buffers, x, dy = inputs.make_inputs(w)

    def build():
        layer = LatentMoELayer(w.config())
        layer.load_state_dict({**params, **buffers}, strict=True)
        return layer.to("cuda:0").to(torch.bfloat16).train()

    eager, captured = build(), build()
    graphed = GraphedLatentMoE(captured, x.to("cuda:0").to(torch.bfloat16))
    g = torch.Generator().manual_seed(9)
    for it in range(3):                                   # new inputs on every replay
        xi = (x + 0.1 * it * torch.randn(x.shape, generator=g)).to("cuda:0").to(torch.bfloat16)
        dyi = (dy * (1 + it)).to("cuda:0").to(torch.bfloat16)
        outs = []
        for mod, layer in ((eager, eager), (graphed, captured)):
            for p in layer.parameters():
                p.grad = None
            xg = xi.clone().requires_grad_(True)
            y = mod(xg)
            (y.float() * dyi.float()).sum().add(2.0 * layer.get_aux_loss()).backward()
            torch.cuda.synchronize()
            outs.append((y.detach().clone(), xg.grad.clone(), {k: p.grad.clone() for k, p in layer.named_parameters()},
                         layer.get_aux_loss().detach().clone(), layer.router._last_counts.clone()))
        (y1, dx1, g1, a1, c1), (y2, dx2, g2, a2, c2) = outs
        assert torch.equal(y1, y2) and torch.equal(dx1, dx2) and torch.equal(a1, a2) and torch.equal(c1, c2), it
        for k in g1:
            assert torch.equal(g1[k], g2[k]), (it, k)
        # the reference's training loop updates the selection bias after every backward (models/moe.py:244-252);
        # the update clears the router's "last forward" state, which a replay must attach again
        for layer in (eager, captured):
            layer.router.update_bias_from_last_forward()
        for name in ("expert_bias", "load_history", "update_count"):
            assert torch.equal(getattr(eager.router, name), getattr(captured.router, name)), (it, name)
        assert int(captured.router.update_count) == it + 1
    assert eager.router.expert_bias.abs().max().item() > 0
