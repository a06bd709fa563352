"""Constructor semantics of the drop-in modules against the reference classes (CPU only; no kernel is called)."""
from types import SimpleNamespace

import pytest
import torch

from oracle import inputs, ref_shim

CONFIGS = [
    dict(n_embd=1024, n_experts=32, n_activated=3, n_shared_experts=1, latent_ratio=4, expert_dim=1024),     # moe-1b
    dict(n_embd=1024, n_experts=32, n_activated=3, n_shared_experts=1, latent_ratio=4, expert_dim=3072),     # moe-2b
    dict(n_embd=1024, n_experts=64, n_activated=4, latent_ratio=4, expert_dim=1024),
    dict(n_embd=512, n_experts=8, n_activated=2, latent_ratio=2, expert_dim=512, latent_n_experts=24, latent_n_activated=5),
    dict(n_embd=512, latent_ratio=4, latent_dim=256, n_experts=4, n_activated=1, expert_dim=512),            # explicit latent_dim
    dict(n_embd=512, latent_ratio=4, n_experts=4, n_activated=2, expert_dim=256, latent_preserve_expert_dim=True),
    dict(n_embd=256),                                                                                         # all defaults
    dict(n_embd=256, n_experts=4, n_activated=1, n_shared_experts=2, latent_ratio=4, expert_dim=256),         # two shared experts
]


def _shapes(module):
    return {k: tuple(v.shape) for k, v in module.state_dict().items()}


@pytest.mark.skipif(not ref_shim.available(), reason="reference source tree not present")
@pytest.mark.parametrize("cfg", CONFIGS)
def test_latent_layer_ctor_matches_reference(cfg):
    from swamla_b200.layer import LatentMoELayer
    moe = ref_shim.load_reference_moe()
    ours, ref = LatentMoELayer(SimpleNamespace(**cfg)), moe.LatentMoELayer(SimpleNamespace(**cfg))
    assert _shapes(ours) == _shapes(ref)
    assert [k for k, _ in ours.named_parameters()] == [k for k, _ in ref.named_parameters()]
    for attr in ("n_experts", "n_shared", "n_activated", "d_model", "latent_dim", "expert_dim", "latent_ratio",
                 "latent_expert_dim"):
        assert getattr(ours, attr) == getattr(ref, attr), attr
    assert (ours.router.top_k, ours.router.gamma, ours.router.z_loss_coef) == (ref.router.top_k, ref.router.gamma,
                                                                               ref.router.z_loss_coef)
    assert type(ours).__name__ == type(ref).__name__ == "LatentMoELayer"
    assert ours.get_load_balance_stats() == ref.get_load_balance_stats()


@pytest.mark.skipif(not ref_shim.available(), reason="reference source tree not present")
@pytest.mark.parametrize("cfg", [dict(n_embd=256, n_experts=8, n_activated=2, expert_dim=128),
                                 dict(n_embd=1024, n_experts=32, n_activated=3, expert_dim=1024), dict(n_embd=512),
                                 dict(n_embd=256, n_experts=8, n_activated=2, expert_dim=128, n_shared_experts=3)])
def test_moe_layer_ctor_matches_reference(cfg):
    from swamla_b200.layer import MoELayer, create_moe_layer
    moe = ref_shim.load_reference_moe()
    ours, ref = create_moe_layer(SimpleNamespace(**cfg)), moe.create_moe_layer(SimpleNamespace(**cfg))
    assert isinstance(ours, MoELayer) and type(ref).__name__ == "MoELayer"
    assert _shapes(ours) == _shapes(ref)
    assert [k for k, _ in ours.named_parameters()] == [k for k, _ in ref.named_parameters()]
    for attr in ("n_experts", "n_shared", "n_activated", "d_model", "expert_dim"):
        assert getattr(ours, attr) == getattr(ref, attr), attr


def test_ctor_refuses_what_the_kernels_do_not_cover():
    from swamla_b200.layer import LatentMoELayer, MoELayer
    base = dict(n_embd=1024, n_experts=32, n_activated=3, latent_ratio=4, expert_dim=1024)
    with pytest.raises(NotImplementedError):
        LatentMoELayer(SimpleNamespace(**base, bias=True))
    with pytest.raises(NotImplementedError):
        LatentMoELayer(SimpleNamespace(**base, n_shared_experts=0))
    with pytest.raises(ValueError):
        LatentMoELayer(SimpleNamespace(**{**base, "n_experts": 128}))            # 512 routed experts > 256
    with pytest.raises(ValueError):
        LatentMoELayer(SimpleNamespace(**{**base, "expert_dim": 1000}))          # routed expert dim 250 is not a multiple of 64
    with pytest.raises(ValueError):
        LatentMoELayer(SimpleNamespace(**base, ep_mode="bogus"))
    with pytest.raises(NotImplementedError):
        MoELayer(SimpleNamespace(n_embd=256, n_experts=8, n_activated=2, expert_dim=128, moe_fp8=True))


def test_workload_flops_match_the_stated_figures():
    W = inputs.WORKLOADS
    assert W["cfg2"].flops_fwd_per_token() == 12_320_768 and 3 * W["cfg2"].flops_fwd_per_token() == 36_962_304
    assert W["cfg3"].flops_fwd_per_token() == 34_340_864
    assert W["cfg5"].flops_fwd_per_token() == 14_155_776
    assert W["cfg2_literal"].flops_fwd_per_token() == 8_585_216
    assert W["cfg5_literal"].flops_fwd_per_token() == 9_043_968
    assert (W["cfg5"].E, W["cfg5"].K, W["cfg5"].T) == (256, 16, 32768)
