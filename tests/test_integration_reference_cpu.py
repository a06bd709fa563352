"""The drop-in layer inside the reference's OWN model code (``models/swa_mla_model.py``, ``models/mla_block.py``), on CPU.

The reference model is built twice from the same state: once as it ships (its ``LatentMoELayer``, with the two
device-only Triton entry points replaced by torch equivalents through ``oracle/ref_shim.py``) and once with
``moe.create_moe_layer`` patched to return this repository's ``LatentMoELayer``.  One training step then runs through
the reference's call sites in both: ``MLABlock._ffn_block`` under non-reentrant activation checkpointing
(``mla_block.py:83-85,144-151``), ``SWAMLAModel.get_moe_aux_loss`` (``swa_mla_model.py:432-444``), ``backward``,
``SWAMLAModel.update_moe_bias`` (``swa_mla_model.py:455-467``).

The kernels of the product path need a GPU and the reference tree exists only where this repository is developed, so
in THIS test the two calls that reach the CUDA library are stood in for by the CPU oracle (test infrastructure): what
is checked is the module contract the reference model relies on (constructor arguments, attribute and state_dict
names, forward signature, aux-loss accessor, deferred bias update, checkpoint recomputation), not the kernels, which
``-m gpu`` tests cover.
"""
import ctypes
import sys

import numpy as np
import pytest
import torch

from oracle import latent_moe_ref as R
from oracle import ref_shim

pytestmark = pytest.mark.skipif(not ref_shim.available(), reason="reference source tree not present")

MODEL_KW = dict(vocab_size=512, block_size=64, n_layer=2, n_embd=256, n_head=4, local_layers_per_cycle=0,
                mla_layers_per_cycle=1, use_moe=True, use_latent_moe=True, n_experts=4, n_activated=1, expert_dim=256,
                use_gradient_checkpointing=True)


def _oracle_latent_moe(x2d, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias, top_k, z_coef,
                       fp8=False):
    """Stand-in for ``swamla_b200.functional.latent_moe`` with the same signature and return values."""
    params = {"router.gate.weight": w_gate, "down_proj.weight": w_down, "up_proj.weight": w_up,
              "shared_experts.0.gate_up_proj.weight": w_gate_up_s, "shared_experts.0.down_proj.weight": w_down_s,
              "experts.gate_up_weight": w_gate_up, "experts.down_weight": w_down_e}
    out = R.layer_forward(params, {"router.expert_bias": expert_bias}, x2d.unsqueeze(0), top_k, z_loss_coef=z_coef)
    return out["y"].squeeze(0), out["aux_loss"], out["sel"].to(torch.int32), out["counts"].to(torch.int32)


def _oracle_cabi_call(name, *args):
    """Stand-in for ``_cabi.call``: only the bias update is expected here (models/moe.py:254-275)."""
    assert name == "lmoe_router_bias_update", name
    shape, counts_ptr, gamma, bias_ptr, hist_ptr, _stream = args
    E = shape.E
    counts = np.ctypeslib.as_array((ctypes.c_int32 * E).from_address(counts_ptr))
    bias = np.ctypeslib.as_array((ctypes.c_float * E).from_address(bias_ptr))
    hist = np.ctypeslib.as_array((ctypes.c_float * E).from_address(hist_ptr))
    load = counts.astype(np.float32)
    expected = np.float32(load.sum() / E)
    bias -= np.float32(gamma) * np.sign(load - expected).astype(np.float32)
    hist[:] = np.float32(0.99) * hist + np.float32(0.01) * load


def _build(patched, monkeypatch):
    moe = ref_shim.load_reference_moe()
    import swamla_b200.layer as ours
    if patched:
        monkeypatch.setattr(moe, "create_moe_layer", ours.create_moe_layer)   # the one-line patch of INTEGRATION.md
    if ref_shim.REFERENCE_ROOT not in sys.path:
        sys.path.insert(0, ref_shim.REFERENCE_ROOT)
    import swa_mla_model
    torch.manual_seed(0)
    return swa_mla_model.create_swa_mla_model("small", **MODEL_KW)


def test_reference_model_trains_one_step_with_the_drop_in_layer(monkeypatch):
    import swamla_b200.layer as ours
    from swamla_b200 import _cabi
    ref_model = _build(False, monkeypatch)
    new_model = _build(True, monkeypatch)
    ffns = [b.ffn for b in new_model.transformer.h]
    assert all(isinstance(f, ours.LatentMoELayer) for f in ffns)
    assert all(type(b.ffn).__module__ == "moe" for b in ref_model.transformer.h)
    # same parameter and buffer names / shapes / order: a reference checkpoint loads into the patched model
    ref_state = ref_model.state_dict()
    assert [(k, tuple(v.shape)) for k, v in new_model.state_dict().items()] == [(k, tuple(v.shape)) for k, v in ref_state.items()]
    assert [n for n, _ in new_model.named_parameters()] == [n for n, _ in ref_model.named_parameters()]
    new_model.load_state_dict(ref_state, strict=True)

    monkeypatch.setattr(ours, "latent_moe", _oracle_latent_moe)
    monkeypatch.setattr(_cabi, "call", _oracle_cabi_call)
    monkeypatch.setattr(ours, "_stream", lambda: None)                  # no CUDA stream on this host
    g = torch.Generator().manual_seed(1)
    idx = torch.randint(0, MODEL_KW["vocab_size"], (2, 64), generator=g)
    results = []
    for model in (ref_model, new_model):
        model.train()
        out = model(idx, targets=idx)
        loss = out[1] if isinstance(out, tuple) else out.loss
        aux = model.get_moe_aux_loss()
        (loss + aux).backward()
        model.update_moe_bias()
        results.append((loss.detach(), aux.detach(), {n: p.grad for n, p in model.named_parameters()}))
    (l1, a1, g1), (l2, a2, g2) = results
    torch.testing.assert_close(l2, l1, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(a2, a1, rtol=1e-5, atol=1e-7)
    assert a1.item() > 0
    for n in g1:
        if g1[n] is None:
            # the reference's grouped-GEMM kernel has no autograd wrapper (models/moe_triton.py:200-242); with the shim
            # standing in for it the reference does get these gradients, so None may only mean "unused parameter"
            assert g2[n] is None or g2[n].abs().max().item() == 0, n
            continue
        assert g2[n] is not None, n
        torch.testing.assert_close(g2[n], g1[n], rtol=2e-4, atol=1e-6, msg=lambda m, n=n: f"{n}: {m}")
    for b1, b2 in zip(ref_model.transformer.h, new_model.transformer.h):
        r1, r2 = b1.ffn.router, b2.ffn.router
        assert int(r2.update_count) == int(r1.update_count) == 1
        assert torch.equal(r2.expert_bias, r1.expert_bias) and r1.expert_bias.abs().max().item() > 0
        torch.testing.assert_close(r2.load_history, r1.load_history)
        assert r2._last_counts is None and r2._last_selected_experts is None       # cleared as the reference does
    s1, s2 = ref_model.get_moe_load_balance_stats(), new_model.get_moe_load_balance_stats()
    assert s1.keys() == s2.keys()
