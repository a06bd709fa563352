"""Runs the UNMODIFIED reference ``LatentMoELayer`` / ``MoELayer`` on CPU (TEST INFRASTRUCTURE).

The reference module imports its two device-only entry points from
``moe_triton`` (``models/moe.py:21-29``); both need a GPU.  After import they
are replaced by torch equivalents with the same semantics:

  * ``fused_moe_routing`` (``models/moe_triton.py:36-78``): bincount, cumsum and a
    stable argsort instead of the atomic-cursor kernel;
  * ``moe_gemm`` (``models/moe_triton.py:200-242``): ``C[rows_e] = A[rows_e] @ B[e]``.

The reference source tree is only present where this repository is developed;
``available()`` says whether it can be used.  Golden fixtures generated through
this module are committed under ``tests/golden``.
"""
from __future__ import annotations

import os
import sys

import torch

# the reference checkout: $SWAMLA_REFERENCE_ROOT, else a directory "reference" beside this repository
REFERENCE_ROOT = os.environ.get(
    "SWAMLA_REFERENCE_ROOT",
    os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))


def available() -> bool:
    return os.path.isfile(os.path.join(REFERENCE_ROOT, "models", "moe.py"))


def _routing_shim(expert_indices: torch.Tensor, n_experts: int):
    flat = expert_indices.reshape(-1).contiguous()
    counts = torch.bincount(flat.int(), minlength=n_experts).to(torch.int64)
    offsets = torch.zeros(n_experts + 1, dtype=torch.int64, device=flat.device)
    offsets[1:] = torch.cumsum(counts, 0)
    perm = torch.argsort(flat, stable=True)
    return counts, offsets, perm


def _gemm_shim(a, b, expert_offsets, activation="", max_tokens_hint=None):
    assert activation == ""
    off = expert_offsets.tolist()
    pieces = [a[off[e]:off[e + 1]] @ b[e] for e in range(b.shape[0]) if off[e + 1] > off[e]]
    if not pieces:
        return a.new_zeros(a.shape[0], b.shape[2])
    return torch.cat(pieces, 0)


_moe = None


def load_reference_moe():
    """Imports the reference ``moe`` module and installs the two shims."""
    global _moe
    if _moe is not None:
        return _moe
    if not available():
        raise RuntimeError(f"reference tree not found under {REFERENCE_ROOT}")
    models_dir = os.path.join(REFERENCE_ROOT, "models")
    if models_dir not in sys.path:
        sys.path.insert(0, models_dir)
    import moe  # noqa: E402  (the reference module, unmodified)
    moe.moe_gemm = _gemm_shim
    moe.fused_moe_routing = _routing_shim
    _moe = moe
    return moe


def build_reference_layer(workload, params, buffers):
    """Reference ``LatentMoELayer(config)`` (or ``MoELayer(config)`` for a non-latent workload) loaded with the
    given state, built through the reference's own factory (``models/moe.py:869-882``)."""
    moe = load_reference_moe()
    layer = moe.create_moe_layer(workload.config(), use_latent=getattr(workload, "latent", True))
    assert type(layer).__name__ == ("LatentMoELayer" if getattr(workload, "latent", True) else "MoELayer")
    state = dict(params)
    state.update(buffers)
    missing, unexpected = layer.load_state_dict(state, strict=True)
    assert not missing and not unexpected
    return layer


def run_reference(workload, params, buffers, x, dy=None, aux_grad: float = 0.0):
    """fwd (+bwd when dy is given) of the reference module in fp32 on CPU."""
    layer = build_reference_layer(workload, params, buffers)
    layer.train()
    xr = x.detach().clone().requires_grad_(dy is not None)
    y = layer(xr)
    out = dict(y=y.detach(), aux_loss=layer.aux_loss.detach(),
               sel=layer.router._last_selected_experts.clone())
    grads = None
    if dy is not None:
        loss = (y * dy).sum() + aux_grad * layer.aux_loss
        loss.backward()
        grads = {k: p.grad for k, p in layer.named_parameters()}
        grads["x"] = xr.grad
    return out, grads, layer
