"""CUDA-graph replay of the LatentMoE layer's forward and backward for a fixed input shape.

The layer launches ~40 kernels per step and allocates ~50 buffers from Python; captured once, a step becomes two
graph launches (forward, backward) with static buffers, which removes the host work and the launch gaps between
kernels.  Built on ``torch.cuda.make_graphed_callables`` (the C-ABI calls launch on the capturing stream, the side
stream of the row kernels forks from and joins it, nothing synchronises).  Single-GPU layers only: the expert-parallel
modes issue collectives and size buffers per step.
"""
from __future__ import annotations

import torch
import torch.nn as nn


class _Core(nn.Module):
    """forward(x) -> (y, aux_loss): both differentiable outputs of the layer as graph outputs."""

    def __init__(self, layer):
        super().__init__()
        self.layer = layer

    def forward(self, x):
        y = self.layer(x)
        return y, self.layer.aux_loss


class GraphedLatentMoE(nn.Module):
    """``GraphedLatentMoE(layer, sample_x)(x)``: same result as ``layer(x)`` for inputs of ``sample_x``'s shape and
    dtype.  ``layer.aux_loss``, ``router._last_selected_experts`` and ``router._last_counts`` refer to static buffers
    that every replay overwrites; they are attached to the router again on every training-mode call, so the
    reference's per-step ``update_bias_from_last_forward()`` (``models/moe.py:244-252``, which clears them) keeps
    working across replays.  Parameters must keep their storage (in-place optimizer updates are fine)."""

    def __init__(self, layer, sample_x: torch.Tensor, num_warmup_iters: int = 3):
        super().__init__()
        if getattr(layer, "ep_size", 1) > 1:
            raise ValueError("graph replay is for single-GPU layers (expert-parallel steps issue collectives)")
        self.layer = layer
        sample = sample_x.detach().clone().requires_grad_(True)
        was_training = layer.training
        layer.train()                      # capture in training mode so that the routing outputs are recorded
        self._graphed = torch.cuda.make_graphed_callables(_Core(layer), (sample,), num_warmup_iters=num_warmup_iters)
        r = layer.router
        # static buffers of the captured forward: every replay rewrites them in place
        self._static = (r._last_selected_experts, r._last_counts, r._last_num_tokens)
        layer.train(was_training)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y, aux = self._graphed(x)
        self.layer.aux_loss = aux
        if self.layer.training:
            r = self.layer.router
            r._last_selected_experts, r._last_counts, r._last_num_tokens = self._static
        return y

    def get_aux_loss(self):
        return self.layer.aux_loss
