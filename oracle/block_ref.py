"""fp32 restatement of the steps either side of the MoE layer in the reference's block (TEST INFRASTRUCTURE).

``rmsnorm``: models/normalization.py:25-39 (RMSNorm: x * rsqrt(mean(x^2) + eps) * weight; the reference evaluates the
same expression in the input dtype for bf16 inputs and in fp32 otherwise -- this restatement is the fp32 form).
``ffn_block_residual``: models/mla_block.py:83-85 (``self.ffn(self.ffn_norm(x))``) and :159 (``x = x + ...``).
Pinned against the reference's own RMSNorm class where the reference tree is present (tests/test_block_cpu.py) and
against the fixture tests/golden/rmsnorm.pt generated from it.
"""
from __future__ import annotations

import torch


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """models/normalization.py:25-26, 34-39."""
    xf = x.float()
    return weight.float() * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps))


def ffn_block_residual(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, ffn) -> torch.Tensor:
    """models/mla_block.py:83-85, 159: x + ffn(ffn_norm(x)); ``ffn`` is a callable on the normed activations."""
    return x + ffn(rmsnorm(x, norm_weight, eps))
