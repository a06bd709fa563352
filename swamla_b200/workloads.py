"""Benchmark / parity workloads of the LatentMoE path and their canonical seeded inputs.

Every tensor comes from ONE CPU generator so that the CPU oracle and the GPU
kernels see identical bits: parameters first, in the registration order of the
reference module (``models/moe.py:662-694``: ``down_proj``, ``up_proj``, the
shared experts, the routed experts, the router gate), each N(0, 0.02) as the
model-level init does (``models/swa_mla_model.py:314-320``), then ``x`` and the
upstream gradient ``dy`` ~ N(0, 1).  Buffers start at zero.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Dict, Optional

import torch


@dataclass
class Workload:
    """One benchmark / parity configuration."""
    name: str
    n_embd: int = 1024
    n_experts: int = 32          # base value; the ctor multiplies by latent_ratio
    n_activated: int = 3         # base value; the ctor multiplies by latent_ratio
    n_shared_experts: int = 1
    latent_ratio: int = 4
    expert_dim: int = 1024
    batch: int = 2
    seq: int = 512
    dtype: str = "fp32"          # "fp32" | "bf16" | "fp8"
    zipf_s: float = 0.0          # >0: Zipf-skewed expert_bias
    zipf_beta: float = 0.25
    uniform_gate: bool = False   # router gate ~ U(-1/sqrt(D), 1/sqrt(D))
    router_z_loss_coef: float = 0.001
    latent: bool = True          # False: the non-latent MoELayer (models/moe.py:294-559): experts work at width D
    literal_counts: bool = False # True: n_experts / n_activated are the layer's own counts (config.latent_n_experts /
                                 # latent_n_activated, models/moe.py:639-646) instead of being scaled by latent_ratio
    extra: dict = field(default_factory=dict)

    # ---- derived sizes, following models/moe.py:630-685 ----
    @property
    def D(self) -> int: return self.n_embd
    @property
    def L(self) -> int: return self.n_embd // self.latent_ratio if self.latent else self.n_embd
    @property
    def E(self) -> int:
        return self.n_experts * self.latent_ratio if (self.latent and not self.literal_counts) else self.n_experts
    @property
    def K(self) -> int:
        return self.n_activated * self.latent_ratio if (self.latent and not self.literal_counts) else self.n_activated
    @property
    def F(self) -> int: return self.expert_dim // self.latent_ratio if self.latent else self.expert_dim
    @property
    def Fs(self) -> int: return self.expert_dim
    @property
    def T(self) -> int: return self.batch * self.seq

    def config(self) -> SimpleNamespace:
        """The object handed to ``LatentMoELayer(config)`` (read with getattr)."""
        cfg = SimpleNamespace(
            n_embd=self.n_embd, n_experts=self.n_experts, n_activated=self.n_activated,
            n_shared_experts=self.n_shared_experts, latent_ratio=self.latent_ratio,
            expert_dim=self.expert_dim, bias=False, dropout=0.0,
            router_z_loss_coef=self.router_z_loss_coef, use_latent_moe=self.latent,
        )
        if self.literal_counts:
            cfg.latent_n_experts, cfg.latent_n_activated = self.n_experts, self.n_activated
        return cfg

    def flops_fwd_per_token(self) -> int:
        """GEMM FLOPs only: router + down + routed + up + shared."""
        D, L, E, K, F, Fs = self.D, self.L, self.E, self.K, self.F, self.Fs
        if not self.latent:
            return 2 * D * E + 6 * K * D * F + 6 * self.n_shared_experts * D * Fs
        return 2 * D * E + 2 * D * L + 6 * K * L * F + 2 * L * D + 6 * self.n_shared_experts * D * Fs


WORKLOADS: Dict[str, Workload] = {
    # small shapes for exhaustive parity (all dims are multiples of 64 so they fit the kernels)
    "tiny": Workload("tiny", n_embd=256, n_experts=4, n_activated=1, expert_dim=256, batch=2, seq=96),
    "tiny_ragged": Workload("tiny_ragged", n_embd=256, n_experts=8, n_activated=2, expert_dim=256, batch=1, seq=131),
    # two shared experts (models/moe.py:671-674, 713-715)
    "tiny_shared2": Workload("tiny_shared2", n_embd=256, n_experts=4, n_activated=1, n_shared_experts=2, expert_dim=256,
                             batch=2, seq=80),
    # e4m3 GEMMs contract over multiples of 128: latent 128, routed hidden 128
    "tiny_fp8": Workload("tiny_fp8", n_embd=512, n_experts=4, n_activated=1, expert_dim=512, batch=2, seq=160, dtype="fp8"),
    # the five benchmark configurations
    "cfg1": Workload("cfg1", batch=2, seq=512, dtype="fp32"),
    "cfg2": Workload("cfg2", batch=8, seq=2048, dtype="bf16"),
    # cfg2's layer on a quarter of the tokens: the small case for multi-pass profiler captures
    "cfg2_4k": Workload("cfg2_4k", batch=2, seq=2048, dtype="bf16"),
    "cfg3": Workload("cfg3", expert_dim=3072, batch=32, seq=2048, dtype="bf16", zipf_s=1.2),
    "cfg4": Workload("cfg4", batch=64, seq=2048, dtype="fp8"),
    "cfg5": Workload("cfg5", n_experts=64, n_activated=4, batch=16, seq=2048, dtype="bf16", uniform_gate=True),
    # cfg5's layer (E=256, top-16, uniform gate) on a token count the CPU oracle finishes in seconds
    "cfg5_2k": Workload("cfg5_2k", n_experts=64, n_activated=4, batch=1, seq=2048, dtype="bf16", uniform_gate=True),
    # secondary reading of the benchmark text: 32 experts / top-3 (64 / top-4) taken literally as the layer's counts
    "cfg2_literal": Workload("cfg2_literal", batch=8, seq=2048, dtype="bf16", literal_counts=True),
    "cfg5_literal": Workload("cfg5_literal", n_experts=64, n_activated=4, batch=16, seq=2048, dtype="bf16",
                             uniform_gate=True, literal_counts=True),
    # the non-latent MoELayer (the other branch of create_moe_layer)
    "tiny_moe": Workload("tiny_moe", n_embd=256, n_experts=8, n_activated=2, expert_dim=128, batch=2, seq=96, latent=False),
    "tiny_moe_ragged": Workload("tiny_moe_ragged", n_embd=256, n_experts=16, n_activated=3, expert_dim=128, batch=1, seq=131,
                                latent=False),
    "tiny_moe_shared2": Workload("tiny_moe_shared2", n_embd=256, n_experts=8, n_activated=2, n_shared_experts=2, expert_dim=128,
                                 batch=2, seq=96, latent=False),
    "moe_1b": Workload("moe_1b", n_embd=1024, n_experts=32, n_activated=3, expert_dim=1024, batch=2, seq=2048,
                       dtype="bf16", latent=False),
}


def param_shapes(w: Workload) -> Dict[str, tuple]:
    """state_dict key -> shape, in the reference's registration order."""
    shapes = {} if not w.latent else {
        "down_proj.weight": (w.L, w.D),
        "up_proj.weight": (w.D, w.L),
    }
    for i in range(w.n_shared_experts):
        shapes[f"shared_experts.{i}.gate_up_proj.weight"] = (2 * w.Fs, w.D)
        shapes[f"shared_experts.{i}.down_proj.weight"] = (w.D, w.Fs)
    shapes["experts.gate_up_weight"] = (w.E, w.L, 2 * w.F)
    shapes["experts.down_weight"] = (w.E, w.F, w.L)
    shapes["router.gate.weight"] = (w.E, w.D)
    return shapes


def make_inputs(w: Workload, seed: int = 0, tokens: Optional[int] = None, with_dy: bool = True):
    """Returns (params, buffers, x, dy), all fp32 CPU tensors.

    ``tokens`` overrides batch*seq (x is then [1, tokens, D]); used to draw a
    bounded sample of a large workload with the same distributions.
    """
    g = torch.Generator("cpu").manual_seed(seed)
    params = {}
    for name, shape in param_shapes(w).items():
        p = torch.empty(shape, dtype=torch.float32)
        if name == "router.gate.weight" and w.uniform_gate:
            bound = 1.0 / math.sqrt(w.D)
            p.uniform_(-bound, bound, generator=g)
        else:
            p.normal_(0.0, 0.02, generator=g)
        params[name] = p
    B, S = (w.batch, w.seq) if tokens is None else (1, tokens)
    x = torch.randn(B, S, w.D, generator=g)
    dy = torch.randn(B, S, w.D, generator=g) if with_dy else None
    buffers = {
        "router.expert_bias": torch.zeros(w.E),
        "router.load_history": torch.zeros(w.E),
        "router.update_count": torch.tensor(0),
    }
    if w.zipf_s > 0:
        # expert_bias[pi(j)] = beta * (j+1)^(-s): a Zipf skew over experts that
        # stresses load imbalance (selection only; gating weights ignore the bias).
        pi = torch.randperm(w.E, generator=g)
        j = torch.arange(1, w.E + 1, dtype=torch.float32)
        bias = torch.zeros(w.E)
        bias[pi] = w.zipf_beta * j.pow(-w.zipf_s)
        buffers["router.expert_bias"] = bias
    return params, buffers, x, dy


def round_to_bf16(t: torch.Tensor) -> torch.Tensor:
    """fp32 tensor holding bf16-representable values (what a bf16 module stores)."""
    return t.to(torch.bfloat16).to(torch.float32)
