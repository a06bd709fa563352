"""Pure-torch fp32 restatement of the reference LatentMoE layer (TEST INFRASTRUCTURE).

Each function cites the reference lines it follows (paths are relative to the
reference project).  Everything is differentiable through autograd, which also
supplies the gradients of the grouped GEMM that the reference's Triton kernel
leaves undefined (``models/moe_triton.py:200-242`` has no autograd wrapper).

Canonical integer semantics (the reference leaves both unspecified):
  * top-k: slot k holds the k-th largest score, ties broken by the lower expert
    index (= stable descending sort).  ``torch.topk`` (``models/moe.py:229``)
    returns one member of the same family on tie-free rows.
  * permutation: stable ascending sort of the flat expert ids, i.e. ascending
    flat index t*K+k within an expert.  The reference's atomic cursor
    (``models/moe_triton.py:12-33``) yields an arbitrary order inside an
    expert; the layer output does not depend on it.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn.functional as F


def canonical_topk(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Indices [T,k] of the k largest scores, lower index first among equals."""
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices
    return order[:, :k].contiguous()


def router_forward(x_flat, gate_w, expert_bias, top_k: int, z_loss_coef: float,
                   logits: Optional[torch.Tensor] = None, use_torch_topk: bool = False):
    """models/moe.py:196-242 (AuxLossFreeRouter.forward).

    ``logits`` may be supplied to bypass the gate GEMM (parity "given fp32
    gate logits").
    """
    if logits is None:
        logits = x_flat @ gate_w.t()                                           # moe.py:217
    z_loss = z_loss_coef * torch.logsumexp(logits, dim=-1).pow(2).mean()       # moe.py:220
    affinity = torch.sigmoid(logits)                                           # moe.py:223
    scores = affinity + expert_bias                                            # moe.py:226
    if use_torch_topk:
        sel = torch.topk(scores, top_k, dim=-1).indices                        # moe.py:229
    else:
        sel = canonical_topk(scores.detach(), top_k)
    sel_aff = torch.gather(affinity, 1, sel)                                   # moe.py:232
    weights = sel_aff / (sel_aff.sum(dim=-1, keepdim=True) + 1e-9)             # moe.py:233
    return logits, sel, weights, z_loss


def route_permute(sel: torch.Tensor, n_experts: int):
    """models/moe_triton.py:36-78 (fused_moe_routing), canonical order."""
    flat = sel.reshape(-1)
    counts = torch.bincount(flat, minlength=n_experts).to(torch.int64)         # moe_triton.py:60-62
    offsets = torch.zeros(n_experts + 1, dtype=torch.int64, device=flat.device)
    offsets[1:] = torch.cumsum(counts, 0)                                      # moe_triton.py:65-66
    perm = torch.argsort(flat, stable=True)                                    # moe_triton.py:12-33,73-76
    return counts, offsets, perm


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """models/moe_triton.py:200-242 (moe_gemm): C[rows_e] = A[rows_e] @ B[e]."""
    out = a.new_zeros(a.shape[0], b.shape[2])
    off = offsets.tolist()
    pieces = []
    for e in range(b.shape[0]):
        lo, hi = off[e], off[e + 1]
        if hi > lo:
            pieces.append(a[lo:hi] @ b[e])
    if pieces:
        out = torch.cat(pieces, 0)
    return out


def swiglu_expert(x, gate_up_w, down_w):
    """models/moe.py:55-69 (SwiGLUExpert.forward); gate = first half."""
    gu = x @ gate_up_w.t()
    gate, up = gu.chunk(2, dim=-1)
    hidden = F.silu(gate) * up
    return hidden @ down_w.t(), gu, hidden


def layer_forward(params: Dict[str, torch.Tensor], buffers: Dict[str, torch.Tensor],
                  x: torch.Tensor, top_k: int, z_loss_coef: float = 0.001,
                  logits_override: Optional[torch.Tensor] = None,
                  sel_override: Optional[torch.Tensor] = None,
                  use_torch_topk: bool = False) -> Dict[str, torch.Tensor]:
    """models/moe.py:702-784,786-839 (LatentMoELayer.forward and helpers).

    Without ``down_proj.weight`` / ``up_proj.weight`` in ``params`` this is the non-latent ``MoELayer``
    (models/moe.py:344-372 forward, 437-482 grouped path, 484-537 expert GEMMs): the experts read x itself and
    their weighted sum is added to the shared expert's output directly.

    Returns every intermediate the kernels are checked against.
    ``sel_override`` forces the routing decision (used to compare the float
    path on identical routing when a near-tie flips a selection).
    """
    B, S, D = x.shape
    x_flat = x.reshape(-1, D)                                                  # moe.py:710
    T = x_flat.shape[0]
    n_shared = sum(1 for k in params if k.endswith("gate_up_proj.weight"))
    E = params["experts.gate_up_weight"].shape[0]

    # 1. shared expert(s)                                                      # moe.py:713-715
    shared = torch.zeros_like(x_flat)
    h1_s = hidden_s = None
    for i in range(n_shared):
        o, h1_s, hidden_s = swiglu_expert(x_flat, params[f"shared_experts.{i}.gate_up_proj.weight"],
                                          params[f"shared_experts.{i}.down_proj.weight"])
        shared = shared + o

    # 2. router                                                                # moe.py:718-719
    logits, sel, weights, z_loss = router_forward(
        x_flat, params["router.gate.weight"], buffers["router.expert_bias"], top_k, z_loss_coef,
        logits=logits_override, use_torch_topk=use_torch_topk)
    if sel_override is not None:
        sel = sel_override
        aff = torch.sigmoid(logits)
        sa = torch.gather(aff, 1, sel)
        weights = sa / (sa.sum(-1, keepdim=True) + 1e-9)

    # 3. latent down-projection                                                # moe.py:722
    latent = "down_proj.weight" in params
    x_latent = x_flat @ params["down_proj.weight"].t() if latent else x_flat   # MoELayer: moe.py:361

    # 4. grouped experts                                                       # moe.py:736-784
    counts, offsets, perm = route_permute(sel, E)                              # moe.py:757
    L = x_latent.shape[1]
    x_exp = x_latent.unsqueeze(1).expand(-1, top_k, -1).reshape(-1, L)         # moe.py:762
    w_flat = weights.reshape(-1, 1)                                            # moe.py:763
    x_sorted = x_exp[perm]                                                     # moe.py:766
    w_sorted = w_flat[perm]                                                    # moe.py:767
    h1 = grouped_gemm(x_sorted, params["experts.gate_up_weight"], offsets)     # moe.py:814
    gate, up = h1.chunk(2, dim=-1)                                             # moe.py:822
    hidden = F.silu(gate) * up                                                 # moe.py:823
    y_sorted = grouped_gemm(hidden, params["experts.down_weight"], offsets)    # moe.py:828
    y_weighted = y_sorted * w_sorted                                           # moe.py:837
    y_exp = torch.zeros_like(y_weighted)                                       # moe.py:778
    y_exp = y_exp.index_put((perm,), y_weighted)                               # moe.py:779
    routed = y_exp.view(T, top_k, L).sum(dim=1)                                # moe.py:782

    # 5./6. up-projection and final add (dropout p=0)                          # moe.py:728-734
    routed_out = routed @ params["up_proj.weight"].t() if latent else routed   # MoELayer: moe.py:366
    y = (shared + routed_out).view(B, S, D)
    return dict(y=y, aux_loss=z_loss, logits=logits, sel=sel, weights=weights, counts=counts,
                offsets=offsets, perm=perm, x_latent=x_latent, x_sorted=x_sorted, h1=h1, hidden=hidden,
                y_sorted=y_sorted, routed=routed, h1_s=h1_s, hidden_s=hidden_s, shared=shared)


def layer_forward_backward(params, buffers, x, dy, top_k, z_loss_coef=0.001, aux_grad: float = 0.0,
                           sel_override=None):
    """fwd + autograd bwd.  Loss = <y, dy> + aux_grad * aux_loss.  Returns (fwd dict, grads dict)."""
    p = {k: v.detach().clone().requires_grad_(True) for k, v in params.items()}
    xr = x.detach().clone().requires_grad_(True)
    out = layer_forward(p, buffers, xr, top_k, z_loss_coef, sel_override=sel_override)
    loss = (out["y"] * dy).sum() + aux_grad * out["aux_loss"]
    loss.backward()
    grads = {k: v.grad for k, v in p.items()}
    grads["x"] = xr.grad
    return {k: (v.detach() if torch.is_tensor(v) else v) for k, v in out.items()}, grads


@torch.no_grad()
def update_bias(sel: torch.Tensor, num_tokens: int, buffers: Dict[str, torch.Tensor], top_k: int,
                gamma: float = 0.001) -> None:
    """models/moe.py:254-275 (_update_bias), in place on ``buffers``."""
    E = buffers["router.expert_bias"].shape[0]
    load = torch.zeros(E, dtype=torch.float32)
    flat = sel.reshape(-1)
    load.scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.float32))      # moe.py:259-264
    expected = num_tokens * top_k / E                                          # moe.py:267
    buffers["router.expert_bias"] -= gamma * (load - expected).sign()          # moe.py:271
    buffers["router.load_history"] = 0.99 * buffers["router.load_history"] + 0.01 * load   # moe.py:274
    buffers["router.update_count"] = buffers["router.update_count"] + 1        # moe.py:275


def tolerance_ok(test: torch.Tensor, ref: torch.Tensor, rtol: float):
    """|test-ref| <= rtol * (|ref| + rms(ref)) elementwise; returns (ok, worst ratio)."""
    ref = ref.double()
    test = test.double()
    rms = ref.pow(2).mean().sqrt()
    bound = rtol * (ref.abs() + rms)
    ratio = ((test - ref).abs() / bound.clamp_min(1e-300)).max().item() if ref.numel() else 0.0
    return ratio <= 1.0, ratio


def closeness(test: torch.Tensor, ref: torch.Tensor, rtol: float) -> dict:
    """Error report of ``test`` against ``ref`` for a tolerance ``rtol``:
    rel_fro  = ||test-ref||_F / ||ref||_F
    frac_out = share of elements with |err| > rtol * (|ref| + rms(ref))
    max_ratio = largest |err| / (rtol * (|ref| + rms(ref)))."""
    ref = ref.double().reshape(-1)
    test = test.double().reshape(-1)
    if ref.numel() == 0:
        return dict(rel_fro=0.0, frac_out=0.0, max_ratio=0.0)
    rms = ref.pow(2).mean().sqrt()
    err = (test - ref).abs()
    bound = (rtol * (ref.abs() + rms)).clamp_min(1e-300)
    return dict(rel_fro=(err.norm() / ref.norm().clamp_min(1e-300)).item(),
                frac_out=(err > bound).double().mean().item(), max_ratio=(err / bound).max().item())


def within_tolerance(test: torch.Tensor, ref: torch.Tensor, rtol: float):
    """The acceptance criterion for floating-point results at tolerance ``rtol``.

    A tensor of millions of bf16-rounded values always has a few elements in the far tail of the
    rounding-error distribution, so a pure element-wise maximum does not express "within rtol".  The
    criterion is: relative Frobenius error <= rtol/2, at most 0.1 % of the elements outside
    rtol * (|ref| + rms(ref)), and no element beyond 3x that bound (no gross outlier)."""
    rep = closeness(test, ref, rtol)
    ok = rep["rel_fro"] <= rtol / 2 and rep["frac_out"] <= 1e-3 and rep["max_ratio"] <= 3.0
    return ok, rep
