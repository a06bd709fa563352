"""CPU model of the bf16 pipeline (TEST INFRASTRUCTURE).

Same mathematics as ``latent_moe_ref.py`` (and therefore as ``models/moe.py:702-839`` of the
reference), but every tensor the kernels keep in bf16 is rounded to bf16 at the point where the
kernels store it, and the backward is written out stage by stage with the same rounding points.
Arithmetic between rounding points is fp32, as in the kernels (fp32 accumulation in tensor memory).

Purpose: the GPU path is compared with the fp32 oracle within the bf16 tolerance (2e-2), which cannot
tell a small kernel defect from rounding.  Against this model the GPU results agree to about one
bf16 ulp, so a defect that hides inside the 2e-2 band still shows.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn.functional as F

from . import latent_moe_ref as R


def rb(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def fq(t: torch.Tensor) -> torch.Tensor:
    """Per-tensor e4m3 fake quantisation ("tensorwise" recipe, ``optimization/fp8_native.py:103-110``; the
    arithmetic itself is torchao's, which the reference does not vendor -- parity unpinned for this part):
    scale = 448 / amax, q = clamp(x * scale, +-448) rounded to e4m3, returned de-scaled in fp32."""
    amax = t.abs().max()
    if amax == 0:
        return t.clone()
    scale = 448.0 / amax
    q = (t * scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).to(torch.float32)
    return q * (amax / 448.0)


def _swiglu_bwd(h1, d_hidden):
    g, u = h1.chunk(2, -1)
    sg = torch.sigmoid(g)
    return rb(torch.cat([d_hidden * u * sg * (1 + g * (1 - sg)), d_hidden * g * sg], -1))


def _grouped(a, b, offsets, transpose_b=False):
    E = b.shape[0]
    out = [a[offsets[e]:offsets[e + 1]] @ (b[e].t() if transpose_b else b[e]) for e in range(E)]
    return torch.cat(out, 0)


def forward_backward(params: Dict[str, torch.Tensor], buffers, x, dy, top_k: int, z_coef: float = 0.001,
                     aux_grad: float = 0.0, sel_override=None, param_grads_bf16: bool = True, fp8: bool = False):
    """Returns (forward dict, grads dict) of the bf16 pipeline for bf16-representable inputs.
    ``fp8``: the six operands of the routed-expert GEMMs are fake-quantised to e4m3 per tensor."""
    q8 = fq if fp8 else (lambda t: t)
    p = {k: rb(v) for k, v in params.items()}
    B, S, D = x.shape
    x = rb(x).reshape(-1, D)
    dy = rb(dy).reshape(-1, D)
    T = x.shape[0]
    K = top_k
    latent = "down_proj.weight" in p      # False: the non-latent MoELayer (experts read x, their sum is added directly)
    Wg = p["router.gate.weight"]
    Wdn, Wup = (p["down_proj.weight"], p["up_proj.weight"]) if latent else (None, None)
    Wgus, Wds = p["shared_experts.0.gate_up_proj.weight"], p["shared_experts.0.down_proj.weight"]
    Wgu, Wde = p["experts.gate_up_weight"], p["experts.down_weight"]
    E, L, _ = Wgu.shape

    # ---- forward ----
    logits = x @ Wg.t()                                   # fp32 logits
    _, sel, w, z = R.router_forward(None, None, buffers["router.expert_bias"], K, z_coef, logits=logits)
    if sel_override is not None:
        sel = sel_override
        a = torch.gather(torch.sigmoid(logits), 1, sel)
        w = a / (a.sum(-1, keepdim=True) + 1e-9)
    x_latent = rb(x @ Wdn.t()) if latent else x
    counts, offsets, perm = R.route_permute(sel, E)
    tok = perm // K
    x_sorted = x_latent[tok]
    xs_q, wgu_q, wde_q = q8(x_sorted), q8(Wgu), q8(Wde)
    h1 = rb(_grouped(xs_q, wgu_q, offsets))
    g, u = h1.chunk(2, -1)
    hidden = rb(F.silu(g) * u)
    hid_q = q8(hidden)
    y_sorted = rb(_grouped(hid_q, wde_q, offsets))
    w_sorted = w.reshape(-1)[perm]
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel())
    routed = torch.zeros(T, L)
    for k in range(K):                                     # slot order, fp32 accumulate
        rows = inv[torch.arange(T) * K + k]
        routed = routed + w[:, k:k + 1] * y_sorted[rows]
    h1_s = rb(x @ Wgus.t())
    gs, us = h1_s.chunk(2, -1)
    hidden_s = rb(F.silu(gs) * us)
    if latent:
        routed = rb(routed)
        y = rb(hidden_s @ Wds.t() + routed @ Wup.t())
    else:
        # the shared expert's output is stored in bf16, then the weighted expert rows are added to it in fp32 (slot order)
        y = rb(hidden_s @ Wds.t())
        for k in range(K):
            y = y + w[:, k:k + 1] * y_sorted[inv[torch.arange(T) * K + k]]
        y = rb(y)
        routed = rb(routed)
    lse = torch.logsumexp(logits, -1)

    # ---- backward ----
    d_routed = rb(dy @ Wup) if latent else dy
    d_hidden_s = rb(dy @ Wds)
    d_h1_s = _swiglu_bwd(h1_s, d_hidden_s)
    d_y_sorted = rb(w_sorted[:, None] * d_routed[tok])
    d_w_sorted = (d_routed[tok] * y_sorted).sum(-1)
    d_w = torch.empty(T * K)
    d_w[perm] = d_w_sorted
    d_w = d_w.view(T, K)
    dy_q = q8(d_y_sorted)
    d_hidden = rb(_grouped(dy_q, wde_q, offsets, transpose_b=True))
    d_h1 = _swiglu_bwd(h1, d_hidden)
    dh1_q = q8(d_h1)
    d_x_sorted = rb(_grouped(dh1_q, wgu_q, offsets, transpose_b=True))
    d_x_latent = torch.zeros(T, L)
    for k in range(K):
        d_x_latent = d_x_latent + d_x_sorted[inv[torch.arange(T) * K + k]]
    if latent:
        d_x_latent = rb(d_x_latent)
    a = torch.gather(torch.sigmoid(logits), 1, sel)
    S_ = a.sum(-1, keepdim=True) + 1e-9
    d_a = (d_w - (d_w * w).sum(-1, keepdim=True)) / S_
    d_logits = torch.zeros(T, E)
    d_logits.scatter_(1, sel, d_a * a * (1 - a))
    if aux_grad != 0.0:
        d_logits = d_logits + aux_grad * z_coef * 2.0 * lse[:, None] * torch.exp(logits - lse[:, None]) / T
    d_logits = rb(d_logits)
    if latent:
        dx = rb(d_h1_s @ Wgus + d_x_latent @ Wdn + d_logits @ Wg)
    else:
        # dense part stored in bf16, then the expert-path rows are added in fp32 (slot order)
        dx = rb(d_h1_s @ Wgus + d_logits @ Wg)
        for k in range(K):
            dx = dx + d_x_sorted[inv[torch.arange(T) * K + k]]
        dx = rb(dx)

    pg = rb if param_grads_bf16 else (lambda t: t)
    grads = {
        "x": dx.view(B, S, D),
        "router.gate.weight": pg(d_logits.t() @ x),
        **({"down_proj.weight": pg(d_x_latent.t() @ x), "up_proj.weight": pg(dy.t() @ routed)} if latent else {}),
        "shared_experts.0.gate_up_proj.weight": pg(d_h1_s.t() @ x),
        "shared_experts.0.down_proj.weight": pg(dy.t() @ hidden_s),
        "experts.gate_up_weight": rb(torch.stack([xs_q[offsets[e]:offsets[e + 1]].t() @ dh1_q[offsets[e]:offsets[e + 1]]
                                                  for e in range(E)])),
        "experts.down_weight": rb(torch.stack([hid_q[offsets[e]:offsets[e + 1]].t() @ dy_q[offsets[e]:offsets[e + 1]]
                                               for e in range(E)])),
    }
    fwd = dict(y=y.view(B, S, D), aux_loss=z, logits=logits, sel=sel, weights=w, counts=counts, offsets=offsets,
               perm=perm, x_latent=x_latent, x_sorted=x_sorted, h1=h1, hidden=hidden, y_sorted=y_sorted, routed=routed,
               h1_s=h1_s, hidden_s=hidden_s, d_routed=d_routed, d_hidden_s=d_hidden_s, d_h1_s=d_h1_s,
               d_y_sorted=d_y_sorted, d_weights=d_w, d_hidden=d_hidden, d_h1=d_h1, d_x_sorted=d_x_sorted,
               d_x_latent=d_x_latent, d_logits=d_logits)
    return fwd, grads
