"""``torch.library`` custom operators around the LatentMoE path, so that ``torch.compile`` keeps ONE graph across the
layer (the reference compiles the whole model by default, ``train.py:936-942``).

Two opaque operators, ``swamla_b200::latent_moe_fwd`` and ``swamla_b200::latent_moe_bwd``, each with a fake (shape-only)
implementation for tracing, tied together with ``register_autograd``.  Their real implementations run the very same
code as the eager autograd function (``functional.LatentMoEFunction.forward`` / ``.backward`` with a stand-in context
object), so compiled and eager execution launch the same kernels and give the same bits.

An operator's outputs may alias neither its inputs nor one another, so the forward operator returns only tensors it
creates (the routing tables travel as their one int32 allocation) and the backward operator takes the layer's inputs
again and re-derives the bf16 operands from them (a no-op for a bf16 module).

Covers the single-GPU bf16 layer; FP8 experts and the expert-parallel modes stay opaque eager calls
(``torch.compiler.disable``) because they keep Python-side state (collectives, symmetric buffers, scale caches).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import Tensor

from . import functional as Fn

BF = torch.bfloat16
_FWD_OUT = 15   # y, z_loss, sel, counts, route storage, status, logits, weights, lse, x_sorted, h1, hidden, y_sorted, act_cat, h1_s


class _Ctx:
    """Stands in for the autograd context when the function bodies run inside the operators."""

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors

    def mark_non_differentiable(self, *tensors):
        pass


def _dims(x: Tensor, w_gate_up: Tensor, w_down_s: Tensor, top_k: int):
    T, D = x.shape
    E, L, F2 = w_gate_up.shape
    return T, D, L, E, int(top_k), F2 // 2, w_down_s.shape[1]


@torch.library.custom_op("swamla_b200::latent_moe_fwd", mutates_args=())
def latent_moe_fwd(x: Tensor, w_gate: Tensor, w_down: Tensor, w_up: Tensor, w_gate_up_s: Tensor, w_down_s: Tensor,
                   w_gate_up: Tensor, w_down_e: Tensor, expert_bias: Tensor, top_k: int, z_coef: float
                   ) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor,
                              Tensor, Tensor, Tensor, Tensor]:
    ctx = _Ctx()
    y, z_loss, sel, counts = Fn.LatentMoEFunction.forward(ctx, x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up,
                                                          w_down_e, expert_bias, int(top_k), float(z_coef), False)
    if ctx.gather:
        raise RuntimeError("LMOE_TMA_GATHER is not available under torch.compile")
    (_xb, _wg, _wdn, _wup, _wgus, _wds, _wgu, _wde, logits, sel_s, weights, lse, x_sorted, h1, hidden, y_sorted, act_cat,
     h1_s) = ctx.saved_tensors
    return (y, z_loss, sel_s, counts.clone(), ctx.route.storage, ctx.status, logits, weights, lse, x_sorted, h1, hidden,
            y_sorted, act_cat, h1_s)


@latent_moe_fwd.register_fake
def _(x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias, top_k, z_coef):
    T, D, L, E, K, F, Fs = _dims(x, w_gate_up, w_down_s, top_k)
    P = Fn.padded_rows_of(T, K, E)
    new = lambda *shape, dtype: x.new_empty(shape, dtype=dtype)
    return (new(T, D, dtype=x.dtype), new(dtype=torch.float32), new(T, K, dtype=torch.int32), new(E, dtype=torch.int32),
            new(Fn.RouteTables.storage_numel(T, K, E), dtype=torch.int32), new(1, dtype=torch.int32),
            new(T, E, dtype=torch.float32), new(T, K, dtype=torch.float32), new(T, dtype=torch.float32),
            new(P, L, dtype=BF), new(P, 2 * F, dtype=BF), new(P, F, dtype=BF), new(P, L, dtype=BF),
            new(T, L + Fs, dtype=BF), new(T, 2 * Fs, dtype=BF))


@torch.library.custom_op("swamla_b200::latent_moe_bwd", mutates_args=())
def latent_moe_bwd(dy: Tensor, d_z: Optional[Tensor], x: Tensor, w_gate: Tensor, w_down: Tensor, w_up: Tensor,
                   w_gate_up_s: Tensor, w_down_s: Tensor, w_gate_up: Tensor, w_down_e: Tensor, route_storage: Tensor,
                   status: Tensor, sel: Tensor, logits: Tensor, weights: Tensor, lse: Tensor, x_sorted: Tensor, h1: Tensor,
                   hidden: Tensor, y_sorted: Tensor, act_cat: Tensor, h1_s: Tensor, top_k: int, z_coef: float
                   ) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    T, D, L, E, K, F, Fs = _dims(x, w_gate_up, w_down_s, top_k)
    ctx = _Ctx()
    ctx.shape = Fn.make_shape(T, D, L, E, K, F, Fs)
    ctx.route = Fn.RouteTables(ctx.shape, x.device, storage=route_storage)
    ctx.status, ctx.fp8_saved, ctx.gather, ctx.z_coef = status, None, False, float(z_coef)
    params = (x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e)
    ctx.dtypes = [t.dtype for t in params]
    ctx.saved_tensors = tuple(Fn._as_bf16(t) for t in params) + (logits, sel, weights, lse, x_sorted, h1, hidden, y_sorted,
                                                                 act_cat, h1_s)
    grads = Fn.LatentMoEFunction.backward(ctx, dy, d_z, None, None)[:8]
    # an operator's outputs must be fresh tensors (as_param may hand back a buffer unchanged, which is fresh already)
    return tuple(grads)


@latent_moe_bwd.register_fake
def _(dy, d_z, x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, route_storage, status, sel, logits,
      weights, lse, x_sorted, h1, hidden, y_sorted, act_cat, h1_s, top_k, z_coef):
    return tuple(torch.empty_like(t) for t in (x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e))


def _setup_context(ctx, inputs, output):
    (x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, _bias, top_k, z_coef) = inputs
    ctx.top_k, ctx.z_coef = int(top_k), float(z_coef)
    ctx.save_for_backward(x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, *output[2:3], *output[4:])
    ctx.set_materialize_grads(False)


def _backward(ctx, *grads):
    dy, d_z = grads[0], grads[1]
    (x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, sel, storage, status, logits, weights, lse,
     x_sorted, h1, hidden, y_sorted, act_cat, h1_s) = ctx.saved_tensors
    if dy is None:
        dy = x.new_zeros(x.shape)
    out = torch.ops.swamla_b200.latent_moe_bwd(dy, d_z, x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e,
                                               storage, status, sel, logits, weights, lse, x_sorted, h1, hidden, y_sorted,
                                               act_cat, h1_s, ctx.top_k, ctx.z_coef)
    return (*out, None, None, None)


latent_moe_fwd.register_autograd(_backward, setup_context=_setup_context)


def latent_moe_compiled(x2d, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias, top_k: int,
                        z_coef: float):
    """Same return values as ``functional.latent_moe`` through the custom operators (traceable without graph break)."""
    out = torch.ops.swamla_b200.latent_moe_fwd(x2d, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e,
                                               expert_bias, int(top_k), float(z_coef))
    return out[0], out[1], out[2], out[3]
