"""``x + ffn(ffn_norm(x))``: the feed-forward half of the reference's block (``models/mla_block.py:83-85, 159``) with
the RMSNorm (``models/normalization.py:25-39``) and the residual add as fused row kernels of ``liblmoe.so``.

``NormedResidualFFN(ffn, dim, eps)`` owns the norm weight under the reference's name (``ffn_norm.weight``) and wraps any
feed-forward module (here: ``LatentMoELayer`` / ``MoELayer``).  Forward: one kernel for the norm (one read of x, one
write), the layer, one kernel for the add.  Backward: ONE kernel for the adjoint of the norm and the residual branch
(``dx = norm_bwd(d_xn) + dy``), plus a deterministic two-stage sum for the weight gradient.  No CPU fallback.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _cabi
from ._cabi import ptr
from .functional import BF, _as_bf16, _stream


class _NormAndPass(torch.autograd.Function):
    """(xn, x_pass) = (rmsnorm(x) * weight, x).  ``x_pass`` is x itself, handed on to the residual add, so that the
    backward sees the gradient of both branches in one call and adds them inside the norm's backward kernel."""

    @staticmethod
    def forward(ctx, x2d, weight, eps: float):
        if not x2d.is_cuda:
            raise _cabi.LmoeError("the fused norm runs on a CUDA device only (no CPU fallback)")
        T, D = x2d.shape
        xb = _as_bf16(x2d)
        w32 = weight.detach().to(torch.float32).contiguous()
        xn = torch.empty(T, D, dtype=BF, device=x2d.device)
        rstd = torch.empty(T, dtype=torch.float32, device=x2d.device)
        _cabi.call("lmoe_rmsnorm_fwd", ptr(xb), ptr(w32), float(eps), T, D, ptr(xn), ptr(rstd), _stream())
        ctx.save_for_backward(xb, w32, rstd)
        ctx.dtypes = (x2d.dtype, weight.dtype)
        # the residual branch keeps the input's dtype: under the reference's autocast training the residual stream
        # is fp32 (train.py:1195, normalization.py:25-39) and must not be rounded to bf16 at every block
        return (xn if x2d.dtype == BF else xn.to(x2d.dtype)), (xb if x2d.dtype == BF else x2d)

    @staticmethod
    def backward(ctx, d_xn, d_pass):
        xb, w32, rstd = ctx.saved_tensors
        T, D = xb.shape
        dev = xb.device
        lib = _cabi.load()
        if d_xn is None:
            d_xn = torch.zeros(T, D, dtype=BF, device=dev)
        g = _as_bf16(d_xn)
        x_dtype, w_dtype = ctx.dtypes
        # bf16 stream: the residual gradient is added inside the kernel; wider stream: added afterwards in that dtype
        r = None if (d_pass is None or x_dtype != BF) else _as_bf16(d_pass)
        dx = torch.empty(T, D, dtype=BF, device=dev)
        d_w = torch.empty(D, dtype=torch.float32, device=dev)
        ws = torch.empty(lib.lmoe_rmsnorm_workspace_bytes(D), dtype=torch.uint8, device=dev)
        _cabi.call("lmoe_rmsnorm_bwd", ptr(xb), ptr(w32), ptr(rstd), ptr(g), ptr(r), T, D, ptr(dx), ptr(d_w), ptr(ws),
                   ws.numel(), _stream())
        if x_dtype != BF:
            dx = dx.to(x_dtype)
            if d_pass is not None:
                dx = dx + d_pass.to(x_dtype)
        return dx, (d_w if w_dtype == torch.float32 else d_w.to(w_dtype)), None


class _Add(torch.autograd.Function):
    """out = a + b (fused kernel for bf16 rows; a wider residual stream is added in its own dtype); both inputs receive
    the output's gradient as it is."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.dtypes = (a.dtype, b.dtype)
        if a.dtype != BF:                     # fp32 residual stream: the add stays in that dtype
            return a + b.to(a.dtype)
        ab, bb = _as_bf16(a), _as_bf16(b)
        out = torch.empty_like(ab)
        _cabi.call("lmoe_add_bf16", ptr(ab), ptr(bb), ptr(out), ab.numel(), _stream())
        ctx.dtypes = (a.dtype, b.dtype)
        return out

    @staticmethod
    def backward(ctx, d_out):
        da, db = ctx.dtypes
        return (d_out if d_out.dtype == da else d_out.to(da)), (d_out if d_out.dtype == db else d_out.to(db))


class _NormWeight(nn.Module):
    """Holds ``weight`` [dim] (ones at init) under the reference's parameter name ``ffn_norm.weight``."""

    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))


class NormedResidualFFN(nn.Module):
    """``forward(x) = x + ffn(rmsnorm(x))`` for x[B, S, D]; output dtype = input dtype, arithmetic bf16/fp32.
    ``state_dict`` keys: ``ffn_norm.weight`` and ``ffn.*`` as in the reference block."""

    def __init__(self, ffn: nn.Module, dim: int, eps: float = 1e-6):
        super().__init__()
        if dim % 8 or dim > 2048:
            raise ValueError("kernel constraints: dim a multiple of 8, at most 2048")
        self.ffn_norm = _NormWeight(dim, eps)
        self.ffn = ffn

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, D = x.shape
        xn, x_pass = _norm_and_pass(x.reshape(-1, D), self.ffn_norm.weight, self.ffn_norm.eps)
        y = self.ffn(xn.view(B, S, D))
        out = _add(x_pass, y.reshape(-1, D))
        return (out if x.dtype == BF else out.to(x.dtype)).view(B, S, D)


@torch.compiler.disable   # opaque to torch.compile (ctypes calls into the kernel library)
def _norm_and_pass(x2d, weight, eps):
    return _NormAndPass.apply(x2d, weight, eps)


@torch.compiler.disable
def _add(a, b):
    return _Add.apply(a, b)
