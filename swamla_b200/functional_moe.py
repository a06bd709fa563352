"""The non-latent ``MoELayer`` of Orolol/swamla (``models/moe.py:294-559``) on the same sm_100a kernels.

Same routing, grouped GEMMs and row kernels as the latent layer, with the experts working at the model width:
there is no down/up projection, ``x`` itself is gathered into the padded expert layout and the weighted sum of the
expert outputs is added to the shared expert's output (``moe.py:366``).  Everything goes through the generic
entry points of ``include/lmoe.h`` (``lmoe_gemm_bf16``, ``lmoe_gemm_swiglu_bf16``, ``lmoe_grouped_*``,
``lmoe_combine_rows_add`` ...); no CPU fallback.
"""
from __future__ import annotations

import torch

from . import _cabi, functional
from ._cabi import ptr
from .functional import BF, RouteTables, _as_bf16, _stream, make_shape

_SMS = 148


def _split_k(M: int, N: int, K: int) -> int:
    """k-slices of a weight gradient [M, N] contracting over K rows: enough tiles to fill the SMs, each slice at least
    512 rows deep."""
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    return max(1, min(16, _SMS // max(tiles, 1), K // 512))


def _gemm(lib, M, N, K, A, lda, a_mn, B, ldb, b_mn, C, ldc, c_type, status, st, split_k=1):
    ws = None
    if split_k > 1:
        ws = torch.empty(lib.lmoe_gemm_workspace_bytes(M, N, split_k), dtype=torch.uint8, device=C.device)
    _cabi.call("lmoe_gemm_bf16", M, N, K, ptr(A), lda, a_mn, ptr(B), ldb, b_mn, ptr(C), ldc, c_type, split_k, ptr(ws),
               0 if ws is None else ws.numel(), ptr(status), st)


class MoEFunction(torch.autograd.Function):
    """y, aux_loss, sel, counts = f(x, w_gate, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias)."""

    @staticmethod
    def forward(ctx, x, w_gate, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias, top_k: int, z_coef: float):
        if not x.is_cuda:
            raise _cabi.LmoeError("the MoE path runs on a CUDA device only (no CPU fallback)")
        lib = _cabi.load()
        dev = x.device
        T, D = x.shape
        E, _, F2 = w_gate_up.shape
        F, Fs, K = F2 // 2, w_down_s.shape[1], top_k
        shape = make_shape(T, D, D, E, K, F, Fs)
        st = _stream()
        bf = dict(dtype=BF, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)

        xb = _as_bf16(x)
        wg, wgus, wds = _as_bf16(w_gate), _as_bf16(w_gate_up_s), _as_bf16(w_down_s)
        wgu, wde = _as_bf16(w_gate_up), _as_bf16(w_down_e)
        bias = expert_bias.to(torch.float32).contiguous()
        status = torch.zeros(1, dtype=torch.int32, device=dev)

        # router: fp32 logits, top-k, z-loss; routing tables                         (moe.py:357-358)
        logits = torch.empty(T, E, **f32)
        _gemm(lib, T, E, D, xb, D, 0, wg, D, 0, logits, E, _cabi.F32, status, st)
        sel = torch.empty(T, K, dtype=torch.int32, device=dev)
        weights = torch.empty(T, K, **f32)
        lse = torch.empty(T, **f32)
        z_partial = torch.empty((T + 7) // 8, **f32)
        z_loss = torch.empty(1, **f32)
        _cabi.call("lmoe_gate_topk_fwd", shape, ptr(logits), ptr(bias), float(z_coef), ptr(sel), ptr(weights), ptr(lse),
                   ptr(z_partial), ptr(z_loss), st)
        forced = functional._testing.forced_selection(logits)      # parity tests only
        if forced is not None:
            sel, weights = forced
        route = RouteTables(shape, dev)
        P = route.padded_rows
        ws = torch.empty(max(16, lib.lmoe_route_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
        _cabi.call("lmoe_route_permute", shape, ptr(sel), route.struct, ptr(ws), ws.numel(), st)
        # routed experts on x itself                                                 (moe.py:462-470, 509-532)
        x_sorted = torch.empty(P, D, **bf)
        _cabi.call("lmoe_gather_rows", ptr(xb), ptr(route.row_src), K, P, D, ptr(route.n_tiles), ptr(x_sorted), st)
        h1 = torch.empty(P, 2 * F, **bf)
        hidden = torch.empty(P, F, **bf)
        y_sorted = torch.empty(P, D, **bf)
        _cabi.call("lmoe_grouped_fwd", P, E, D, F, ptr(x_sorted), ptr(wgu), ptr(wde), ptr(route.tile_expert),
                   ptr(route.n_tiles), ptr(route.pad_offsets), ptr(h1), ptr(hidden), ptr(y_sorted), ptr(status), st)
        # shared expert                                                              (moe.py:351-354, 63-69)
        h1_s = torch.empty(T, 2 * Fs, **bf)
        hidden_s = torch.empty(T, Fs, **bf)
        _cabi.call("lmoe_gemm_swiglu_bf16", T, Fs, D, ptr(xb), D, ptr(wgus), D, ptr(h1_s), 2 * Fs, ptr(hidden_s), Fs,
                   ptr(status), st)
        y_shared = torch.empty(T, D, **bf)
        _gemm(lib, T, D, Fs, hidden_s, Fs, 0, wds, Fs, 0, y_shared, D, _cabi.BF16, status, st)
        # y = shared + sum_k w_k * expert_k(x)                                       (moe.py:534, 473-479, 366)
        y = torch.empty(T, D, **bf)
        _cabi.call("lmoe_combine_rows_add", ptr(y_sorted), ptr(route.pos), ptr(weights), ptr(y_shared), D, T, K, D, ptr(y),
                   D, st)

        ctx.shape, ctx.route, ctx.z_coef, ctx.status = shape, route, float(z_coef), status
        ctx.dtypes = [t.dtype for t in (x, w_gate, w_gate_up_s, w_down_s, w_gate_up, w_down_e)]
        ctx.save_for_backward(xb, wg, wgus, wds, wgu, wde, logits, sel, weights, lse, x_sorted, h1, hidden, y_sorted, h1_s,
                              hidden_s)
        ctx.mark_non_differentiable(sel, route.counts)
        functional.status_monitor.post(status, "MoE forward")
        out = y if x.dtype == BF else y.to(x.dtype)
        return out, z_loss.reshape(()), sel, route.counts

    @staticmethod
    def backward(ctx, dy, d_z, _d_sel, _d_counts):
        (xb, wg, wgus, wds, wgu, wde, logits, sel, weights, lse, x_sorted, h1, hidden, y_sorted, h1_s,
         hidden_s) = ctx.saved_tensors
        shape, route, status = ctx.shape, ctx.route, ctx.status
        T, D, E, K, F, Fs = shape.T, shape.D, shape.E, shape.K, shape.F, shape.Fs
        P = route.padded_rows
        dev = xb.device
        st = _stream()
        lib = _cabi.load()
        bf = dict(dtype=BF, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        if dy is None:
            dy = torch.zeros(T, D, **bf)
        dyb = _as_bf16(dy.reshape(T, D))
        dt = ctx.dtypes
        lin_dtype = torch.float32 if any(d == torch.float32 for d in dt[1:4]) else BF
        gtype = _cabi.F32 if lin_dtype == torch.float32 else _cabi.BF16
        lin = dict(dtype=lin_dtype, device=dev)
        ld_cat = 2 * Fs + E

        # shared expert: d_hidden_s = dy * Wd_s, SwiGLU adjoint -> dgrad_cat[:, :2Fs]; d_Wd_s = dy^T * hidden_s
        d_hidden_s = torch.empty(T, Fs, **bf)
        _gemm(lib, T, Fs, D, dyb, D, 0, wds, Fs, 1, d_hidden_s, Fs, _cabi.BF16, status, st)
        dgrad_cat = torch.empty(T, ld_cat, **bf)                   # [d_h1_s | d_logits]
        _cabi.call("lmoe_swiglu_bwd", T, Fs, ptr(h1_s), ptr(d_hidden_s), ptr(dgrad_cat), ld_cat, None, st)
        d_w_down_s = torch.empty(D, Fs, **lin)
        _gemm(lib, D, Fs, T, dyb, D, 1, hidden_s, Fs, 1, d_w_down_s, Fs, gtype, status, st, _split_k(D, Fs, T))
        # adjoint of the weighted sum: d_y_sorted = w * dy[t], d_w = <dy[t], y_sorted>
        d_y_sorted = torch.empty(P, D, **bf)
        d_weights = torch.empty(T, K, **f32)
        _cabi.call("lmoe_combine_bwd_rows", ptr(dyb), ptr(y_sorted), ptr(weights), ptr(route.row_src), P, K, D,
                   ptr(route.n_tiles), ptr(d_y_sorted), ptr(d_weights), st)
        # routed experts
        d_hidden = torch.empty(P, F, **bf)
        d_h1 = torch.empty(P, 2 * F, **bf)
        d_x_sorted = torch.empty(P, D, **bf)
        _cabi.call("lmoe_grouped_bwd_dgrad", P, E, D, F, ptr(d_y_sorted), ptr(h1), ptr(wgu), ptr(wde),
                   ptr(route.tile_expert), ptr(route.n_tiles), ptr(route.pad_offsets), ptr(d_hidden), ptr(d_h1), ptr(d_x_sorted), ptr(status), st)
        d_w_gate_up = torch.empty(E, D, 2 * F, **bf)
        d_w_down_e = torch.empty(E, F, D, **bf)
        _cabi.call("lmoe_grouped_bwd_wgrad", P, E, D, F, ptr(x_sorted), ptr(d_h1), ptr(hidden), ptr(d_y_sorted),
                   ptr(route.pad_offsets), ptr(d_w_gate_up), ptr(d_w_down_e), ptr(status), st)
        # router adjoint (+ z-loss) -> dgrad_cat[:, 2Fs:]   (the entry point places d_logits after 2Fs + L columns)
        cat_shape = make_shape(T, D, 0, E, K, F, Fs)
        dz = None if d_z is None else d_z.to(torch.float32).reshape(1).contiguous()
        _cabi.call("lmoe_gate_topk_bwd", cat_shape, ptr(logits), ptr(sel), ptr(weights), ptr(d_weights), ptr(lse), ptr(dz),
                   ctx.z_coef, ptr(dgrad_cat), st)
        # x side: dx = [d_h1_s | d_logits] * [Wgu_s ; Wg] + sum_k d_x_sorted ; [d_Wgu_s ; d_Wg] = [d_h1_s | d_logits]^T * x
        w_cat = torch.cat([wgus, wg], 0)                              # [2Fs + E, D]
        dx_dense = torch.empty(T, D, **bf)
        _gemm(lib, T, D, ld_cat, dgrad_cat, ld_cat, 0, w_cat, D, 1, dx_dense, D, _cabi.BF16, status, st)
        dx = torch.empty(T, D, **bf)
        _cabi.call("lmoe_combine_rows_add", ptr(d_x_sorted), ptr(route.pos), None, ptr(dx_dense), D, T, K, D, ptr(dx), D, st)
        d_w_cat = torch.empty(ld_cat, D, **lin)
        _gemm(lib, ld_cat, D, T, dgrad_cat, ld_cat, 1, xb, D, 1, d_w_cat, D, gtype, status, st, _split_k(ld_cat, D, T))
        d_w_gate_up_s, d_w_gate = d_w_cat[:2 * Fs], d_w_cat[2 * Fs:]

        def as_param(g, d):
            return g if g.dtype == d else g.to(d)

        functional.status_monitor.post(status, "MoE backward")
        return (as_param(dx, dt[0]), as_param(d_w_gate, dt[1]), as_param(d_w_gate_up_s, dt[2]),
                as_param(d_w_down_s, dt[3]), as_param(d_w_gate_up, dt[4]), as_param(d_w_down_e, dt[5]), None, None, None)


@torch.compiler.disable   # opaque to torch.compile: the layer runs as an eager call between compiled regions
def moe(x2d: torch.Tensor, w_gate, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias, top_k: int, z_coef: float):
    """Functional form on a [T, D] activation.  Returns (y [T,D], aux_loss scalar, sel [T,K] int32, counts [E] int32)."""
    return MoEFunction.apply(x2d, w_gate, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias, int(top_k),
                             float(z_coef))
