"""Routed experts in FP8 (e4m3) with per-tensor dynamic scaling.

Recipe: ``optimization/fp8_native.py:103-110`` ("tensorwise": one amax per tensor, scale = 448 / amax), which the
reference applies to ``nn.Linear`` modules through torchao; here it is applied to the six operands of the routed
expert GEMMs (x_sorted, gate_up weights, hidden, down weights in forward; d_y_sorted and d_h1 in backward).
Accumulation is fp32 in tensor memory and every GEMM output is bf16.  A tensor is quantised once and reused by
the forward, dgrad and wgrad GEMMs that read it.
"""
from __future__ import annotations

import torch

from . import _cabi
from ._cabi import ptr

BF = torch.bfloat16


def quantize(t: torch.Tensor, rows: int, row_len: int, n_tiles, stream):
    """bf16 [rows, row_len] -> (e4m3 bytes [rows, row_len], deq [1] = amax / 448).  ``n_tiles``: optional device
    int32 scalar; only the first 128 * n_tiles rows are touched (padded routed layout)."""
    q = torch.empty(rows, row_len, dtype=torch.uint8, device=t.device)
    scal = torch.empty(2, dtype=torch.float32, device=t.device)      # [amax, deq]
    _cabi.call("lmoe_fp8_quantize", ptr(t), rows, row_len, ptr(n_tiles), ptr(q), ptr(scal[0:1]), ptr(scal[1:2]), stream)
    return q, scal[1:2]


def experts_fwd(shape, route, x_sorted, wgu, wde, status, stream):
    """e4m3 gate_up (SwiGLU epilogue) + e4m3 down on the gathered rows x_sorted[P, L] (bf16, padded layout).
    Returns hidden, y_sorted and what backward needs."""
    P, E, L, F = route.padded_rows, shape.E, shape.L, shape.F
    dev = x_sorted.device
    bf = dict(dtype=BF, device=dev)
    xq, dq_x = quantize(x_sorted, P, L, route.n_tiles, stream)
    wguq, dq_wgu = quantize(wgu.reshape(E * L, 2 * F), E * L, 2 * F, None, stream)
    wdq, dq_wd = quantize(wde.reshape(E * F, L), E * F, L, None, stream)
    h1 = torch.empty(P, 2 * F, **bf)
    hidden = torch.empty(P, F, **bf)
    _cabi.call("lmoe_grouped_gateup_fp8", P, E, L, F, ptr(xq), ptr(wguq), ptr(dq_x), ptr(dq_wgu), ptr(route.tile_expert),
               ptr(route.n_tiles), ptr(h1), ptr(hidden), ptr(status), stream)
    hq, dq_h = quantize(hidden, P, F, route.n_tiles, stream)
    y_sorted = torch.empty(P, L, **bf)
    _cabi.call("lmoe_grouped_rows_fp8", P, E, F, L, ptr(hq), ptr(wdq), 1, ptr(dq_h), ptr(dq_wd), ptr(route.tile_expert),
               ptr(route.n_tiles), ptr(y_sorted), ptr(status), stream)
    saved = dict(xq=xq, dq_x=dq_x, wguq=wguq, dq_wgu=dq_wgu, wdq=wdq, dq_wd=dq_wd, hq=hq, dq_h=dq_h, h1=h1)
    return hidden, y_sorted, saved


def experts_bwd(shape, route, d_y_sorted, s, status, stream):
    """e4m3 dgrads and wgrads of the routed experts.  ``s``: the dict saved by experts_fwd."""
    P, E, L, F = route.padded_rows, shape.E, shape.L, shape.F
    dev = d_y_sorted.device
    bf = dict(dtype=BF, device=dev)
    dyq, dq_dy = quantize(d_y_sorted, P, L, route.n_tiles, stream)
    d_hidden = torch.empty(P, F, **bf)
    # d_hidden = d_y * Wd[e]^T: the down weights [E, F, L] read as [N = F rows, K = L] (K-major operand)
    _cabi.call("lmoe_grouped_rows_fp8", P, E, L, F, ptr(dyq), ptr(s["wdq"]), 0, ptr(dq_dy), ptr(s["dq_wd"]),
               ptr(route.tile_expert), ptr(route.n_tiles), ptr(d_hidden), ptr(status), stream)
    d_h1 = torch.empty(P, 2 * F, **bf)
    _cabi.call("lmoe_swiglu_bwd", P, F, ptr(s["h1"]), ptr(d_hidden), ptr(d_h1), 2 * F, ptr(route.n_tiles), stream)
    dh1q, dq_dh1 = quantize(d_h1, P, 2 * F, route.n_tiles, stream)
    d_x_sorted = torch.empty(P, L, **bf)
    # d_x_sorted = d_h1 * Wgu[e]^T: the gate_up weights [E, L, 2F] read as [N = L rows, K = 2F]
    _cabi.call("lmoe_grouped_rows_fp8", P, E, 2 * F, L, ptr(dh1q), ptr(s["wguq"]), 0, ptr(dq_dh1), ptr(s["dq_wgu"]),
               ptr(route.tile_expert), ptr(route.n_tiles), ptr(d_x_sorted), ptr(status), stream)
    d_w_gate_up = torch.empty(E, L, 2 * F, **bf)
    d_w_down = torch.empty(E, F, L, **bf)
    _cabi.call("lmoe_grouped_wgrad_fp8", P, E, L, 2 * F, ptr(s["xq"]), ptr(dh1q), ptr(s["dq_x"]), ptr(dq_dh1),
               ptr(route.pad_offsets), ptr(d_w_gate_up), ptr(status), stream)
    _cabi.call("lmoe_grouped_wgrad_fp8", P, E, F, L, ptr(s["hq"]), ptr(dyq), ptr(s["dq_h"]), ptr(dq_dy),
               ptr(route.pad_offsets), ptr(d_w_down), ptr(status), stream)
    return d_hidden, d_h1, d_x_sorted, d_w_gate_up, d_w_down
