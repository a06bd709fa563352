"""Autograd binding of the LatentMoE path: forward and backward assembled from the C-ABI
entry points of ``liblmoe.so``.  PyTorch only provides device memory and the stream.

Forward follows ``models/moe.py:702-734`` of the reference (``LatentMoELayer.forward``); the
backward is the adjoint of each cited line (the reference defines it only through autograd and
not at all for its grouped GEMM, ``models/moe_triton.py:200-242``).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _cabi, _testing, status as status_monitor
from ._cabi import Route, Shape, ptr

BF = torch.bfloat16

# LMOE_TMA_GATHER=1: the gate_up GEMMs (forward and weight gradient) read the latent rows through TMA gathers
# (tile::gather4) driven by the routing table, with no gather kernel and no x_sorted buffer (P*L*2 bytes less memory).
# Off by default: results are bit-identical but four-row gathers of 128-byte rows sustained only about 8 GB/s per SM.
import os as _os
TMA_GATHER = _os.environ.get("LMOE_TMA_GATHER", "0") == "1"


def d_hidden_scratch(lib, P, L, F, **kw):
    """The routed dgrad stage needs no [P, F] scratch: the SwiGLU adjoint runs in the epilogue of the d_hidden GEMM
    (saved gate / up staged by TMA), or inside the chain kernel; d_hidden never reaches memory."""
    return None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _as_bf16(t: torch.Tensor) -> torch.Tensor:
    """bf16 copy of a float tensor through the library's cast kernel (no-op for bf16)."""
    if t.dtype == BF:
        return t.contiguous()
    if t.dtype != torch.float32:
        t = t.float()
    t = t.contiguous()
    out = torch.empty(t.shape, dtype=BF, device=t.device)
    _cabi.call("lmoe_cast_f32_to_bf16", ptr(t), ptr(out), t.numel(), _stream())
    return out


_SIDE_STREAMS = {}


class _Fork:
    """Two-stream scheduling inside one forward/backward: HBM-bound row kernels run on a side stream beside the
    tensor-bound GEMMs of the main (current) stream.  `to_side()` makes the side stream wait for everything queued
    on the main stream so far, `to_main()` the reverse.  Every tensor is allocated on the main stream and every
    side-stream section is joined before the function returns, so the caching allocator never recycles a block
    that side-stream work still uses."""

    def __init__(self, device):
        self.main = torch.cuda.current_stream(device)
        key = (device.index, self.main.cuda_stream)
        if key not in _SIDE_STREAMS:
            _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
        self.side = _SIDE_STREAMS[key]
        self.m, self.s = self.main.cuda_stream, self.side.cuda_stream

    def to_side(self):
        ev = torch.cuda.Event()
        ev.record(self.main)
        self.side.wait_event(ev)

    def to_main(self):
        ev = torch.cuda.Event()
        ev.record(self.side)
        self.main.wait_event(ev)


def padded_rows_of(T: int, K: int, E: int) -> int:
    """Static row count of the padded expert layout (what ``lmoe_padded_rows`` returns)."""
    return (T * K + 127) // 128 * 128 + E * 128


class RouteTables:
    """Device buffers behind an ``lmoe_route`` struct: one int32 allocation (``storage``), sliced."""

    @staticmethod
    def storage_numel(T: int, K: int, E: int) -> int:
        P = padded_rows_of(T, K, E)
        return sum((n + 3) // 4 * 4 for n in (E, E + 1, E + 1, 1, P // 128, T * K, T * K, P))

    def __init__(self, shape: Shape, device, storage: Optional[torch.Tensor] = None):
        T, K, E = shape.T, shape.K, shape.E
        self.padded_rows = padded_rows_of(T, K, E)
        i32 = dict(dtype=torch.int32, device=device)
        # one allocation, sliced; every slice starts 16-byte aligned
        sizes = dict(counts=E, offsets=E + 1, pad_offsets=E + 1, n_tiles=1, tile_expert=self.padded_rows // 128,
                     perm=T * K, pos=T * K, row_src=self.padded_rows)
        total = sum((n + 3) // 4 * 4 for n in sizes.values())
        self.storage = torch.empty(total, **i32) if storage is None else storage   # given: tables of an earlier forward
        off = 0
        for name, n in sizes.items():
            setattr(self, name, self.storage[off:off + n])
            off += (n + 3) // 4 * 4
        self.struct = Route(**{k: ptr(getattr(self, k)) for k in sizes})


def make_shape(T, D, L, E, K, F, Fs, n_shared=1) -> Shape:
    return Shape(T=T, D=D, L=L, E=E, K=K, F=F, Fs=Fs, n_shared=n_shared)


def check_status(status: torch.Tensor) -> None:
    """Reads one device status word now (synchronises); raises if a kernel reported a failure.  The layers use the
    non-blocking monitor in ``status.py`` instead; this form serves tests and callers of the functional API."""
    code = int(status.item())
    if code != 0:
        raise _cabi.LmoeError(f"device status {code}: {_cabi.status_string(code)}")


class LatentMoEFunction(torch.autograd.Function):
    """y, aux_loss, sel = f(x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias)."""

    @staticmethod
    def forward(ctx, x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias, top_k: int,
                z_coef: float, fp8: bool = False):
        if not x.is_cuda:
            raise _cabi.LmoeError("the LatentMoE path runs on a CUDA device only (no CPU fallback)")
        lib = _cabi.load()
        dev = x.device
        T, D = x.shape
        E, L, F2 = w_gate_up.shape
        F = F2 // 2
        Fs = w_down_s.shape[1]
        shape = make_shape(T, D, L, E, top_k, F, Fs)
        st = _stream()

        xb = _as_bf16(x)
        wg, wdn, wup = _as_bf16(w_gate), _as_bf16(w_down), _as_bf16(w_up)
        wgus, wds = _as_bf16(w_gate_up_s), _as_bf16(w_down_s)
        wgu, wde = _as_bf16(w_gate_up), _as_bf16(w_down_e)
        bias = expert_bias.to(torch.float32).contiguous()

        status = torch.zeros(1, dtype=torch.int32, device=dev)
        bf = dict(dtype=BF, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)

        # router + latent down-projection
        logits = torch.empty(T, E, **f32)
        # one extra row after the T latent rows: zeros that the pad rows of the routed layout read when the gather runs
        # inside the GEMM's TMA producer
        x_latent_ext = torch.empty(T + 1, L, **bf)
        gather = TMA_GATHER and not fp8 and L % 128 == 0   # whole 128-column tiles of the weight gradient
        if gather:
            x_latent_ext[T].zero_()     # (the gather kernel of the default path writes the pad rows' zeros itself)
        x_latent = x_latent_ext[:T]
        _cabi.call("lmoe_xproj_fwd", shape, ptr(xb), ptr(wg), ptr(wdn), ptr(logits), ptr(x_latent), ptr(status), st)
        sel = torch.empty(T, top_k, dtype=torch.int32, device=dev)
        weights = torch.empty(T, top_k, **f32)
        lse = torch.empty(T, **f32)
        z_partial = torch.empty((T + 7) // 8, **f32)
        z_loss = torch.empty(1, **f32)
        route = RouteTables(shape, dev)
        P = route.padded_rows
        ws = torch.empty(max(16, lib.lmoe_route_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
        x_sorted = None if (gather and not _testing.capturing()) else torch.empty(P, L, **bf)
        h1_s = torch.empty(T, 2 * Fs, **bf)
        act_cat = torch.empty(T, L + Fs, **bf)
        # One stream in forward: the routing kernels use static shared memory that does not fit on an SM beside a GEMM
        # CTA, so on a second stream they would only wait for the shared-expert GEMM to drain.
        _cabi.call("lmoe_gate_topk_fwd", shape, ptr(logits), ptr(bias), float(z_coef), ptr(sel), ptr(weights), ptr(lse),
                   ptr(z_partial), ptr(z_loss), st)
        forced = _testing.forced_selection(logits)
        if forced is not None:
            sel, weights = forced
        _cabi.call("lmoe_route_permute", shape, ptr(sel), route.struct, ptr(ws), ws.numel(), st)
        if x_sorted is not None:
            _cabi.call("lmoe_gather_rows", ptr(x_latent), ptr(route.row_src), top_k, P, L, ptr(route.n_tiles),
                       ptr(x_sorted), st)
        _cabi.call("lmoe_shared_gateup_fwd", shape, ptr(xb), ptr(wgus), ptr(h1_s), ptr(act_cat), ptr(status), st)

        # routed experts in the padded layout
        fp8_saved = None
        if fp8:
            from . import fp8 as fp8_path
            hidden, y_sorted, fp8_saved = fp8_path.experts_fwd(shape, route, x_sorted, wgu, wde, status, st)
            h1 = fp8_saved["h1"]
        else:
            h1 = torch.empty(P, 2 * F, **bf)
            hidden = torch.empty(P, F, **bf)
            y_sorted = torch.empty(P, L, **bf)
            if gather:
                # the TMA unit gathers the latent rows of every tile (row_src holds t*K + k; pad rows -> the zero row)
                _cabi.call("lmoe_grouped_fwd_gather", P, E, L, F, ptr(x_latent_ext), T + 1, ptr(route.row_src), 1, top_k, T,
                           ptr(wgu), ptr(wde), ptr(route.tile_expert), ptr(route.n_tiles), ptr(h1), ptr(hidden),
                           ptr(y_sorted), ptr(status), st)
            else:
                _cabi.call("lmoe_grouped_fwd", P, E, L, F, ptr(x_sorted), ptr(wgu), ptr(wde), ptr(route.tile_expert),
                           ptr(route.n_tiles), ptr(route.pad_offsets), ptr(h1), ptr(hidden), ptr(y_sorted), ptr(status), st)

        # weighted combine, up-projection, shared down-projection, add
        y = torch.empty(T, D, **bf)
        _cabi.call("lmoe_combine_out_fwd", shape, ptr(y_sorted), route.struct, ptr(weights), ptr(act_cat), ptr(wds),
                   ptr(wup), ptr(y), ptr(status), st)
        routed, hidden_s = act_cat[:, :L], act_cat[:, L:]

        ctx.shape = shape
        ctx.route = route
        ctx.fp8_saved = fp8_saved
        ctx.z_coef = float(z_coef)
        ctx.status = status
        ctx.dtypes = [t.dtype for t in (x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e)]
        if fp8:   # the e4m3 copies replace the bf16 operands of the routed GEMMs
            none = torch.empty(0, **bf)
            ctx.save_for_backward(xb, wg, wdn, wup, wgus, wds, none, none, logits, sel, weights, lse, none, h1, none,
                                  y_sorted, act_cat, h1_s)
        else:
            ctx.save_for_backward(xb, wg, wdn, wup, wgus, wds, wgu, wde, logits, sel, weights, lse,
                                  x_latent_ext if gather else x_sorted, h1, hidden, y_sorted, act_cat, h1_s)
        ctx.gather = gather
        ctx.mark_non_differentiable(sel, route.counts)
        _testing.capture(logits=logits, x_latent=x_latent, sel=sel, weights=weights, lse=lse, route=route,
                         x_sorted=x_sorted, h1=h1, hidden=hidden, y_sorted=y_sorted, h1_s=h1_s, hidden_s=hidden_s,
                         routed=routed, status=status)
        status_monitor.post(status, "LatentMoE forward")
        out = y if x.dtype == BF else y.to(x.dtype)
        return out, z_loss.reshape(()), sel, route.counts

    @staticmethod
    def backward(ctx, dy, d_z, _d_sel, _d_counts):
        (xb, wg, wdn, wup, wgus, wds, wgu, wde, logits, sel, weights, lse, x_sorted, h1, hidden, y_sorted, act_cat,
         h1_s) = ctx.saved_tensors
        shape, route, status = ctx.shape, ctx.route, ctx.status
        T, D, L, E, K, F, Fs = shape.T, shape.D, shape.L, shape.E, shape.K, shape.F, shape.Fs
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
        # dense linears share one gradient dtype (fp32 master weights or bf16 module)
        lin_dtype = torch.float32 if any(d == torch.float32 for d in dt[1:6]) else BF
        gtype = _cabi.F32 if lin_dtype == torch.float32 else _cabi.BF16
        lin = dict(dtype=lin_dtype, device=dev)
        ws = torch.empty(max(16, lib.lmoe_wgrad_workspace_bytes(shape)), dtype=torch.uint8, device=dev)

        # All buffers first (main stream), then the schedule: GEMMs on the main stream, row kernels beside them.
        fork = _Fork(dev)
        d_routed = torch.empty(T, L, **bf)
        d_w_up = torch.empty(D, L, **lin)
        d_w_down_s = torch.empty(D, Fs, **lin)
        # the three x-side gradients live side by side in dgrad_cat[T, 2Fs+L+E]
        dgrad_cat = torch.empty(T, 2 * Fs + L + E, **bf)
        d_h1_s, d_x_latent, d_logits = dgrad_cat[:, :2 * Fs], dgrad_cat[:, 2 * Fs:2 * Fs + L], dgrad_cat[:, 2 * Fs + L:]
        d_y_sorted = torch.empty(P, L, **bf)
        d_weights = torch.empty(T, K, **f32)
        dx = torch.empty(T, D, **bf)
        d_w_gate_up_s = torch.empty(2 * Fs, D, **lin)
        d_w_down = torch.empty(L, D, **lin)
        d_w_gate = torch.empty(E, D, **lin)
        dz = None
        if d_z is not None:
            dz = d_z.to(torch.float32).reshape(1).contiguous()
        ld_cat = 2 * Fs + L + E

        # output stage dgrads, then: [adjoint of the combine] beside [output-stage weight gradients]
        # d_hidden_s = NULL: the shared expert's SwiGLU adjoint runs in the epilogue of the d_hidden_s GEMM
        _cabi.call("lmoe_combine_out_bwd_dgrad", shape, ptr(dyb), ptr(wup), ptr(wds), ptr(h1_s), ptr(d_routed),
                   None, ptr(dgrad_cat), ptr(status), st)
        fork.to_side()
        _cabi.call("lmoe_combine_bwd", shape, ptr(d_routed), ptr(y_sorted), ptr(weights), route.struct, ptr(d_y_sorted),
                   ptr(d_weights), fork.s)
        _cabi.call("lmoe_combine_out_bwd_wgrad", shape, ptr(dyb), ptr(act_cat), ptr(d_w_up), ptr(d_w_down_s), gtype,
                   ptr(ws), ws.numel(), ptr(status), st)
        fork.to_main()

        if ctx.fp8_saved is not None:
            from . import fp8 as fp8_path
            d_hidden, d_h1, d_x_sorted, d_w_gate_up, d_w_down_e = fp8_path.experts_bwd(shape, route, d_y_sorted,
                                                                                       ctx.fp8_saved, status, st)
            _cabi.call("lmoe_unpermute_sum_bwd", shape, ptr(d_x_sorted), route.struct, ptr(dgrad_cat), st)
            _cabi.call("lmoe_gate_topk_bwd", shape, ptr(logits), ptr(sel), ptr(weights), ptr(d_weights), ptr(lse), ptr(dz),
                       ctx.z_coef, ptr(dgrad_cat), st)
        else:
            d_h1 = torch.empty(P, 2 * F, **bf)
            d_x_sorted = torch.empty(P, L, **bf)
            d_w_gate_up = torch.empty(E, L, 2 * F, **bf)
            d_w_down_e = torch.empty(E, F, L, **bf)
            te, nt = ptr(route.tile_expert), ptr(route.n_tiles)
            # d_h1 = swiglu'(h1, d_y_sorted * Wd[e]^T), d_x_sorted = d_h1 * Wgu[e]^T: one chained kernel
            d_hidden = d_hidden_scratch(lib, P, L, F, **bf)
            _cabi.call("lmoe_grouped_bwd_dgrad", P, E, L, F, ptr(d_y_sorted), ptr(h1), ptr(wgu), ptr(wde), te, nt, ptr(route.pad_offsets),
                       ptr(d_hidden), ptr(d_h1), ptr(d_x_sorted), ptr(status), st)
            # [gather adjoint + router adjoint] beside [routed weight gradients]
            fork.to_side()
            _cabi.call("lmoe_unpermute_sum_bwd", shape, ptr(d_x_sorted), route.struct, ptr(dgrad_cat), fork.s)
            _cabi.call("lmoe_gate_topk_bwd", shape, ptr(logits), ptr(sel), ptr(weights), ptr(d_weights), ptr(lse), ptr(dz),
                       ctx.z_coef, ptr(dgrad_cat), fork.s)
            if ctx.gather:   # x_sorted is the latent rows [T + 1, L] here, gathered by the TMA unit
                _cabi.call("lmoe_grouped_bwd_wgrad_gather", P, E, L, F, ptr(x_sorted), T + 1, ptr(route.row_src), 1, K, T,
                           ptr(d_h1), ptr(hidden), ptr(d_y_sorted), ptr(route.pad_offsets), ptr(d_w_gate_up),
                           ptr(d_w_down_e), ptr(status), st)
            else:
                _cabi.call("lmoe_grouped_bwd_wgrad", P, E, L, F, ptr(x_sorted), ptr(d_h1), ptr(hidden), ptr(d_y_sorted),
                           ptr(route.pad_offsets), ptr(d_w_gate_up), ptr(d_w_down_e), ptr(status), st)
            fork.to_main()

        # x side: dx and the three weight gradients that contract with x
        _cabi.call("lmoe_xside_bwd", shape, ptr(dgrad_cat), ptr(wgus), ptr(wdn), ptr(wg), ptr(xb), ptr(dx),
                   ptr(d_w_gate_up_s), ptr(d_w_down), ptr(d_w_gate), gtype, ptr(ws), ws.numel(), ptr(status), st)

        _testing.capture(d_routed=d_routed, d_h1_s=d_h1_s, d_y_sorted=d_y_sorted, d_weights=d_weights, d_h1=d_h1,
                         d_x_sorted=d_x_sorted, d_x_latent=d_x_latent, d_logits=d_logits)
        status_monitor.post(status, "LatentMoE backward")
        def as_param(g, d):
            return g if g.dtype == d else g.to(d)

        grads = (
            as_param(dx, dt[0]), as_param(d_w_gate, dt[1]), as_param(d_w_down, dt[2]), as_param(d_w_up, dt[3]),
            as_param(d_w_gate_up_s, dt[4]), as_param(d_w_down_s, dt[5]), as_param(d_w_gate_up, dt[6]),
            as_param(d_w_down_e, dt[7]),
        )
        return grads + (None, None, None, None)


@torch.compiler.disable   # opaque to torch.compile: the layer runs as an eager call between compiled regions
def latent_moe(x2d: torch.Tensor, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias,
               top_k: int, z_coef: float, fp8: bool = False):
    """Functional form on a [T, D] activation.  Returns (y [T,D], aux_loss scalar, sel [T,K] int32, counts [E] int32).
    ``fp8``: run the routed expert GEMMs in e4m3 with per-tensor scaling (latent and routed hidden dims % 128 == 0)."""
    return LatentMoEFunction.apply(x2d, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up, w_down_e, expert_bias,
                                   int(top_k), float(z_coef), bool(fp8))
