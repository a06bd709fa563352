"""Expert-parallel LatentMoE: the routed experts sharded over the ranks of a process group.

The reference has data parallelism only (``train.py:944-949``); expert parallelism is the sharding its
design note sketches (``aidocs/moe.md:940-997``).  Partition: every rank keeps its own tokens end to end
(router, latent projections, shared expert, combine) and owns the contiguous expert block
``[rank*E/G, (rank+1)*E/G)`` of ``experts.gate_up_weight`` / ``experts.down_weight``.  One exchange step each way:

  forward   dispatch all-to-all of latent rows (canonical expert order is also destination-rank order,
            so the send buffer is the expert-sorted row list) -> local grouped experts -> combine all-to-all
  backward  the same two exchanges with gradients

Tokens travel in latent space (L = D/4 elements per row).  Row counts are exchanged with one all-gather of
the per-expert histogram; the split sizes NCCL needs are read on the host once per forward (the only host
synchronisation), after the shared-expert GEMM has been queued so the GPU stays busy meanwhile.
Gradients of the replicated parameters are local sums (averaging them across ranks is the data-parallel
wrapper's job, as in the reference); gradients of the expert shard are complete on the owning rank.
"""
from __future__ import annotations

import os
from typing import List, Tuple

import torch
import torch.distributed as dist

from . import _cabi, status as status_monitor
from ._cabi import Route, ptr
from .functional import BF, RouteTables, _as_bf16, _stream, d_hidden_scratch, make_shape


def expert_shard_parameter_names(model: torch.nn.Module) -> List[str]:
    """Names (as in ``model.named_parameters()``) of the expert-sharded parameters of every expert-parallel layer."""
    return [n for n, p_ in model.named_parameters() if getattr(p_, "expert_shard", False)]


def ddp_ignore_expert_shards(model: torch.nn.Module, average_like_ddp: bool = True) -> List[str]:
    """Prepare ``model`` for ``DistributedDataParallel`` (the reference wraps the model at ``train.py:944-949``).

    The expert shards are different tensors on every rank and their gradients are already complete on the owner
    (sums over the tokens of all ranks), so DDP must neither broadcast nor all-reduce them: their names are put into
    ``model._ddp_params_and_buffers_to_ignore``, which DDP reads at construction.  DDP AVERAGES the replicated
    parameters' gradients over the G ranks; with ``average_like_ddp`` the shard gradients are divided by G through a
    gradient hook so that all parameters see the same loss scaling (mean over the global batch).
    Call it once, before wrapping; returns the ignored names."""
    names = expert_shard_parameter_names(model)
    ignored = list(getattr(model, "_ddp_params_and_buffers_to_ignore", []))
    model._ddp_params_and_buffers_to_ignore = ignored + [n for n in names if n not in ignored]
    if average_like_ddp:
        for mod in model.modules():
            group = getattr(mod, "ep_group", None)
            if group is None or not hasattr(mod, "gate_up_weight"):
                continue
            scale = 1.0 / dist.get_world_size(group)
            for p_ in (mod.gate_up_weight, mod.down_weight):
                if not getattr(p_, "_ep_grad_hook", False):
                    p_.register_hook(lambda g, s=scale: g * s)
                    p_._ep_grad_hook = True
    return names


def gather_full_state_dict(model: torch.nn.Module) -> dict:
    """``model.state_dict()`` with every expert shard replaced by the full [E_global, ...] tensor of the reference's
    layout (``models/moe.py:582-586``), identical on every rank.  A COLLECTIVE: every rank of each layer's
    expert-parallel group must call it (``model.state_dict()`` itself is local and returns the rank's block).  In the
    reference's loop (``train.py:1470-1506``) call it on all ranks before the ``master_process`` guard and save the
    result on rank 0."""
    state = model.state_dict()
    for prefix, mod in model.named_modules():
        group = getattr(mod, "ep_group", None)
        if group is None or not hasattr(mod, "gate_up_weight") or getattr(mod, "ep_size", 1) == 1:
            continue
        for name in ("gate_up_weight", "down_weight"):
            key = f"{prefix}.{name}" if prefix else name
            shard = state[key].detach().contiguous()
            full = torch.empty((mod.ep_size * shard.shape[0],) + tuple(shard.shape[1:]), dtype=shard.dtype,
                               device=shard.device)
            dist.all_gather_into_tensor(full, shard, group=group)           # rank order = expert order
            state[key] = full
    return state


def splits_from_counts(counts_all: torch.Tensor, rank: int) -> Tuple[List[int], List[int]]:
    """counts_all[G, E] (rows every source routes to every expert) -> (send_splits, recv_splits) of ``rank``:
    rows it sends to each destination rank and rows it receives from each source rank."""
    G, E = counts_all.shape
    El = E // G
    per_dest = counts_all.view(G, G, El).sum(-1)          # [source, destination]
    return per_dest[rank].tolist(), per_dest[:, rank].tolist()


def _a2a(rows_in: torch.Tensor, out_rows: int, in_splits, out_splits, group) -> torch.Tensor:
    out = torch.empty(out_rows, rows_in.shape[1], dtype=rows_in.dtype, device=rows_in.device)
    dist.all_to_all_single(out, rows_in, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
    return out


class ExpertParallelLatentMoE(torch.autograd.Function):
    """Same signature as ``functional.LatentMoEFunction`` with the expert weights being the local shard."""

    @staticmethod
    def forward(ctx, x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc, expert_bias,
                top_k: int, z_coef: float, group):
        if not x.is_cuda:
            raise _cabi.LmoeError("the LatentMoE path runs on a CUDA device only (no CPU fallback)")
        lib = _cabi.load()
        G, rank = dist.get_world_size(group), dist.get_rank(group)
        dev = x.device
        T, D = x.shape
        El, L, F2 = w_gate_up_loc.shape
        E, F, Fs, K = El * G, F2 // 2, w_down_s.shape[1], top_k
        shape = make_shape(T, D, L, E, K, F, Fs)
        st = _stream()
        bf = dict(dtype=BF, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)

        xb = _as_bf16(x)
        wg, wdn, wup = _as_bf16(w_gate), _as_bf16(w_down), _as_bf16(w_up)
        wgus, wds = _as_bf16(w_gate_up_s), _as_bf16(w_down_s)
        wgu, wde = _as_bf16(w_gate_up_loc), _as_bf16(w_down_e_loc)
        bias = expert_bias.to(torch.float32).contiguous()
        status = torch.zeros(1, **i32)

        # local router over the GLOBAL expert set
        logits = torch.empty(T, E, **f32)
        x_latent = torch.empty(T, L, **bf)
        _cabi.call("lmoe_xproj_fwd", shape, ptr(xb), ptr(wg), ptr(wdn), ptr(logits), ptr(x_latent), ptr(status), st)
        sel = torch.empty(T, K, **i32)
        weights = torch.empty(T, K, **f32)
        lse = torch.empty(T, **f32)
        z_partial = torch.empty((T + 7) // 8, **f32)
        z_loss = torch.empty(1, **f32)
        _cabi.call("lmoe_gate_topk_fwd", shape, ptr(logits), ptr(bias), float(z_coef), ptr(sel), ptr(weights), ptr(lse),
                   ptr(z_partial), ptr(z_loss), st)
        route = RouteTables(shape, dev)
        ws = torch.empty(max(16, lib.lmoe_route_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
        _cabi.call("lmoe_route_permute", shape, ptr(sel), route.struct, ptr(ws), ws.numel(), st)
        counts_all = torch.empty(G, E, **i32)
        dist.all_gather_into_tensor(counts_all, route.counts.contiguous(), group=group)

        # work that needs no routing result goes first: it keeps the GPU busy across the host read below
        h1_s = torch.empty(T, 2 * Fs, **bf)
        act_cat = torch.empty(T, L + Fs, **bf)
        _cabi.call("lmoe_shared_gateup_fwd", shape, ptr(xb), ptr(wgus), ptr(h1_s), ptr(act_cat), ptr(status), st)
        n_send = T * K
        send_rows = torch.empty(n_send, L, **bf)      # expert-sorted rows = destination-rank order
        _cabi.call("lmoe_gather_rows", ptr(x_latent), ptr(route.perm), K, n_send, L, None, ptr(send_rows), st)
        inv = torch.empty(n_send, **i32)              # flat index t*K+k -> position in send order
        _cabi.call("lmoe_invert_perm", ptr(route.perm), n_send, ptr(inv), st)

        send_splits, recv_splits = splits_from_counts(counts_all.cpu(), rank)   # the one host sync
        n_recv = int(sum(recv_splits))
        recv_rows = _a2a(send_rows, n_recv, send_splits, recv_splits, group)    # dispatch

        # regroup the received rows expert by expert (padded) and run the local experts
        P = (n_recv + 127) // 128 * 128 + El * 128
        recv_pos = torch.empty(max(n_recv, 1), **i32)
        row_src = torch.empty(P, **i32)
        pad_offsets = torch.empty(El + 1, **i32)
        tile_expert = torch.empty(P // 128, **i32)
        n_tiles = torch.empty(1, **i32)
        _cabi.call("lmoe_ep_plan", ptr(counts_all), G, E, rank, ptr(recv_pos), ptr(row_src), ptr(pad_offsets),
                   ptr(tile_expert), ptr(n_tiles), st)
        x_sorted = torch.empty(P, L, **bf)
        h1 = torch.empty(P, 2 * F, **bf)
        hidden = torch.empty(P, F, **bf)
        y_sorted = torch.empty(P, L, **bf)
        y_recv = torch.empty(n_recv, L, **bf)
        if n_recv > 0:
            _cabi.call("lmoe_gather_rows", ptr(recv_rows), ptr(row_src), 1, P, L, ptr(n_tiles), ptr(x_sorted), st)
            _cabi.call("lmoe_grouped_fwd", P, El, L, F, ptr(x_sorted), ptr(wgu), ptr(wde), ptr(tile_expert), ptr(n_tiles), ptr(pad_offsets),
                       ptr(h1), ptr(hidden), ptr(y_sorted), ptr(status), st)
            _cabi.call("lmoe_gather_rows", ptr(y_sorted), ptr(recv_pos), 1, n_recv, L, None, ptr(y_recv), st)
        y_back = _a2a(y_recv, n_send, recv_splits, send_splits, group)          # combine

        # weighted combine over the returned rows, up-projection, shared down-projection, add
        y = torch.empty(T, D, **bf)
        back_route = Route(counts=ptr(route.counts), offsets=ptr(route.offsets), perm=ptr(route.perm),
                           pad_offsets=ptr(route.pad_offsets), pos=ptr(inv), row_src=ptr(route.row_src),
                           tile_expert=ptr(route.tile_expert), n_tiles=ptr(route.n_tiles))
        _cabi.call("lmoe_combine_out_fwd", shape, ptr(y_back), back_route, ptr(weights), ptr(act_cat), ptr(wds),
                   ptr(wup), ptr(y), ptr(status), st)

        ctx.shape, ctx.route, ctx.group, ctx.z_coef, ctx.status = shape, route, group, float(z_coef), status
        ctx.splits = (send_splits, recv_splits, n_recv, P, El)
        ctx.dtypes = [t.dtype for t in (x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc)]
        ctx.save_for_backward(xb, wg, wdn, wup, wgus, wds, wgu, wde, logits, sel, weights, lse, inv, y_back, act_cat,
                              h1_s, x_sorted, h1, hidden, recv_pos, row_src, pad_offsets, tile_expert, n_tiles)
        global_counts = counts_all.sum(0, dtype=torch.int32)
        ctx.mark_non_differentiable(sel, global_counts)
        status_monitor.post(status, "expert-parallel LatentMoE forward")
        out = y if x.dtype == BF else y.to(x.dtype)
        return out, z_loss.reshape(()), sel, global_counts

    @staticmethod
    def backward(ctx, dy, d_z, _d_sel, _d_counts):
        (xb, wg, wdn, wup, wgus, wds, wgu, wde, logits, sel, weights, lse, inv, y_back, act_cat, h1_s, x_sorted, h1,
         hidden, recv_pos, row_src, pad_offsets, tile_expert, n_tiles) = ctx.saved_tensors
        shape, route, group, status = ctx.shape, ctx.route, ctx.group, ctx.status
        send_splits, recv_splits, n_recv, P, El = ctx.splits
        T, D, L, E, K, F, Fs = shape.T, shape.D, shape.L, shape.E, shape.K, shape.F, shape.Fs
        dev = xb.device
        st = _stream()
        lib = _cabi.load()
        bf = dict(dtype=BF, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        if dy is None:
            dy = torch.zeros(T, D, **bf)
        dyb = _as_bf16(dy.reshape(T, D))
        dt = ctx.dtypes
        lin_dtype = torch.float32 if any(d == torch.float32 for d in dt[1:6]) else BF
        gtype = _cabi.F32 if lin_dtype == torch.float32 else _cabi.BF16
        lin = dict(dtype=lin_dtype, device=dev)
        ws = torch.empty(max(16, lib.lmoe_wgrad_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
        n_send = T * K

        # output stage (local)
        d_routed = torch.empty(T, L, **bf)
        dgrad_cat = torch.empty(T, 2 * Fs + L + E, **bf)
        _cabi.call("lmoe_combine_out_bwd_dgrad", shape, ptr(dyb), ptr(wup), ptr(wds), ptr(h1_s), ptr(d_routed),
                   None, ptr(dgrad_cat), ptr(status), st)
        # adjoint of the combine in send order, then back to the expert ranks
        d_y_send = torch.empty(n_send, L, **bf)
        d_weights = torch.empty(T, K, **f32)
        _cabi.call("lmoe_combine_bwd_rows", ptr(d_routed), ptr(y_back), ptr(weights), ptr(route.perm), n_send, K, L, None,
                   ptr(d_y_send), ptr(d_weights), st)
        d_y_recv = _a2a(d_y_send, n_recv, send_splits, recv_splits, group)

        # local work that overlaps nothing yet but needs no exchange
        d_w_up = torch.empty(D, L, **lin)
        d_w_down_s = torch.empty(D, Fs, **lin)
        _cabi.call("lmoe_combine_out_bwd_wgrad", shape, ptr(dyb), ptr(act_cat), ptr(d_w_up), ptr(d_w_down_s), gtype,
                   ptr(ws), ws.numel(), ptr(status), st)

        # local experts: dgrads and the shard's weight gradients
        d_w_gate_up = torch.zeros(El, L, 2 * F, **bf)
        d_w_down_e = torch.zeros(El, F, L, **bf)
        d_x_recv = torch.empty(n_recv, L, **bf)
        if n_recv > 0:
            d_y_sorted = torch.empty(P, L, **bf)
            _cabi.call("lmoe_gather_rows", ptr(d_y_recv), ptr(row_src), 1, P, L, ptr(n_tiles), ptr(d_y_sorted), st)
            d_h1 = torch.empty(P, 2 * F, **bf)
            d_x_sorted = torch.empty(P, L, **bf)
            d_hidden = d_hidden_scratch(lib, P, L, F, **bf)
            _cabi.call("lmoe_grouped_bwd_dgrad", P, El, L, F, ptr(d_y_sorted), ptr(h1), ptr(wgu), ptr(wde),
                       ptr(tile_expert), ptr(n_tiles), ptr(pad_offsets), ptr(d_hidden), ptr(d_h1), ptr(d_x_sorted), ptr(status), st)
            _cabi.call("lmoe_grouped_bwd_wgrad", P, El, L, F, ptr(x_sorted), ptr(d_h1), ptr(hidden), ptr(d_y_sorted),
                       ptr(pad_offsets), ptr(d_w_gate_up), ptr(d_w_down_e), ptr(status), st)
            _cabi.call("lmoe_gather_rows", ptr(d_x_sorted), ptr(recv_pos), 1, n_recv, L, None, ptr(d_x_recv), st)
        d_x_back = _a2a(d_x_recv, n_send, recv_splits, send_splits, group)
        # adjoint of the gather: d_x_latent[t] = sum_k d_x_back[inv[t*K+k]]  -> dgrad_cat[:, 2Fs:2Fs+L]
        d_x_latent = dgrad_cat[:, 2 * Fs:]
        _cabi.call("lmoe_combine_rows", ptr(d_x_back), ptr(inv), None, T, K, L, ptr(d_x_latent), 2 * Fs + L + E, st)

        dz = None if d_z is None else d_z.to(torch.float32).reshape(1).contiguous()
        _cabi.call("lmoe_gate_topk_bwd", shape, ptr(logits), ptr(sel), ptr(weights), ptr(d_weights), ptr(lse), ptr(dz),
                   ctx.z_coef, ptr(dgrad_cat), st)
        dx = torch.empty(T, D, **bf)
        d_w_gate_up_s = torch.empty(2 * Fs, D, **lin)
        d_w_down = torch.empty(L, D, **lin)
        d_w_gate = torch.empty(E, D, **lin)
        _cabi.call("lmoe_xside_bwd", shape, ptr(dgrad_cat), ptr(wgus), ptr(wdn), ptr(wg), ptr(xb), ptr(dx),
                   ptr(d_w_gate_up_s), ptr(d_w_down), ptr(d_w_gate), gtype, ptr(ws), ws.numel(), ptr(status), st)

        status_monitor.post(status, "expert-parallel LatentMoE backward")

        def as_param(g, d):
            return g if g.dtype == d else g.to(d)

        return (as_param(dx, dt[0]), as_param(d_w_gate, dt[1]), as_param(d_w_down, dt[2]), as_param(d_w_up, dt[3]),
                as_param(d_w_gate_up_s, dt[4]), as_param(d_w_down_s, dt[5]), as_param(d_w_gate_up, dt[6]),
                as_param(d_w_down_e, dt[7]), None, None, None, None)


@torch.compiler.disable   # opaque to torch.compile: the layer runs as an eager call between compiled regions
def latent_moe_ep(x2d, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc, expert_bias, top_k,
                  z_coef, group):
    """Functional form; the expert weights are this rank's shard.  Returns (y, aux_loss, sel, global counts)."""
    return ExpertParallelLatentMoE.apply(x2d, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc,
                                         expert_bias, int(top_k), float(z_coef), group)


# ======================================================================================================
# One-sided exchange over NVLink: rows are stored straight into the destination rank's padded expert
# layout through peer pointers of symmetric buffers (csrc/ep_p2p.cu).  No send buffer, no all-to-all, no
# regroup copy and no host synchronisation: sizes stay on the device, capacities are static.
# ======================================================================================================
class _FlagBarrier:
    """Barrier across the ranks on flag words in symmetric memory (``lmoe_ep_flag_barrier``): one small kernel per rank
    instead of a one-word all-reduce.  ``LMOE_EP_FLAG_BARRIER=0`` keeps the collective.  A rank that waits longer than
    about two seconds records device status 202 in ``status`` (read by the status monitor like any other)."""

    def __init__(self, group, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.G = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.use_flags = os.environ.get("LMOE_EP_FLAG_BARRIER", "1") != "0"
        self.sync_word = torch.zeros(1, dtype=torch.int32, device=device)
        if self.use_flags:
            self.flags = symm_mem.empty(32, dtype=torch.int32, device=device)
            self.flags.zero_()
            self.handle = symm_mem.rendezvous(self.flags, group)
            self.peer_flags = torch.tensor(list(self.handle.buffer_ptrs), dtype=torch.int64, device=device)
            self.status = torch.zeros(1, dtype=torch.int32, device=device)
            self.epoch = torch.zeros(1, dtype=torch.int32, device=device)   # barriers so far; the kernel counts
            torch.cuda.synchronize(device)
            dist.all_reduce(self.sync_word, group=group)     # every rank's flags are zero before anyone's first barrier
            torch.cuda.synchronize(device)

    def __call__(self, status=None):
        if not self.use_flags:
            dist.all_reduce(self.sync_word, group=self.group)
            return
        st = status if status is not None else self.status
        _cabi.call("lmoe_ep_flag_barrier", self.peer_flags.data_ptr(), self.epoch.data_ptr(), self.rank, self.G,
                   st.data_ptr(), _stream())


class SymmetricBuffers:
    """Per-layer symmetric buffers and their peer pointer tables.

    x_in / dy_in  [capacity, L]  rows arriving from all ranks in this rank's padded expert layout (fwd / bwd)
    y_ret / dx_ret [n_send, L]   result rows coming back, in this rank's expert-sorted (send) order
    capacity = roundup(capacity_factor * n_send, 128) + 128 * E/G rows; an expert shard that receives more
    than that raises device status 201 (rows beyond the capacity are dropped).
    """

    def __init__(self, group, n_send: int, L: int, El: int, capacity_factor: float, device):
        import torch.distributed._symmetric_memory as symm_mem
        t = torch.tensor([n_send], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)       # symmetric allocations: same size everywhere
        self.n_send_max = int(t.item())
        self.capacity = (int(capacity_factor * self.n_send_max) + 127) // 128 * 128 + El * 128
        self.L = L
        mk = lambda rows: symm_mem.empty(rows, L, dtype=BF, device=device)
        self.x_in, self.dy_in = mk(self.capacity), mk(self.capacity)
        self.y_ret, self.dx_ret = mk(self.n_send_max), mk(self.n_send_max)
        self.handles = [symm_mem.rendezvous(b, group) for b in (self.x_in, self.dy_in, self.y_ret, self.dx_ret)]
        ptrs = lambda h: torch.tensor(list(h.buffer_ptrs), dtype=torch.int64, device=device)
        self.peer_x_in, self.peer_dy_in, self.peer_y_ret, self.peer_dx_ret = (ptrs(h) for h in self.handles)
        self._barrier = _FlagBarrier(group, device)
        self.side = torch.cuda.Stream(device=device)   # the exchange kernels run here, beside independent GEMMs

    def barrier(self, group, status=None):
        """Stream-ordered barrier across the ranks.  Every kernel queued before it on any rank has completed (its peer
        stores included) before any kernel queued after it starts."""
        self._barrier(status)


class ExpertParallelP2P(torch.autograd.Function):
    """Expert-parallel forward/backward with one-sided NVLink stores (see the banner above)."""

    @staticmethod
    def forward(ctx, x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc, expert_bias,
                top_k: int, z_coef: float, group, bufs: SymmetricBuffers):
        if not x.is_cuda:
            raise _cabi.LmoeError("the LatentMoE path runs on a CUDA device only (no CPU fallback)")
        lib = _cabi.load()
        G, rank = dist.get_world_size(group), dist.get_rank(group)
        dev = x.device
        T, D = x.shape
        El, L, F2 = w_gate_up_loc.shape
        E, F, Fs, K = El * G, F2 // 2, w_down_s.shape[1], top_k
        shape = make_shape(T, D, L, E, K, F, Fs)
        st = _stream()
        bf = dict(dtype=BF, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        n_send, P = T * K, bufs.capacity
        if n_send > bufs.n_send_max:
            raise _cabi.LmoeError("more rows than the symmetric buffers were sized for")

        xb = _as_bf16(x)
        wg, wdn, wup = _as_bf16(w_gate), _as_bf16(w_down), _as_bf16(w_up)
        wgus, wds = _as_bf16(w_gate_up_s), _as_bf16(w_down_s)
        wgu, wde = _as_bf16(w_gate_up_loc), _as_bf16(w_down_e_loc)
        bias = expert_bias.to(torch.float32).contiguous()
        status = torch.zeros(1, **i32)

        logits = torch.empty(T, E, **f32)
        x_latent = torch.empty(T, L, **bf)
        _cabi.call("lmoe_xproj_fwd", shape, ptr(xb), ptr(wg), ptr(wdn), ptr(logits), ptr(x_latent), ptr(status), st)
        sel = torch.empty(T, K, **i32)
        weights = torch.empty(T, K, **f32)
        lse = torch.empty(T, **f32)
        z_partial = torch.empty((T + 7) // 8, **f32)
        z_loss = torch.empty(1, **f32)
        _cabi.call("lmoe_gate_topk_fwd", shape, ptr(logits), ptr(bias), float(z_coef), ptr(sel), ptr(weights), ptr(lse),
                   ptr(z_partial), ptr(z_loss), st)
        route = RouteTables(shape, dev)
        ws = torch.empty(max(16, lib.lmoe_route_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
        _cabi.call("lmoe_route_permute", shape, ptr(sel), route.struct, ptr(ws), ws.numel(), st)
        # the histogram exchange is also the barrier that orders this step's peer stores after every
        # rank's previous use of its buffers
        counts_all = torch.empty(G, E, **i32)
        dist.all_gather_into_tensor(counts_all, route.counts.contiguous(), group=group)

        src_off = torch.empty(G * E, **i32)
        dst_base = torch.empty(E, **i32)
        seg_cum = torch.empty(El * G, **i32)
        pad_offsets = torch.empty(El + 1, **i32)
        tile_expert = torch.empty(P // 128, **i32)
        n_tiles = torch.empty(1, **i32)
        _cabi.call("lmoe_ep_tables", ptr(counts_all), G, E, rank, P, ptr(src_off), ptr(dst_base), ptr(seg_cum),
                   ptr(pad_offsets), ptr(tile_expert), ptr(n_tiles), ptr(status), st)
        # the stores over NVLink run on a side stream, beside the shared-expert GEMM (which needs no exchange)
        main, side = torch.cuda.current_stream(), bufs.side
        ready = torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        sst = side.cuda_stream
        _cabi.call("lmoe_ep_dispatch", ptr(x_latent), ptr(route.perm), ptr(sel), ptr(route.offsets), ptr(dst_base), n_send,
                   K, E, G, L, P, ptr(bufs.peer_x_in), ptr(status), sst)
        _cabi.call("lmoe_ep_zero_pads", ptr(bufs.x_in), L, ptr(pad_offsets), ptr(seg_cum), ptr(counts_all), G, E, rank, sst)
        sent = torch.cuda.Event()
        sent.record(side)
        inv = torch.empty(n_send, **i32)
        _cabi.call("lmoe_invert_perm", ptr(route.perm), n_send, ptr(inv), st)
        h1_s = torch.empty(T, 2 * Fs, **bf)
        act_cat = torch.empty(T, L + Fs, **bf)
        _cabi.call("lmoe_shared_gateup_fwd", shape, ptr(xb), ptr(wgus), ptr(h1_s), ptr(act_cat), ptr(status), st)
        main.wait_event(sent)
        bufs.barrier(group, status)                                   # all rows have landed in x_in

        h1 = torch.empty(P, 2 * F, **bf)
        hidden = torch.empty(P, F, **bf)
        y_sorted = torch.empty(P, L, **bf)
        _cabi.call("lmoe_grouped_fwd", P, El, L, F, ptr(bufs.x_in), ptr(wgu), ptr(wde), ptr(tile_expert), ptr(n_tiles), ptr(pad_offsets),
                   ptr(h1), ptr(hidden), ptr(y_sorted), ptr(status), st)
        _cabi.call("lmoe_ep_return", ptr(y_sorted), ptr(tile_expert), ptr(n_tiles), ptr(pad_offsets), ptr(seg_cum),
                   ptr(src_off), ptr(counts_all), G, E, rank, L, P, ptr(bufs.peer_y_ret), st)
        bufs.barrier(group, status)                                   # all results have landed in y_ret

        y = torch.empty(T, D, **bf)
        back_route = Route(counts=ptr(route.counts), offsets=ptr(route.offsets), perm=ptr(route.perm),
                           pad_offsets=ptr(route.pad_offsets), pos=ptr(inv), row_src=ptr(route.row_src),
                           tile_expert=ptr(route.tile_expert), n_tiles=ptr(route.n_tiles))
        _cabi.call("lmoe_combine_out_fwd", shape, ptr(bufs.y_ret), back_route, ptr(weights), ptr(act_cat), ptr(wds),
                   ptr(wup), ptr(y), ptr(status), st)

        ctx.shape, ctx.route, ctx.group, ctx.z_coef, ctx.status, ctx.bufs = shape, route, group, float(z_coef), status, bufs
        ctx.dims = (G, rank, El, P)
        ctx.dtypes = [t.dtype for t in (x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc)]
        ctx.save_for_backward(xb, wg, wdn, wup, wgus, wds, wgu, wde, logits, sel, weights, lse, inv, act_cat, h1_s, h1,
                              hidden, counts_all, src_off, dst_base, seg_cum, pad_offsets, tile_expert, n_tiles)
        global_counts = counts_all.sum(0, dtype=torch.int32)
        ctx.mark_non_differentiable(sel, global_counts)
        status_monitor.post(status, "expert-parallel LatentMoE forward")
        out = y if x.dtype == BF else y.to(x.dtype)
        return out, z_loss.reshape(()), sel, global_counts

    @staticmethod
    def backward(ctx, dy, d_z, _d_sel, _d_counts):
        (xb, wg, wdn, wup, wgus, wds, wgu, wde, logits, sel, weights, lse, inv, act_cat, h1_s, h1, hidden, counts_all,
         src_off, dst_base, seg_cum, pad_offsets, tile_expert, n_tiles) = ctx.saved_tensors
        shape, route, group, status, bufs = ctx.shape, ctx.route, ctx.group, ctx.status, ctx.bufs
        G, rank, El, P = ctx.dims
        T, D, L, E, K, F, Fs = shape.T, shape.D, shape.L, shape.E, shape.K, shape.F, shape.Fs
        dev = xb.device
        st = _stream()
        lib = _cabi.load()
        bf = dict(dtype=BF, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        if dy is None:
            dy = torch.zeros(T, D, **bf)
        dyb = _as_bf16(dy.reshape(T, D))
        dt = ctx.dtypes
        lin_dtype = torch.float32 if any(d == torch.float32 for d in dt[1:6]) else BF
        gtype = _cabi.F32 if lin_dtype == torch.float32 else _cabi.BF16
        lin = dict(dtype=lin_dtype, device=dev)
        ws = torch.empty(max(16, lib.lmoe_wgrad_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
        n_send = T * K

        d_routed = torch.empty(T, L, **bf)
        dgrad_cat = torch.empty(T, 2 * Fs + L + E, **bf)
        _cabi.call("lmoe_combine_out_bwd_dgrad", shape, ptr(dyb), ptr(wup), ptr(wds), ptr(h1_s), ptr(d_routed),
                   None, ptr(dgrad_cat), ptr(status), st)
        # adjoint of the combine fused into the dispatch: rows w * d_routed go to the expert ranks, the gating
        # gradients <d_routed, y> are formed from the returned rows kept in y_ret
        d_weights = torch.empty(T, K, **f32)
        main, side = torch.cuda.current_stream(), bufs.side
        ready = torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        sst = side.cuda_stream
        _cabi.call("lmoe_ep_dispatch_bwd", ptr(d_routed), ptr(bufs.y_ret), ptr(weights), ptr(route.perm), ptr(sel),
                   ptr(route.offsets), ptr(dst_base), n_send, K, E, G, L, P, ptr(bufs.peer_dy_in), ptr(d_weights),
                   ptr(status), sst)
        _cabi.call("lmoe_ep_zero_pads", ptr(bufs.dy_in), L, ptr(pad_offsets), ptr(seg_cum), ptr(counts_all), G, E, rank, sst)
        sent = torch.cuda.Event()
        sent.record(side)
        # local work that needs no exchange overlaps the peers' stores
        d_w_up = torch.empty(D, L, **lin)
        d_w_down_s = torch.empty(D, Fs, **lin)
        _cabi.call("lmoe_combine_out_bwd_wgrad", shape, ptr(dyb), ptr(act_cat), ptr(d_w_up), ptr(d_w_down_s), gtype,
                   ptr(ws), ws.numel(), ptr(status), st)
        main.wait_event(sent)
        bufs.barrier(group, status)                                   # all gradient rows have landed in dy_in

        d_h1 = torch.empty(P, 2 * F, **bf)
        d_x_sorted = torch.empty(P, L, **bf)
        d_hidden = d_hidden_scratch(lib, P, L, F, **bf)
        _cabi.call("lmoe_grouped_bwd_dgrad", P, El, L, F, ptr(bufs.dy_in), ptr(h1), ptr(wgu), ptr(wde), ptr(tile_expert),
                   ptr(n_tiles), ptr(pad_offsets), ptr(d_hidden), ptr(d_h1), ptr(d_x_sorted), ptr(status), st)
        ready2 = torch.cuda.Event()
        ready2.record(main)
        side.wait_event(ready2)
        _cabi.call("lmoe_ep_return", ptr(d_x_sorted), ptr(tile_expert), ptr(n_tiles), ptr(pad_offsets), ptr(seg_cum),
                   ptr(src_off), ptr(counts_all), G, E, rank, L, P, ptr(bufs.peer_dx_ret), sst)
        returned = torch.cuda.Event()
        returned.record(side)
        # the shard's weight gradients need no exchange: they run beside the return stores
        d_w_gate_up = torch.empty(El, L, 2 * F, **bf)
        d_w_down_e = torch.empty(El, F, L, **bf)
        _cabi.call("lmoe_grouped_bwd_wgrad", P, El, L, F, ptr(bufs.x_in), ptr(d_h1), ptr(hidden), ptr(bufs.dy_in),
                   ptr(pad_offsets), ptr(d_w_gate_up), ptr(d_w_down_e), ptr(status), st)
        main.wait_event(returned)
        bufs.barrier(group, status)                                   # all rows have landed in dx_ret

        d_x_latent = dgrad_cat[:, 2 * Fs:]
        _cabi.call("lmoe_combine_rows", ptr(bufs.dx_ret), ptr(inv), None, T, K, L, ptr(d_x_latent), 2 * Fs + L + E, st)
        dz = None if d_z is None else d_z.to(torch.float32).reshape(1).contiguous()
        _cabi.call("lmoe_gate_topk_bwd", shape, ptr(logits), ptr(sel), ptr(weights), ptr(d_weights), ptr(lse), ptr(dz),
                   ctx.z_coef, ptr(dgrad_cat), st)
        dx = torch.empty(T, D, **bf)
        d_w_gate_up_s = torch.empty(2 * Fs, D, **lin)
        d_w_down = torch.empty(L, D, **lin)
        d_w_gate = torch.empty(E, D, **lin)
        _cabi.call("lmoe_xside_bwd", shape, ptr(dgrad_cat), ptr(wgus), ptr(wdn), ptr(wg), ptr(xb), ptr(dx),
                   ptr(d_w_gate_up_s), ptr(d_w_down), ptr(d_w_gate), gtype, ptr(ws), ws.numel(), ptr(status), st)

        status_monitor.post(status, "expert-parallel LatentMoE backward")

        def as_param(g, d):
            return g if g.dtype == d else g.to(d)

        return (as_param(dx, dt[0]), as_param(d_w_gate, dt[1]), as_param(d_w_down, dt[2]), as_param(d_w_up, dt[3]),
                as_param(d_w_gate_up_s, dt[4]), as_param(d_w_down_s, dt[5]), as_param(d_w_gate_up, dt[6]),
                as_param(d_w_down_e, dt[7]), None, None, None, None, None)


@torch.compiler.disable   # opaque to torch.compile: the layer runs as an eager call between compiled regions
def latent_moe_ep_p2p(x2d, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc, expert_bias, top_k,
                      z_coef, group, bufs: SymmetricBuffers):
    return ExpertParallelP2P.apply(x2d, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc,
                                   expert_bias, int(top_k), float(z_coef), group, bufs)


# ======================================================================================================
# De-duplicated one-sided exchange (csrc/ep_dedup.cu): one row per (token, destination rank) each way.
# ======================================================================================================
class DedupBuffers:
    """Symmetric buffers of the de-duplicated exchange and their peer pointer tables.

    stage_x / stage_dy [G*stride, L]  staging slots: token t of source s lands in slot s*stride + t (fwd / bwd)
    ret_y / ret_dx     [G*stride, L]  one partial-sum row per (owner g, token t) coming back: slot g*stride + t
    meta [capacity] {slot, weight}, mask [G*stride], slots [G*stride*K]   routing words written by the sources
    dw [stride*K]                     gating gradients coming back in backward
    stride = the largest token count of any rank.  The expert layout capacity is as in ``SymmetricBuffers``.
    One forward must be followed by its backward before the next forward reuses the buffers.
    """

    def __init__(self, group, T: int, K: int, L: int, El: int, capacity_factor: float, device):
        import torch.distributed._symmetric_memory as symm_mem
        G = dist.get_world_size(group)
        t = torch.tensor([T], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)       # symmetric allocations: same size everywhere
        self.stride = int(t.item())
        self.K = K
        self.capacity = (int(capacity_factor * self.stride * K) + 127) // 128 * 128 + El * 128
        n = G * self.stride
        rows = lambda: symm_mem.empty(n, L, dtype=BF, device=device)
        self.stage_x, self.stage_dy, self.ret_y, self.ret_dx = rows(), rows(), rows(), rows()
        self.meta = symm_mem.empty(self.capacity, dtype=torch.int64, device=device)
        self.mask = symm_mem.empty(n, dtype=torch.int32, device=device)
        self.slots = symm_mem.empty(n * K, dtype=torch.int32, device=device)
        self.dw = symm_mem.empty(self.stride * K, dtype=torch.float32, device=device)
        bufs = (self.stage_x, self.stage_dy, self.ret_y, self.ret_dx, self.meta, self.mask, self.slots, self.dw)
        self.handles = [symm_mem.rendezvous(b, group) for b in bufs]
        ptrs = lambda h: torch.tensor(list(h.buffer_ptrs), dtype=torch.int64, device=device)
        (self.peer_stage_x, self.peer_stage_dy, self.peer_ret_y, self.peer_ret_dx, self.peer_meta, self.peer_mask,
         self.peer_slots, self.peer_dw) = (ptrs(h) for h in self.handles)
        self._barrier = _FlagBarrier(group, device)
        self.side = torch.cuda.Stream(device=device)

    def barrier(self, group, status=None):
        """Stream-ordered barrier across the ranks (flag words in symmetric memory, ``_FlagBarrier``)."""
        self._barrier(status)


class ExpertParallelDedup(torch.autograd.Function):
    """Expert-parallel forward/backward over the de-duplicated exchange (see the banner above)."""

    @staticmethod
    def forward(ctx, x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc, expert_bias,
                top_k: int, z_coef: float, group, bufs: DedupBuffers):
        if not x.is_cuda:
            raise _cabi.LmoeError("the LatentMoE path runs on a CUDA device only (no CPU fallback)")
        lib = _cabi.load()
        G, rank = dist.get_world_size(group), dist.get_rank(group)
        dev = x.device
        T, D = x.shape
        El, L, F2 = w_gate_up_loc.shape
        E, F, Fs, K = El * G, F2 // 2, w_down_s.shape[1], top_k
        shape = make_shape(T, D, L, E, K, F, Fs)
        st = _stream()
        bf = dict(dtype=BF, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        P, stride = bufs.capacity, bufs.stride
        if T > stride or K != bufs.K:
            raise _cabi.LmoeError("more tokens than the symmetric buffers were sized for")

        xb = _as_bf16(x)
        wg, wdn, wup = _as_bf16(w_gate), _as_bf16(w_down), _as_bf16(w_up)
        wgus, wds = _as_bf16(w_gate_up_s), _as_bf16(w_down_s)
        wgu, wde = _as_bf16(w_gate_up_loc), _as_bf16(w_down_e_loc)
        bias = expert_bias.to(torch.float32).contiguous()
        status = torch.zeros(1, **i32)

        logits = torch.empty(T, E, **f32)
        x_latent = torch.empty(T, L, **bf)
        _cabi.call("lmoe_xproj_fwd", shape, ptr(xb), ptr(wg), ptr(wdn), ptr(logits), ptr(x_latent), ptr(status), st)
        sel = torch.empty(T, K, **i32)
        weights = torch.empty(T, K, **f32)
        lse = torch.empty(T, **f32)
        z_partial = torch.empty((T + 7) // 8, **f32)
        z_loss = torch.empty(1, **f32)
        _cabi.call("lmoe_gate_topk_fwd", shape, ptr(logits), ptr(bias), float(z_coef), ptr(sel), ptr(weights), ptr(lse),
                   ptr(z_partial), ptr(z_loss), st)
        route = RouteTables(shape, dev)
        ws = torch.empty(max(16, lib.lmoe_route_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
        _cabi.call("lmoe_route_permute", shape, ptr(sel), route.struct, ptr(ws), ws.numel(), st)
        # the histogram exchange is also the barrier that orders this step's peer stores after every
        # rank's previous use of its buffers
        counts_all = torch.empty(G, E, **i32)
        dist.all_gather_into_tensor(counts_all, route.counts.contiguous(), group=group)

        src_off = torch.empty(G * E, **i32)
        dst_base = torch.empty(E, **i32)
        seg_cum = torch.empty(El * G, **i32)
        pad_offsets = torch.empty(El + 1, **i32)
        tile_expert = torch.empty(P // 128, **i32)
        n_tiles = torch.empty(1, **i32)
        _cabi.call("lmoe_ep_tables", ptr(counts_all), G, E, rank, P, ptr(src_off), ptr(dst_base), ptr(seg_cum),
                   ptr(pad_offsets), ptr(tile_expert), ptr(n_tiles), ptr(status), st)
        inv = torch.empty(T * K, **i32)
        _cabi.call("lmoe_invert_perm", ptr(route.perm), T * K, ptr(inv), st)
        # the stores over NVLink run on a side stream, beside the shared-expert GEMM (which needs no exchange)
        main, side = torch.cuda.current_stream(), bufs.side
        ready = torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        sst = side.cuda_stream
        # the GEMM is queued first: its CTAs take their place on every SM, and the send kernel's small blocks (four
        # warps, 32 registers per thread) fit into what the GEMM leaves free; the other way round the send's blocks
        # fill the SMs' thread slots and the GEMM waits for them to drain
        h1_s = torch.empty(T, 2 * Fs, **bf)
        act_cat = torch.empty(T, L + Fs, **bf)
        _cabi.call("lmoe_shared_gateup_fwd", shape, ptr(xb), ptr(wgus), ptr(h1_s), ptr(act_cat), ptr(status), st)
        _cabi.call("lmoe_epd_send", ptr(x_latent), ptr(sel), ptr(inv), ptr(route.offsets), ptr(dst_base), ptr(weights), T,
                   K, E, G, rank, L, P, stride, ptr(bufs.peer_stage_x), ptr(bufs.peer_meta), ptr(bufs.peer_mask),
                   ptr(bufs.peer_slots), ptr(status), sst)
        sent = torch.cuda.Event()
        sent.record(side)
        main.wait_event(sent)
        bufs.barrier(group, status)                                   # all rows and routing words have landed

        x_in = torch.empty(P, L, **bf)
        _cabi.call("lmoe_epd_gather", ptr(bufs.stage_x), ptr(bufs.meta), ptr(tile_expert), ptr(n_tiles), ptr(pad_offsets),
                   ptr(seg_cum), ptr(counts_all), G, E, rank, L, P, G * stride, None, ptr(x_in), None, st)
        h1 = torch.empty(P, 2 * F, **bf)
        hidden = torch.empty(P, F, **bf)
        y_sorted = torch.empty(P, L, **bf)
        _cabi.call("lmoe_grouped_fwd", P, El, L, F, ptr(x_in), ptr(wgu), ptr(wde), ptr(tile_expert), ptr(n_tiles), ptr(pad_offsets),
                   ptr(h1), ptr(hidden), ptr(y_sorted), ptr(status), st)
        _cabi.call("lmoe_epd_reduce_return", ptr(y_sorted), ptr(bufs.meta), ptr(bufs.mask), ptr(bufs.slots), None,
                   ptr(src_off), ptr(counts_all), G, E, rank, K, L, stride, P, ptr(bufs.peer_ret_y), None, st)
        bufs.barrier(group, status)                                   # all partial sums have landed in ret_y

        _cabi.call("lmoe_epd_sum", ptr(bufs.ret_y), ptr(sel), T, K, E, G, L, stride, ptr(act_cat), L + Fs, st)
        y = torch.empty(T, D, **bf)
        _cabi.call("lmoe_combine_out_fwd", shape, None, None, None, ptr(act_cat), ptr(wds), ptr(wup), ptr(y),
                   ptr(status), st)

        ctx.shape, ctx.group, ctx.z_coef, ctx.status, ctx.bufs = shape, group, float(z_coef), status, bufs
        ctx.dims = (G, rank, El, P)
        ctx.dtypes = [t.dtype for t in (x, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc)]
        ctx.save_for_backward(xb, wg, wdn, wup, wgus, wds, wgu, wde, logits, sel, weights, lse, act_cat, h1_s, x_in, h1,
                              hidden, y_sorted, counts_all, src_off, seg_cum, pad_offsets, tile_expert, n_tiles)
        global_counts = counts_all.sum(0, dtype=torch.int32)
        ctx.mark_non_differentiable(sel, global_counts)
        status_monitor.post(status, "expert-parallel LatentMoE forward")
        out = y if x.dtype == BF else y.to(x.dtype)
        return out, z_loss.reshape(()), sel, global_counts

    @staticmethod
    def backward(ctx, dy, d_z, _d_sel, _d_counts):
        (xb, wg, wdn, wup, wgus, wds, wgu, wde, logits, sel, weights, lse, act_cat, h1_s, x_in, h1, hidden, y_sorted,
         counts_all, src_off, seg_cum, pad_offsets, tile_expert, n_tiles) = ctx.saved_tensors
        shape, group, status, bufs = ctx.shape, ctx.group, ctx.status, ctx.bufs
        G, rank, El, P = ctx.dims
        T, D, L, E, K, F, Fs = shape.T, shape.D, shape.L, shape.E, shape.K, shape.F, shape.Fs
        dev = xb.device
        st = _stream()
        lib = _cabi.load()
        bf = dict(dtype=BF, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        stride = bufs.stride
        if dy is None:
            dy = torch.zeros(T, D, **bf)
        dyb = _as_bf16(dy.reshape(T, D))
        dt = ctx.dtypes
        lin_dtype = torch.float32 if any(d == torch.float32 for d in dt[1:6]) else BF
        gtype = _cabi.F32 if lin_dtype == torch.float32 else _cabi.BF16
        lin = dict(dtype=lin_dtype, device=dev)
        ws = torch.empty(max(16, lib.lmoe_wgrad_workspace_bytes(shape)), dtype=torch.uint8, device=dev)

        d_routed = torch.empty(T, L, **bf)
        dgrad_cat = torch.empty(T, 2 * Fs + L + E, **bf)
        _cabi.call("lmoe_combine_out_bwd_dgrad", shape, ptr(dyb), ptr(wup), ptr(wds), ptr(h1_s), ptr(d_routed),
                   None, ptr(dgrad_cat), ptr(status), st)
        main, side = torch.cuda.current_stream(), bufs.side
        ready = torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        sst = side.cuda_stream
        _cabi.call("lmoe_epd_send", ptr(d_routed), ptr(sel), None, None, None, None, T, K, E, G, rank, L, P, stride,
                   ptr(bufs.peer_stage_dy), None, None, None, ptr(status), sst)
        sent = torch.cuda.Event()
        sent.record(side)
        # local work that needs no exchange overlaps the peers' stores
        d_w_up = torch.empty(D, L, **lin)
        d_w_down_s = torch.empty(D, Fs, **lin)
        _cabi.call("lmoe_combine_out_bwd_wgrad", shape, ptr(dyb), ptr(act_cat), ptr(d_w_up), ptr(d_w_down_s), gtype,
                   ptr(ws), ws.numel(), ptr(status), st)
        main.wait_event(sent)
        bufs.barrier(group, status)                                   # all gradient rows have landed in stage_dy

        # adjoint of the weighted combine on the owner: d_y rows and the gating gradients of its rows
        dy_in = torch.empty(P, L, **bf)
        d_w_row = torch.empty(P, **f32)
        _cabi.call("lmoe_epd_gather", ptr(bufs.stage_dy), ptr(bufs.meta), ptr(tile_expert), ptr(n_tiles),
                   ptr(pad_offsets), ptr(seg_cum), ptr(counts_all), G, E, rank, L, P, G * stride, ptr(y_sorted), ptr(dy_in),
                   ptr(d_w_row), st)
        d_h1 = torch.empty(P, 2 * F, **bf)
        d_x_sorted = torch.empty(P, L, **bf)
        d_hidden = d_hidden_scratch(lib, P, L, F, **bf)
        _cabi.call("lmoe_grouped_bwd_dgrad", P, El, L, F, ptr(dy_in), ptr(h1), ptr(wgu), ptr(wde), ptr(tile_expert),
                   ptr(n_tiles), ptr(pad_offsets), ptr(d_hidden), ptr(d_h1), ptr(d_x_sorted), ptr(status), st)
        ready2 = torch.cuda.Event()
        ready2.record(main)
        side.wait_event(ready2)
        _cabi.call("lmoe_epd_reduce_return", ptr(d_x_sorted), ptr(bufs.meta), ptr(bufs.mask), ptr(bufs.slots),
                   ptr(d_w_row), ptr(src_off), ptr(counts_all), G, E, rank, K, L, stride, P, ptr(bufs.peer_ret_dx),
                   ptr(bufs.peer_dw), sst)
        returned = torch.cuda.Event()
        returned.record(side)
        # the shard's weight gradients need no exchange: they run beside the return stores
        d_w_gate_up = torch.empty(El, L, 2 * F, **bf)
        d_w_down_e = torch.empty(El, F, L, **bf)
        _cabi.call("lmoe_grouped_bwd_wgrad", P, El, L, F, ptr(x_in), ptr(d_h1), ptr(hidden), ptr(dy_in),
                   ptr(pad_offsets), ptr(d_w_gate_up), ptr(d_w_down_e), ptr(status), st)
        main.wait_event(returned)
        bufs.barrier(group, status)                                   # partial sums in ret_dx, gating gradients in dw

        d_x_latent = dgrad_cat[:, 2 * Fs:]
        _cabi.call("lmoe_epd_sum", ptr(bufs.ret_dx), ptr(sel), T, K, E, G, L, stride, ptr(d_x_latent), 2 * Fs + L + E, st)
        dz = None if d_z is None else d_z.to(torch.float32).reshape(1).contiguous()
        _cabi.call("lmoe_gate_topk_bwd", shape, ptr(logits), ptr(sel), ptr(weights), ptr(bufs.dw), ptr(lse), ptr(dz),
                   ctx.z_coef, ptr(dgrad_cat), st)
        dx = torch.empty(T, D, **bf)
        d_w_gate_up_s = torch.empty(2 * Fs, D, **lin)
        d_w_down = torch.empty(L, D, **lin)
        d_w_gate = torch.empty(E, D, **lin)
        _cabi.call("lmoe_xside_bwd", shape, ptr(dgrad_cat), ptr(wgus), ptr(wdn), ptr(wg), ptr(xb), ptr(dx),
                   ptr(d_w_gate_up_s), ptr(d_w_down), ptr(d_w_gate), gtype, ptr(ws), ws.numel(), ptr(status), st)

        status_monitor.post(status, "expert-parallel LatentMoE backward")

        def as_param(g, d):
            return g if g.dtype == d else g.to(d)

        return (as_param(dx, dt[0]), as_param(d_w_gate, dt[1]), as_param(d_w_down, dt[2]), as_param(d_w_up, dt[3]),
                as_param(d_w_gate_up_s, dt[4]), as_param(d_w_down_s, dt[5]), as_param(d_w_gate_up, dt[6]),
                as_param(d_w_down_e, dt[7]), None, None, None, None, None)


@torch.compiler.disable   # opaque to torch.compile: the layer runs as an eager call between compiled regions
def latent_moe_ep_dedup(x2d, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc, expert_bias,
                        top_k, z_coef, group, bufs: DedupBuffers):
    return ExpertParallelDedup.apply(x2d, w_gate, w_down, w_up, w_gate_up_s, w_down_s, w_gate_up_loc, w_down_e_loc,
                                     expert_bias, int(top_k), float(z_coef), group, bufs)
