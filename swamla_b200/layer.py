"""Drop-in ``LatentMoELayer`` (and the non-latent ``MoELayer``) for Orolol/swamla (``models/moe.py:603-866``, ``294-559``).

Same constructor (one ``config`` object read with ``getattr``), same ``forward(x)`` signature,
attributes, buffers and ``state_dict`` keys as the reference module, so it replaces it behind
``create_moe_layer`` without touching ``swa_mla_model.py``.  The computation runs in bf16 on the
hand-written sm_100a kernels of ``liblmoe.so``; there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _cabi, status as status_monitor
from .functional import latent_moe, make_shape, _stream
from .compiled_ops import latent_moe_compiled


def _ep_size(group) -> int:
    if group is None:
        return 1
    import torch.distributed as dist
    return dist.get_world_size(group)


class SwiGLUExpert(nn.Module):
    """Parameter container of the shared expert (``models/moe.py:32-69``): ``gate_up_proj`` [2*d_ff, d_model]
    (gate = first half) and ``down_proj`` [d_model, d_ff].  The math runs inside the fused layer kernels."""

    def __init__(self, d_model: int, d_ff: int, bias: bool = False):
        super().__init__()
        if bias:
            raise NotImplementedError("config.bias=True is not supported on this path (no preset uses it)")
        self.gate_up_proj = nn.Linear(d_model, 2 * d_ff, bias=False)
        self.down_proj = nn.Linear(d_ff, d_model, bias=False)
        nn.init.normal_(self.gate_up_proj.weight, mean=0.0, std=0.02)   # moe.py:48-49
        nn.init.normal_(self.down_proj.weight, mean=0.0, std=0.02)


class LatentBatchedExperts(nn.Module):
    """Routed expert weights in the reference layout (``models/moe.py:562-600``):
    ``gate_up_weight`` [E, latent, 2*d_ff] and ``down_weight`` [E, d_ff, latent].

    Under expert parallelism (``ep_group`` of G ranks) the parameters hold this rank's contiguous block of
    ``n_experts`` = E_global / G experts.  ``state_dict()`` issues NO collective: it returns this rank's block, so
    the reference's rank-0-only save (``train.py:1471,1486``) cannot hang the other ranks; the checkpoint in the
    reference's layout (full [E_global, ...] tensors) comes from ``ep.gather_full_state_dict(model)``, which every
    rank of the group calls.  Loading accepts the full tensors (each rank takes its block) or block-shaped ones, so
    a checkpoint written by the reference (``train.py:1470-1506``) loads into any group size and the other way
    round."""

    def __init__(self, n_experts: int, latent_dim: int, d_ff: int, bias: bool = False, ep_group=None):
        super().__init__()
        if bias:
            raise NotImplementedError("config.bias=True is not supported on this path (no preset uses it)")
        self.n_experts, self.latent_dim, self.d_ff = n_experts, latent_dim, d_ff
        self.ep_group = ep_group
        self.ep_size = _ep_size(ep_group)
        self.gate_up_weight = nn.Parameter(torch.empty(n_experts, latent_dim, 2 * d_ff))
        self.down_weight = nn.Parameter(torch.empty(n_experts, d_ff, latent_dim))
        self.register_parameter("gate_up_bias", None)
        self.register_parameter("down_bias", None)
        nn.init.normal_(self.gate_up_weight, mean=0.0, std=0.02)         # moe.py:599-600
        nn.init.normal_(self.down_weight, mean=0.0, std=0.02)
        if self.ep_size > 1:
            # the owner's gradient is already the sum over the tokens of ALL ranks: a data-parallel wrapper must
            # not reduce these parameters again (see ep.ddp_ignore_expert_shards)
            self.gate_up_weight.expert_shard = True
            self.down_weight.expert_shard = True

    def _ep_rank(self) -> int:
        import torch.distributed as dist
        return dist.get_rank(self.ep_group)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        if self.ep_size > 1:
            lo = self._ep_rank() * self.n_experts
            for name in ("gate_up_weight", "down_weight"):
                t = state_dict.get(prefix + name)
                if t is not None and t.shape[0] == self.ep_size * self.n_experts:
                    state_dict[prefix + name] = t[lo:lo + self.n_experts]     # a view; the caller's dict is a copy
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)


class AuxLossFreeRouter(nn.Module):
    """Router state (``models/moe.py:156-291``): the gate weight, the selection bias and the load
    statistics.  Top-k runs inside the layer kernels; the bias update reuses the routing histogram."""

    def __init__(self, d_model: int, n_experts: int, top_k: int, bias_update_gamma: float = 0.001,
                 z_loss_coef: float = 0.001):
        super().__init__()
        self.n_experts, self.top_k = n_experts, top_k
        self.gamma, self.z_loss_coef = bias_update_gamma, z_loss_coef
        self.gate = nn.Linear(d_model, n_experts, bias=False)
        self.register_buffer("expert_bias", torch.zeros(n_experts))
        self.register_buffer("load_history", torch.zeros(n_experts))
        self.register_buffer("update_count", torch.tensor(0))
        nn.init.normal_(self.gate.weight, mean=0.0, std=0.01)            # moe.py:194
        self._last_selected_experts = None   # int32 [T, K] of the last training forward
        self._last_counts = None             # int32 [E] routing histogram of the same forward
        self._last_num_tokens = None

    def update_bias_from_last_forward(self):
        """``models/moe.py:244-275``: bias -= gamma * sign(load - T*K/E), after backward."""
        if self._last_counts is None:
            return
        status_monitor.poll()            # a step whose kernels reported a failure raises here (or at the next forward)
        counts, T = self._last_counts, self._last_num_tokens
        # the kernel takes the expected load T*K/E from the histogram itself (sum of counts / E), so a histogram
        # summed over expert-parallel ranks with different token counts gives the same update on every rank
        shape = make_shape(T, 8, 64, self.n_experts, self.top_k, 64, 8)
        if self.expert_bias.dtype != torch.float32 or self.load_history.dtype != torch.float32:
            # inference-style casts of the buffers: update in fp32, store back
            bias, hist = self.expert_bias.float(), self.load_history.float()
            _cabi.call("lmoe_router_bias_update", shape, counts.data_ptr(), float(self.gamma), bias.data_ptr(),
                       hist.data_ptr(), _stream())
            self.expert_bias.copy_(bias)
            self.load_history.copy_(hist)
        else:
            _cabi.call("lmoe_router_bias_update", shape, counts.data_ptr(), float(self.gamma),
                       self.expert_bias.data_ptr(), self.load_history.data_ptr(), _stream())
        self.update_count += 1
        self._last_selected_experts = None
        self._last_counts = None
        self._last_num_tokens = None

    def get_load_balance_stats(self) -> dict:
        """``models/moe.py:277-291``."""
        if self.update_count == 0:
            return {"load_mean": 0, "load_std": 0, "load_ratio": 1}
        load = self.load_history.float() / (self.update_count.float() + 1e-9)
        load_normalized = load / (load.sum() + 1e-9)
        return {
            "load_mean": load_normalized.mean().item(),
            "load_std": load_normalized.std().item(),
            "load_min": load_normalized.min().item(),
            "load_max": load_normalized.max().item(),
            "load_ratio": (load_normalized.max() / (load_normalized.min() + 1e-9)).item(),
        }


def _merged_shared_weights(shared_experts):
    """The shared experts as ONE SwiGLU expert of width ``n * expert_dim`` (``models/moe.py:713-715`` sums their outputs:
    ``sum_i down_i(silu(gate_i x) * up_i x)`` is a single expert whose gate/up rows and whose down columns are the
    experts' stacked).  Returns ``(gate_up [2nFs, D] = [gate_0 .. gate_n-1 | up_0 .. up_n-1], down [D, nFs])``; with
    one expert its own parameters, otherwise concatenations that autograd splits back onto the experts' parameters."""
    if len(shared_experts) == 1:
        return shared_experts[0].gate_up_proj.weight, shared_experts[0].down_proj.weight
    gu = [e.gate_up_proj.weight for e in shared_experts]
    fs = gu[0].shape[0] // 2
    gate_up = torch.cat([w[:fs] for w in gu] + [w[fs:] for w in gu], dim=0)
    down = torch.cat([e.down_proj.weight for e in shared_experts], dim=1)
    return gate_up, down


class LatentMoELayer(nn.Module):
    """LatentMoE feed-forward layer; see the module docstring.  ``models/moe.py:603-866``."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        d_model = config.n_embd
        latent_ratio = getattr(config, "latent_ratio", 4)
        latent_dim = getattr(config, "latent_dim", None)
        if latent_dim is None:
            latent_dim = d_model // latent_ratio
        base_n_experts = getattr(config, "n_experts", 32)
        base_n_activated = getattr(config, "n_activated", 3)
        latent_n_experts = getattr(config, "latent_n_experts", None)
        latent_n_activated = getattr(config, "latent_n_activated", None)
        # base values are scaled by latent_ratio unless explicit latent counts are given (moe.py:639-646)
        n_experts = latent_n_experts if latent_n_experts is not None else base_n_experts * latent_ratio
        n_activated = latent_n_activated if latent_n_activated is not None else base_n_activated * latent_ratio
        n_shared = getattr(config, "n_shared_experts", 1)
        expert_dim = getattr(config, "expert_dim", d_model)
        bias = getattr(config, "bias", False)
        z_loss_coef = getattr(config, "router_z_loss_coef", 0.001)
        if bias:
            raise NotImplementedError("config.bias=True is not supported on this path (no preset uses it)")
        if n_shared < 1:
            raise NotImplementedError("at least one shared expert is required (every preset uses 1)")

        self.n_experts = n_experts
        self.n_shared = n_shared
        self.n_activated = n_activated
        self.d_model = d_model
        self.latent_dim = latent_dim
        self.expert_dim = expert_dim
        self.latent_ratio = d_model // latent_dim

        self.down_proj = nn.Linear(d_model, latent_dim, bias=False)
        self.up_proj = nn.Linear(latent_dim, d_model, bias=False)
        nn.init.normal_(self.down_proj.weight, mean=0.0, std=0.02)        # moe.py:666-667
        nn.init.normal_(self.up_proj.weight, mean=0.0, std=0.02)
        self.shared_experts = nn.ModuleList([SwiGLUExpert(d_model, expert_dim, bias=False) for _ in range(n_shared)])
        preserve = getattr(config, "latent_preserve_expert_dim", False)
        latent_expert_dim = expert_dim if preserve else expert_dim // latent_ratio   # moe.py:680-685
        self.latent_expert_dim = latent_expert_dim
        # Optional expert parallelism: `config.ep_group` (a torch.distributed process group) shards the
        # routed experts; this rank then holds experts [rank*E/G, (rank+1)*E/G) only.  Absent -> all experts.
        self.ep_group = getattr(config, "ep_group", None)
        self.ep_size = _ep_size(self.ep_group)
        # "p2p_dedup": one-sided stores over NVLink, one row per (token, destination rank), partial sums on the owner;
        # "p2p": one row per (token, expert), bit-identical to the single-GPU layer; "nccl": all-to-all through NCCL
        self.ep_mode = getattr(config, "ep_mode", "p2p_dedup")
        if self.ep_mode not in ("p2p_dedup", "p2p", "nccl"):
            raise ValueError("ep_mode must be 'p2p_dedup', 'p2p' or 'nccl'")
        # incoming-buffer capacity of a shard, as a multiple of this rank's own row count T*K (p2p mode)
        self.ep_capacity_factor = float(getattr(config, "ep_capacity_factor", 2.0))
        # The exchange buffers are symmetric allocations sized for the largest token count of any rank; they are
        # (re)allocated collectively, so every rank must outgrow them in the same forward.  `config.ep_max_tokens`
        # sizes them once for the largest batch a rank will ever see (default: the first forward's maximum).
        self.ep_max_tokens = int(getattr(config, "ep_max_tokens", 0) or 0)
        self._ep_bufs = None
        if n_experts % self.ep_size:
            raise ValueError("the expert count must be divisible by the expert-parallel group size")
        self.experts = LatentBatchedExperts(n_experts // self.ep_size, latent_dim, latent_expert_dim, bias=False,
                                            ep_group=self.ep_group)
        self.router = AuxLossFreeRouter(d_model=d_model, n_experts=n_experts, top_k=n_activated, z_loss_coef=z_loss_coef)
        # `config.moe_fp8 = True`: routed expert GEMMs in e4m3 with per-tensor dynamic scaling
        self.fp8_experts = bool(getattr(config, "moe_fp8", False))
        if self.fp8_experts and (latent_dim % 128 or latent_expert_dim % 128):
            raise ValueError("moe_fp8 needs latent_dim and the routed expert dim to be multiples of 128")
        self.dropout = nn.Dropout(getattr(config, "dropout", 0.0))
        self.aux_loss = torch.tensor(0.0)

        if latent_dim % 64 or latent_expert_dim % 64 or d_model % 8 or expert_dim % 8 or n_experts % 8:
            raise ValueError("kernel constraints: latent_dim and routed expert dim multiples of 64; "
                             "n_embd, expert_dim and the expert count multiples of 8")
        if n_experts > 256 or n_activated > 32:
            raise ValueError("kernel constraints: at most 256 routed experts and top-32")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        compiling = torch.compiler.is_compiling()
        if not compiling:
            status_monitor.poll()        # raises if an earlier step's kernels reported a failure (no synchronisation)
        batch_size, seq_len, d_model = x.shape
        x_flat = x.reshape(-1, d_model)
        w_gate_up_s, w_down_s = _merged_shared_weights(self.shared_experts)
        args = (x_flat, self.router.gate.weight, self.down_proj.weight, self.up_proj.weight,
                w_gate_up_s, w_down_s,
                self.experts.gate_up_weight, self.experts.down_weight,
                self.router.expert_bias, self.n_activated, self.router.z_loss_coef)
        if self.ep_size > 1 and self.ep_mode == "p2p_dedup":
            from .ep import DedupBuffers, latent_moe_ep_dedup
            T = x_flat.shape[0]
            if self._ep_bufs is None or self._ep_bufs.stride < T:
                self._ep_bufs = DedupBuffers(self.ep_group, max(T, self.ep_max_tokens), self.n_activated, self.latent_dim,
                                             self.experts.n_experts, self.ep_capacity_factor, x.device)
            y, z_loss, sel, counts = latent_moe_ep_dedup(*args, self.ep_group, self._ep_bufs)
        elif self.ep_size > 1 and self.ep_mode == "p2p":
            # one-sided NVLink stores into the peers' padded expert layout (symmetric buffers owned by the layer;
            # one forward must be followed by its backward before the next forward reuses them)
            from .ep import SymmetricBuffers, latent_moe_ep_p2p
            n_send = x_flat.shape[0] * self.n_activated
            if self._ep_bufs is None or self._ep_bufs.n_send_max < n_send:
                self._ep_bufs = SymmetricBuffers(self.ep_group, max(n_send, self.ep_max_tokens * self.n_activated),
                                                 self.latent_dim, self.experts.n_experts, self.ep_capacity_factor, x.device)
            y, z_loss, sel, counts = latent_moe_ep_p2p(*args, self.ep_group, self._ep_bufs)
        elif self.ep_size > 1:
            from .ep import latent_moe_ep
            y, z_loss, sel, counts = latent_moe_ep(*args, self.ep_group)   # counts: load summed over all ranks
        elif compiling and not self.fp8_experts:
            # torch.compile (the reference's default, train.py:936-942): custom operators with fake implementations
            # keep one graph across the layer; they run the same kernels as the eager call below
            y, z_loss, sel, counts = latent_moe_compiled(*args)
        else:
            y, z_loss, sel, counts = latent_moe(*args, fp8=self.fp8_experts)
        self.aux_loss = z_loss                                            # moe.py:719
        if self.training:                                                 # moe.py:237-240
            self.router._last_selected_experts = sel
            self.router._last_counts = counts
            self.router._last_num_tokens = x_flat.shape[0]
        y = self.dropout(y)                                               # moe.py:732
        return y.view(batch_size, seq_len, d_model)

    def check_status(self) -> None:
        """Waits for the steps queued so far and raises ``LmoeError`` if one of them reported a device failure
        (a bounded wait that expired, or an expert-parallel shard that received more rows than its buffers hold)."""
        status_monitor.poll(block=True)

    def get_aux_loss(self) -> torch.Tensor:
        return self.aux_loss

    def get_load_balance_stats(self) -> dict:
        return self.router.get_load_balance_stats()


class BatchedExperts(nn.Module):
    """Routed expert weights of the non-latent layer in the reference layout (``models/moe.py:72-109``):
    ``gate_up_weight`` [E, d_model, 2*d_ff] and ``down_weight`` [E, d_ff, d_model]."""

    def __init__(self, n_experts: int, d_model: int, d_ff: int, bias: bool = False):
        super().__init__()
        if bias:
            raise NotImplementedError("config.bias=True is not supported on this path (no preset uses it)")
        self.n_experts, self.d_model, self.d_ff = n_experts, d_model, d_ff
        self.gate_up_weight = nn.Parameter(torch.empty(n_experts, d_model, 2 * d_ff))
        self.down_weight = nn.Parameter(torch.empty(n_experts, d_ff, d_model))
        self.register_parameter("gate_up_bias", None)
        self.register_parameter("down_bias", None)
        nn.init.normal_(self.gate_up_weight, mean=0.0, std=0.02)         # moe.py:106-109
        nn.init.normal_(self.down_weight, mean=0.0, std=0.02)


class MoELayer(nn.Module):
    """The non-latent mixture-of-experts layer (``models/moe.py:294-559``): same constructor, ``forward(x)``, attributes
    and ``state_dict`` keys as the reference class; the experts work at the model width on the kernels of
    ``liblmoe.so`` (``functional_moe.py``).  Single GPU, bf16."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        d_model = config.n_embd
        n_experts = getattr(config, "n_experts", 32)
        n_shared = getattr(config, "n_shared_experts", 1)
        n_activated = getattr(config, "n_activated", 3)
        expert_dim = getattr(config, "expert_dim", d_model)
        bias = getattr(config, "bias", False)
        z_loss_coef = getattr(config, "router_z_loss_coef", 0.001)
        if bias:
            raise NotImplementedError("config.bias=True is not supported on this path (no preset uses it)")
        if n_shared < 1:
            raise NotImplementedError("at least one shared expert is required (every preset uses 1)")
        if getattr(config, "ep_group", None) is not None or getattr(config, "moe_fp8", False):
            raise NotImplementedError("expert parallelism and FP8 are provided for the latent layer only")
        self.n_experts, self.n_shared, self.n_activated = n_experts, n_shared, n_activated
        self.d_model, self.expert_dim = d_model, expert_dim
        self.shared_experts = nn.ModuleList([SwiGLUExpert(d_model, expert_dim, bias=False) for _ in range(n_shared)])
        self.experts = BatchedExperts(n_experts, d_model, expert_dim, bias=False)
        self.router = AuxLossFreeRouter(d_model=d_model, n_experts=n_experts, top_k=n_activated, z_loss_coef=z_loss_coef)
        self.dropout = nn.Dropout(getattr(config, "dropout", 0.0))
        self.aux_loss = torch.tensor(0.0)
        if d_model % 64 or expert_dim % 64 or n_experts % 8:
            raise ValueError("kernel constraints: n_embd and expert_dim multiples of 64, expert count a multiple of 8")
        if n_experts > 256 or n_activated > 32:
            raise ValueError("kernel constraints: at most 256 routed experts and top-32")

    def check_status(self) -> None:
        """Waits for the steps queued so far and raises ``LmoeError`` if one of them reported a device failure."""
        status_monitor.poll(block=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .functional_moe import moe
        status_monitor.poll()
        batch_size, seq_len, d_model = x.shape
        x_flat = x.reshape(-1, d_model)
        w_gate_up_s, w_down_s = _merged_shared_weights(self.shared_experts)
        y, z_loss, sel, counts = moe(x_flat, self.router.gate.weight, w_gate_up_s,
                                     w_down_s, self.experts.gate_up_weight, self.experts.down_weight,
                                     self.router.expert_bias, self.n_activated, self.router.z_loss_coef)
        self.aux_loss = z_loss                                            # moe.py:358
        if self.training:                                                 # moe.py:237-240
            self.router._last_selected_experts = sel
            self.router._last_counts = counts
            self.router._last_num_tokens = x_flat.shape[0]
        y = self.dropout(y)                                               # moe.py:367
        return y.view(batch_size, seq_len, d_model)

    def get_aux_loss(self) -> torch.Tensor:
        return self.aux_loss

    def get_load_balance_stats(self) -> dict:
        return self.router.get_load_balance_stats()


def create_moe_layer(config, use_latent: bool = False):
    """``models/moe.py:869-882``: the latent layer when asked for, else the non-latent one."""
    if use_latent or getattr(config, "use_latent_moe", False):
        return LatentMoELayer(config)
    return MoELayer(config)
