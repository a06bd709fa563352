"""Device timeline of ONE eager fwd+bwd step of the layer: start offset, duration and gap to the previous kernel for every
kernel, from the CUDA activity records of ``torch.profiler`` (not an ncu capture: a multi-rank command is never wrapped
in ncu).

    python -m swamla_b200.steptimeline [--workload cfg2] [--min-us 5]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m swamla_b200.steptimeline --workload cfg5 [--ep-mode p2p_dedup] [--ranks 0,5]

Under ``torch.distributed.run`` the routed experts are sharded over the N ranks (rank r keeps experts
[r*E/N, (r+1)*E/N) and runs its own tokens) and the ranks named by ``--ranks`` print their timelines.  A diagnostic, not a
benchmark: profiler records carry a few microseconds of overhead per kernel.
"""
from __future__ import annotations

import argparse
import os

import torch

from . import workloads
from .layer import LatentMoELayer


def _build(w, rank, dev, group, ep_mode):
    params, buffers, x, dy = workloads.make_inputs(w, seed=0)
    if rank > 0:
        g = torch.Generator("cpu").manual_seed(1000 + rank)
        x, dy = torch.randn(x.shape, generator=g), torch.randn(x.shape, generator=g)
    cfg = w.config()
    if w.dtype == "fp8":
        cfg.moe_fp8 = True
    state = {**params, **buffers}
    if group is not None:
        import torch.distributed as dist
        cfg.ep_group, cfg.ep_mode = group, ep_mode
        el = w.E // dist.get_world_size(group)
        for k in ("experts.gate_up_weight", "experts.down_weight"):
            state[k] = state[k][rank * el:(rank + 1) * el].clone()
    layer = LatentMoELayer(cfg)
    layer.load_state_dict(state, strict=True)
    layer = layer.to(dev).to(torch.bfloat16).train()
    return layer, x.to(torch.bfloat16).to(dev).requires_grad_(True), dy.to(torch.bfloat16).to(dev)


def _step(layer, x, dy):
    for p in layer.parameters():
        p.grad = None
    x.grad = None
    y = layer(x)
    torch.autograd.backward([y, layer.get_aux_loss()], [dy, torch.ones_like(layer.get_aux_loss())])
    if hasattr(layer, "router"):
        layer.router.update_bias_from_last_forward()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--ep-mode", default="p2p_dedup")
    ap.add_argument("--ranks", default="0", help="comma-separated ranks that print")
    ap.add_argument("--min-us", type=float, default=0.0, help="leave out kernels shorter than this")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    w = workloads.WORKLOADS[args.workload]
    layer, x, dy = _build(w, rank, dev, group, args.ep_mode)

    from torch.profiler import ProfilerActivity, profile
    for _ in range(4):
        _step(layer, x, dy)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            _step(layer, x, dy)
        torch.cuda.synchronize()
    if rank in {int(r) for r in args.ranks.split(",")}:
        evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
        evs.sort(key=lambda e: e.time_range.start)
        last = evs[len(evs) // 2:]                       # the second of the two profiled steps
        t0 = prev = last[0].time_range.start
        for e in last:
            d = e.time_range.end - e.time_range.start
            if d >= args.min_us:
                print(f"r{rank} {e.time_range.start - t0:9.1f} us +{d:7.1f}  gap {e.time_range.start - prev:7.1f}  {e.name[:90]}")
            prev = max(prev, e.time_range.end)
        print(f"r{rank} step span {max(e.time_range.end for e in last) - t0:.1f} us, {len(last)} kernels", flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
