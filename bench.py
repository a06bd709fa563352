#!/usr/bin/env python
"""Benchmark of the LatentMoE feed-forward path: forward+backward tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfgX]

One step = one forward+backward of the layer over one batch of synthetic tokens.  Rank 0 prints ONE
JSON line.  ``value`` is timed with CUDA events with inputs resident in HBM; ``e2e`` is the same step
driven through the nn.Module with pinned HOST buffers (H2D of x and dy, D2H of y and the aux loss
inside the timed region, copies pipelined on side streams).  ``--impl reference`` times the CPU oracle
(the reference layer's algorithm in fp32 torch) on the host cores on a bounded sample of the workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from swamla_b200 import workloads as inputs  # noqa: E402

METRIC = "LatentMoE fwd+bwd tokens/s"
# dram__bytes_read.sum + dram__bytes_write.sum of ALL tcgen05 GEMM launches of one step (ncu, one three-counter capture
# of an eager step at the workload's full size); a workload without a capture of the current kernels reports null
TRAFFIC_BYTES_PER_STEP = {"cfg2": 2592600832}
SUSTAINED_SECONDS = 2.0
CPU_SAMPLE_TOKENS = 1024


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d.get("bf16_tflops_sustained"),
                    hbm_gbs=d["hbm_gbs"], source="measured")
    return dict(bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons, power = [], None, set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                power.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        power.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "samples": len(sm),
                "power_w": power[len(power) // 2] if power else None, "reasons": sorted(reasons)}


def tokens_of_rank(w, rank, x0=None, dy0=None):
    """(x, dy) of one rank, fp32 on the host: rank 0 uses the workload's canonical tokens, rank r > 0 its own seed."""
    if rank == 0:
        if x0 is None:
            _, _, x0, dy0 = inputs.make_inputs(w, seed=0)
        return x0, dy0
    g = torch.Generator("cpu").manual_seed(1000 + rank)
    shape = (w.batch, w.seq, w.D)
    return torch.randn(shape, generator=g), torch.randn(shape, generator=g)


def ep_parity(w, ep_layer, single, rank, world, dev, dist):
    """One fwd+bwd of the expert-parallel layer (every rank on its own tokens) against the single-GPU layer holding
    ALL experts, run by rank 0 over the tokens of all ranks.  Compared on rank 0: its y and dx rows, the routing of
    its tokens, the global load histogram, the gradient of its expert shard (a sum over the tokens of all ranks)
    and the replicated parameters' gradients summed over the ranks.  Returns the report dict on rank 0, None
    elsewhere."""
    from swamla_b200 import _cabi
    x_host, dy_host = tokens_of_rank(w, rank)
    xg = x_host.to(torch.bfloat16).to(dev).requires_grad_(True)
    zero_grads(ep_layer, xg)
    y = ep_layer(xg)
    y.backward(dy_host.to(torch.bfloat16).to(dev))
    status = 0
    try:
        ep_layer.check_status()
    except _cabi.LmoeError as e:                        # keep going: the report carries the code
        status = int(str(e).split("device status ")[1].split()[0])
    replicated = {}
    for name, p in ep_layer.named_parameters():
        if not getattr(p, "expert_shard", False):
            g = p.grad.float()
            dist.all_reduce(g)
            replicated[name] = g
    st = torch.tensor([status], device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    if rank != 0:
        return None
    from oracle.latent_moe_ref import closeness      # the checker's error report only; nothing of the oracle is timed
    xs, dys = zip(*[tokens_of_rank(w, r) for r in range(world)])
    xa = torch.cat([t.reshape(-1, w.D) for t in xs]).to(torch.bfloat16).to(dev).reshape(1, -1, w.D).requires_grad_(True)
    dya = torch.cat([t.reshape(-1, w.D) for t in dys]).to(torch.bfloat16).to(dev).reshape(1, -1, w.D)
    zero_grads(single, xa)
    ya = single(xa)
    ya.backward(dya)
    single.check_status()
    T, El = w.T, w.E // world
    rep = {"status": int(st.item()), "tokens_compared": T, "tokens_single_gpu_run": T * world}
    rep["routing_equal"] = bool(torch.equal(single.router._last_selected_experts[:T], ep_layer.router._last_selected_experts)
                                and torch.equal(single.router._last_counts, ep_layer.router._last_counts))
    rel = lambda a, b: closeness(a.float(), b.float(), 2e-2)
    worst = 0.0
    r_ = rel(y.detach().reshape(-1, w.D), ya.detach().reshape(-1, w.D)[:T]); rep["y_rel_fro"] = r_["rel_fro"]
    worst = max(worst, r_["max_ratio"])
    r_ = rel(xg.grad.reshape(-1, w.D), xa.grad.reshape(-1, w.D)[:T]); rep["dx_rel_fro"] = r_["rel_fro"]
    worst = max(worst, r_["max_ratio"])
    named1 = dict(single.named_parameters())
    shard = 0.0
    for name, p in ep_layer.named_parameters():
        if getattr(p, "expert_shard", False):
            r_ = rel(p.grad, named1[name].grad[:El])
            shard = max(shard, r_["rel_fro"])
            worst = max(worst, r_["max_ratio"])
    rep["shard_grad_rel_fro"] = shard
    dense = 0.0
    for name, g in replicated.items():
        r_ = rel(g, named1[name].grad)
        dense = max(dense, r_["rel_fro"])
        worst = max(worst, r_["max_ratio"])
    rep["replicated_grad_rel_fro"] = dense
    rep["max_elementwise_ratio_to_2e-2_bound"] = worst
    rep["reference"] = "the same layer with all experts on one GPU (itself checked against the fp32 oracle in tests/)"
    rep["ok"] = bool(rep["status"] == 0 and rep["routing_equal"] and worst <= 3.0 and
                     max(rep["y_rel_fro"], rep["dx_rel_fro"], shard, dense) <= 1e-2)
    return rep


def build_layer(w, rank, device, ep_group=None, ep_mode="p2p_dedup"):
    """The layer with seed-0 parameters (identical on every rank) and this rank's own tokens (seed = rank).
    With `ep_group` the routed experts are sharded: this rank keeps experts [rank*E/G, (rank+1)*E/G)."""
    from swamla_b200.layer import LatentMoELayer
    params, buffers, x, dy = inputs.make_inputs(w, seed=0)
    x, dy = tokens_of_rank(w, rank, x, dy)
    cfg = w.config()
    if w.dtype == "fp8":
        cfg.moe_fp8 = True          # routed expert GEMMs in e4m3 with per-tensor scaling (BASELINE cfg 4)
    state = {**params, **buffers}
    if ep_group is not None:
        import torch.distributed as dist
        cfg.ep_group = ep_group
        cfg.ep_mode = ep_mode
        G = dist.get_world_size(ep_group)
        El = w.E // G
        for k in ("experts.gate_up_weight", "experts.down_weight"):
            state[k] = state[k][rank * El:(rank + 1) * El].clone()
    layer = LatentMoELayer(cfg)
    layer.load_state_dict(state, strict=True)
    layer = layer.to(device).to(torch.bfloat16).train()
    return layer, x.to(torch.bfloat16), dy.to(torch.bfloat16)


def time_steps(layer, x, dy, steps, warmup):
    """ms per fwd+bwd step on this rank alone (CUDA events on the current stream)."""
    for _ in range(warmup):
        zero_grads(layer, x)
        step(layer, x, dy)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        zero_grads(layer, x)
        step(layer, x, dy)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def step(layer, x, dy):
    """One fwd+bwd through the public module API; gradients accumulate into .grad as in training."""
    y = layer(x)
    y.backward(dy)
    return y


def zero_grads(layer, x):
    for p in layer.parameters():
        p.grad = None
    x.grad = None


def cpu_baseline(w, threads):
    """Oracle fwd+bwd in fp32 on the host cores over a bounded sample of the workload."""
    from oracle import latent_moe_ref as R
    torch.set_num_threads(threads)
    params, buffers, x, dy = inputs.make_inputs(w, seed=0, tokens=CPU_SAMPLE_TOKENS)
    best = None
    for i in range(3):
        t0 = time.perf_counter()
        R.layer_forward_backward(params, buffers, x, dy, w.K, z_loss_coef=w.router_z_loss_coef)
        dt = time.perf_counter() - t0
        if i > 0:
            best = dt if best is None else min(best, dt)
    return CPU_SAMPLE_TOKENS / best, best


def run_reference(args, w):
    """--impl reference: the CPU oracle (a port of the reference layer; the reference itself is Python/Triton
    with no CPU path) timed on all host cores; each step = fwd+bwd over CPU_SAMPLE_TOKENS tokens."""
    from oracle import latent_moe_ref as R
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    params, buffers, x, dy = inputs.make_inputs(w, seed=0, tokens=CPU_SAMPLE_TOKENS)
    for _ in range(max(1, min(args.warmup, 2))):
        R.layer_forward_backward(params, buffers, x, dy, w.K, z_loss_coef=w.router_z_loss_coef)
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        R.layer_forward_backward(params, buffers, x, dy, w.K, z_loss_coef=w.router_z_loss_coef)
    dt = (time.perf_counter() - t0) / steps
    value = CPU_SAMPLE_TOKENS / dt
    sample = f"{CPU_SAMPLE_TOKENS} tokens of {w.name} per step, fp32 torch CPU, {steps} steps"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, args.gpus, "cpu"),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(w, n_gpus, parallelism, launch="eager"):
    return {
        "workload": f"{w.name}: LatentMoE FFN fwd+bwd, x[{w.batch},{w.seq},{w.D}] {w.dtype} per GPU, "
                    f"E={w.E} top-{w.K} latent={w.L} F={w.F} Fs={w.Fs} n_shared={w.n_shared_experts}",
        "tokens_per_step_per_gpu": w.T, "parallelism": parallelism, "launch": launch,
        "l2": "per-step working set (~1.5 GB of activations at cfg2) exceeds the 126 MB L2; no explicit flush",
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-sustained", action="store_true", help="skip the second, seconds-long timed region (N=1)")
    ap.add_argument("--ep-mode", default="p2p_dedup", choices=["p2p_dedup", "p2p", "nccl"])
    ap.add_argument("--no-graphs", action="store_true", help="eager launches instead of CUDA-graph replay (N=1)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    wname = args.workload or ("cfg2" if args.gpus == 1 else "cfg5")
    w = inputs.WORKLOADS[wname]
    if args.impl == "reference":
        run_reference(args, w)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from swamla_b200 import _cabi
    lib = _cabi.load()
    same_workload_1gpu = None
    parity = None
    layer, x_host, dy_host = build_layer(w, rank, dev, ep_group=dist.group.WORLD if world > 1 else None,
                                         ep_mode=args.ep_mode)
    x = x_host.to(dev).requires_grad_(True)
    dy = dy_host.to(dev)
    if world > 1:
        # Before anything is timed: the expert-parallel step must reproduce the single-GPU layer on the real config.
        l1 = xh1 = dyh1 = None
        if rank == 0:
            l1, xh1, dyh1 = build_layer(w, 0, dev)
        parity = ep_parity(w, layer, l1, rank, world, dev, dist)
        flag = torch.tensor([1 if (rank != 0 or parity["ok"]) else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if flag.item() == 0:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "error": "expert-parallel step does not match the single-GPU layer",
                                  "ep_parity": parity, "n_gpus": world}))
            dist.destroy_process_group()
            sys.exit(1)
        if rank == 0:
            # the same per-GPU workload on ONE GPU with all experts local: the denominator of the
            # expert-parallel scaling efficiency (measured here because N=1 defaults to another workload)
            x1 = xh1.to(dev).requires_grad_(True)
            ms1 = time_steps(l1, x1, dyh1.to(dev), max(3, args.steps // 2), args.warmup)
            same_workload_1gpu = w.T / (ms1 * 1e-3)
            del l1, x1, xh1, dyh1
            torch.cuda.empty_cache()
        dist.barrier()
    use_graphs = world == 1 and not args.no_graphs
    eager_layer = layer
    if use_graphs:
        # the user-facing way to run a fixed-shape training step: forward and backward replayed as CUDA graphs
        from swamla_b200.graphs import GraphedLatentMoE
        layer = GraphedLatentMoE(layer, x)

    def barrier():
        if dist is not None:
            dist.barrier()

    # ---------------- device-resident timing ----------------
    for _ in range(args.warmup):
        zero_grads(layer, x)
        step(layer, x, dy)
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.lmoe_launch_count()
    ev0.record()
    for _ in range(args.steps):
        zero_grads(layer, x)
        step(layer, x, dy)
    ev1.record()
    torch.cuda.synchronize()
    barrier()
    launches = lib.lmoe_launch_count() - launches0
    ms_total = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    # A second, longer measurement (N=1 only): blocks of `steps` steps back to back for about SUSTAINED_SECONDS, so that
    # the GPU reaches the clocks it holds under a lasting load; median and best block, clocks and power sampled beside.
    sustained = None
    if world == 1 and not args.no_sustained:
        n_blocks = max(10, int(SUSTAINED_SECONDS * 1e3 / max(ms_total, 1e-3)) + 1)
        s2 = ClockSampler(local_rank)
        s2.start()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_blocks + 1)]
        evs[0].record()
        for b in range(n_blocks):
            for _ in range(args.steps):
                zero_grads(layer, x)
                step(layer, x, dy)
            evs[b + 1].record()
        torch.cuda.synchronize()
        c2 = s2.stop()
        per = sorted(evs[b].elapsed_time(evs[b + 1]) / args.steps for b in range(n_blocks))
        sustained = {"blocks": n_blocks, "steps_per_block": args.steps, "seconds": evs[0].elapsed_time(evs[-1]) * 1e-3,
                     "ms_per_step_median": per[len(per) // 2], "ms_per_step_min": per[0], "clocks": c2}
    # per-launch timing of the GEMM kernel over a few extra steps (not part of the timed region)
    gemm_prof = None
    if rank == 0:
        import ctypes
        prof_steps = 5
        lib.lmoe_profile_enable(1)
        eager_launches0 = lib.lmoe_launch_count()
        for _ in range(prof_steps):          # eager launches: events cannot bracket kernels inside a replayed graph
            zero_grads(eager_layer, x)
            step(eager_layer, x, dy)
        torch.cuda.synchronize()
        ms_, n_ = ctypes.c_float(0), ctypes.c_int(0)
        lib.lmoe_profile_collect(ctypes.byref(ms_), ctypes.byref(n_))
        lib.lmoe_profile_enable(0)
        gemm_prof = (ms_.value / prof_steps, n_.value // prof_steps)
        if use_graphs:   # kernels inside the replayed graphs do not pass the library's launch counter: count an eager step
            launches = (lib.lmoe_launch_count() - eager_launches0) // prof_steps * args.steps
    elif world > 1:
        for _ in range(5):
            zero_grads(layer, x)
            step(layer, x, dy)
        torch.cuda.synchronize()
    t = torch.tensor([ms_total], device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = t.item()
    ms_per_step = ms_total / args.steps
    tokens_per_s = w.T * world / (ms_per_step * 1e-3)

    # ---------------- end to end with host buffers ----------------
    e2e = None
    if not args.no_e2e:
        xh, dyh = x_host.pin_memory(), dy_host.pin_memory()
        yh = [torch.empty_like(x_host).pin_memory() for _ in range(2)]
        auxh = torch.empty(2, dtype=torch.float32).pin_memory()
        xd = [torch.empty_like(x) for _ in range(2)]
        dyd = [torch.empty_like(dy) for _ in range(2)]
        s_h2d, s_d2h = torch.cuda.Stream(), torch.cuda.Stream()
        main_s = torch.cuda.current_stream()

        def e2e_loop(n):
            done = [None, None]      # compute finished with buffer b
            copied = [None, None]    # D2H finished with buffer b
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(s_h2d):
                    if done[b] is not None:
                        s_h2d.wait_event(done[b])
                    xd[b].copy_(xh, non_blocking=True)
                    dyd[b].copy_(dyh, non_blocking=True)
                    ready = torch.cuda.Event()
                    ready.record(s_h2d)
                main_s.wait_event(ready)
                zero_grads(layer, x)
                xin = xd[b].detach().requires_grad_(True)
                y = layer(xin)
                y.backward(dyd[b])
                aux = layer.get_aux_loss().detach()
                done[b] = torch.cuda.Event()
                done[b].record(main_s)
                with torch.cuda.stream(s_d2h):
                    s_d2h.wait_event(done[b])
                    if copied[b] is not None:
                        s_d2h.wait_event(copied[b])
                    yh[b].copy_(y.detach(), non_blocking=True)
                    auxh[b:b + 1].copy_(aux.reshape(1), non_blocking=True)
                    y.record_stream(s_d2h)
                    copied[b] = torch.cuda.Event()
                    copied[b].record(s_d2h)
            torch.cuda.synchronize()

        e2e_loop(args.warmup)
        barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_loop(args.steps)
        e1.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3
        ms_e2e = max(e0.elapsed_time(e1), wall)   # the D2H stream may finish after the main stream's event
        barrier()
        t = torch.tensor([ms_e2e], device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = t.item() / args.steps
        e2e = {"value": w.T * world / (ms_e2e * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": 2 * x_host.numel() * 2, "d2h_bytes_per_step": x_host.numel() * 2 + 4,
               "ms_per_step": ms_e2e}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    pk = peaks()
    flops_step = 3 * w.flops_fwd_per_token() * w.T        # per GPU
    achieved = flops_step / (ms_per_step * 1e-3) / 1e12
    # dominant kernel = the tcgen05 GEMM kernels (every GEMM of the step is an instantiation of one of the two): their summed launch
    # durations, measured here with CUDA events around each launch on its stream over `prof_steps` extra steps
    gemm_tflops = gemm_ms_step = None
    gemm_launches = 0
    if gemm_prof is not None:
        gemm_ms_step, gemm_launches = gemm_prof
        gemm_tflops = flops_step / (gemm_ms_step * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "lmoe::gemm_pair_kernel (dense, cta_group::2) + lmoe::gemm_kernel (grouped): all tcgen05 GEMM "
                          "launches of a step",
                "achieved": gemm_tflops, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                "frac": None if gemm_tflops is None else gemm_tflops / pk["bf16_tflops"],
                "traffic": TRAFFIC_BYTES_PER_STEP.get(w.name),
                "traffic_note": "dram read+write bytes of all tcgen05 GEMM launches of one step from an ncu capture of "
                                "the current kernels; null where none exists for this workload",
                "gemm_ms_per_step": gemm_ms_step, "gemm_launches_per_step": gemm_launches,
                "algorithmic_flops_per_step": flops_step,
                "peak_source": f"{pk['source']} cuBLAS bf16 burst (sustained {pk['bf16_tflops_sustained']})",
                "step_achieved": achieved, "step_frac": achieved / pk["bf16_tflops"],
                "step_scope": "whole fwd+bwd step per GPU (all kernels, launch gaps included): "
                              "3 x GEMM FLOPs of the forward (router, down, routed, up, shared)",
                "flops_per_token_fwd_bwd": 3 * w.flops_fwd_per_token()}
    out = {
        "metric": METRIC, "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if w.dtype != "fp8" else "bf16 (routed expert GEMMs e4m3)",
        "data": "synthetic",
        "config": workload_config(w, world, "single GPU" if world == 1 else
                                  f"ep{world}: experts sharded {w.E // world} per GPU, tokens data-parallel, "
                                  + {"p2p_dedup": "one-sided NVLink stores, one row per (token, destination rank), "
                                                  "partial sums on the owner",
                                     "p2p": "one-sided NVLink stores into symmetric buffers, one row per (token, expert)",
                                     "nccl": "dispatch/combine all-to-all (NCCL) of latent rows"}[args.ep_mode],
                                  launch="CUDA graphs (forward, backward)" if use_graphs else "eager"),
        "clocks": clocks, "gpu_launches": int(launches), "roofline": roofline,
    }
    if sustained is not None:
        tps = w.T / (sustained["ms_per_step_median"] * 1e-3)
        sustained["tokens_per_s_median"] = tps
        sustained["step_tflops_median"] = tps * 3 * w.flops_fwd_per_token() / 1e12
        if pk["bf16_tflops_sustained"]:
            sustained["step_frac_of_sustained_peak"] = sustained["step_tflops_median"] / pk["bf16_tflops_sustained"]
            sustained["peak_sustained_tflops"] = pk["bf16_tflops_sustained"]
        out["sustained"] = sustained
    if e2e is not None:
        out["e2e"] = e2e
    if parity is not None:
        out["ep_parity"] = parity
    if same_workload_1gpu is not None:
        out["tokens_per_s_1gpu_same_workload"] = same_workload_1gpu
        out["efficiency_same_workload"] = tokens_per_s / (world * same_workload_1gpu)
        out["efficiency_note"] = ("efficiency_same_workload = value / (n_gpus x tokens_per_s_1gpu_same_workload): the same "
                                  "per-GPU workload with all experts on one GPU, eager launches, measured in this run by "
                                  "rank 0; the default N=1 line is another workload (cfg2, CUDA graphs)")
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        v, secs = cpu_baseline(w, threads)
        out["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port",
                               "sample": f"{CPU_SAMPLE_TOKENS} tokens of {w.name}, fwd+bwd, fp32 torch CPU, "
                                         f"best of 2 after 1 warm-up ({secs:.2f} s)"}
    print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
