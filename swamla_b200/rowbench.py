"""Achieved HBM bandwidth of the library's memory-bound kernels (routing, gather, combine, SwiGLU adjoint, e4m3
quantisation, casts) at a benchmark workload's shapes.

    python -m swamla_b200.rowbench [--workload cfg2] [--reps 20] [--experts]

``--experts`` times the routed expert stage instead (forward: gate_up -> SwiGLU -> down; backward: d_hidden -> SwiGLU
adjoint -> d_x) in its kernel variants: the separate grouped GEMMs (default path), the chain kernel on one CTA per tile
and on CTA pairs.  With ``LMOE_PAIR_GROUPED=1`` in the environment the "separate" rows run the grouped GEMMs on CTA pairs.

Each kernel is called through the C ABI on synthetic tensors of the workload's sizes, timed with CUDA events on the
launching stream (median of ``--reps`` launches after warm-up), with the L2 flushed by a 256 MB write between
launches.  ``bytes`` is the ALGORITHMIC traffic of one launch (every input read once, every output written once; rows
that are gathered several times count once per use because they come from L2), ``GB/s`` = bytes / time, and ``frac`` is
against the measured copy bandwidth in ``MEASURED_PEAKS.json`` when that file exists beside the package.  Prints one
markdown table.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import _cabi, workloads
from .functional import RouteTables, make_shape

BF = torch.bfloat16


def _hbm_peak():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path))["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--experts", action="store_true", help="time the routed expert stage in its kernel variants")
    args = ap.parse_args()
    w = workloads.WORKLOADS[args.workload]
    lib = _cabi.load()
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    T, D, L, E, K, F, Fs = w.T, w.D, w.L, w.E, w.K, w.F, w.Fs
    shape = make_shape(T, D, L, E, K, F, Fs)
    g = torch.Generator(device=dev).manual_seed(0)
    f32 = dict(dtype=torch.float32, device=dev)
    bf = dict(dtype=BF, device=dev)
    p = lambda t: None if t is None else t.data_ptr()

    logits = torch.randn(T, E, generator=g, **f32)
    bias = torch.zeros(E, **f32)
    sel = torch.empty(T, K, dtype=torch.int32, device=dev)
    weights = torch.empty(T, K, **f32)
    lse = torch.empty(T, **f32)
    z_partial = torch.empty((T + 7) // 8, **f32)
    z_loss = torch.empty(1, **f32)
    route = RouteTables(shape, dev)
    P = route.padded_rows
    ws = torch.empty(max(16, lib.lmoe_route_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
    x_latent = torch.randn(T, L, generator=g, **f32).to(BF)
    x_sorted = torch.empty(P, L, **bf)
    y_sorted = torch.randn(P, L, generator=g, **f32).to(BF)
    act_cat = torch.empty(T, L + Fs, **bf)
    d_routed = torch.randn(T, L, generator=g, **f32).to(BF)
    d_y_sorted = torch.empty(P, L, **bf)
    d_weights = torch.empty(T, K, **f32)
    h1 = torch.randn(P, 2 * F, generator=g, **f32).to(BF)
    d_hidden = torch.randn(P, F, generator=g, **f32).to(BF)
    d_h1 = torch.empty(P, 2 * F, **bf)
    dgrad_cat = torch.empty(T, 2 * Fs + L + E, **bf)
    h1_s = torch.randn(T, 2 * Fs, generator=g, **f32).to(BF)
    d_hidden_s = torch.randn(T, Fs, generator=g, **f32).to(BF)
    q8 = torch.empty(P, L, dtype=torch.uint8, device=dev)
    scal = torch.empty(2, **f32)
    w32 = torch.randn(E * L * 2 * F, generator=g, **f32)
    w16 = torch.empty(E * L * 2 * F, **bf)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    call = _cabi.call
    call("lmoe_gate_topk_fwd", shape, p(logits), p(bias), 0.001, p(sel), p(weights), p(lse), p(z_partial), p(z_loss), st)
    call("lmoe_route_permute", shape, p(sel), route.struct, p(ws), ws.numel(), st)
    torch.cuda.synchronize()
    used = int(route.n_tiles.item()) * 128            # padded rows in use
    n = T * K

    kernels = [
        ("gate_topk (sigmoid, top-%d of %d, lse)" % (K, E), T * E * 4 + n * 8 + T * 4,
         lambda: call("lmoe_gate_topk_fwd", shape, p(logits), p(bias), 0.001, p(sel), p(weights), p(lse), p(z_partial),
                      p(z_loss), st)),
        ("route hist + scan + scatter (3 launches)", 2 * n * 4 + 3 * n * 4 + used * 4,
         lambda: call("lmoe_route_permute", shape, p(sel), route.struct, p(ws), ws.numel(), st)),
        ("gather_rows (latent rows -> padded layout)", T * L * 2 + used * L * 2,
         lambda: call("lmoe_gather_rows", p(x_latent), p(route.row_src), K, P, L, p(route.n_tiles), p(x_sorted), st)),
        ("combine (weighted sum of K rows per token)", n * L * 2 + T * L * 2,
         lambda: call("lmoe_combine_rows", p(y_sorted), p(route.pos), p(weights), T, K, L, p(act_cat), L + Fs, st)),
        ("combine_bwd (d_y rows + gating gradients)", 2 * used * L * 2 + T * L * 2,
         lambda: call("lmoe_combine_bwd", shape, p(d_routed), p(y_sorted), p(weights), route.struct, p(d_y_sorted),
                      p(d_weights), st)),
        ("unpermute_sum_bwd (gather adjoint)", n * L * 2 + T * L * 2,
         lambda: call("lmoe_unpermute_sum_bwd", shape, p(y_sorted), route.struct, p(dgrad_cat), st)),
        ("swiglu_bwd, routed rows", used * F * 2 * 5,
         lambda: call("lmoe_swiglu_bwd", P, F, p(h1), p(d_hidden), p(d_h1), 2 * F, p(route.n_tiles), st)),
        ("swiglu_bwd, shared expert", T * Fs * 2 * 5,
         lambda: call("lmoe_swiglu_bwd", T, Fs, p(h1_s), p(d_hidden_s), p(dgrad_cat), 2 * Fs + L + E, None, st)),
        ("gate_topk_bwd (router adjoint)", T * E * 4 + T * E * 2 + n * 16,
         lambda: call("lmoe_gate_topk_bwd", shape, p(logits), p(sel), p(weights), p(d_weights), p(lse), None, 0.001,
                      p(dgrad_cat), st)),
        ("fp8_quantize (amax + e4m3 cast of x_sorted)", used * L * (2 + 2 + 1),
         lambda: call("lmoe_fp8_quantize", p(x_sorted), P, L, p(route.n_tiles), p(q8), p(scal[0:1]), p(scal[1:2]), st)),
        ("cast fp32 -> bf16 (expert gate_up weights)", w32.numel() * 6,
         lambda: call("lmoe_cast_f32_to_bf16", p(w32), p(w16), w32.numel(), st)),
    ]
    peak, src = _hbm_peak()

    def median_us(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(args.reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    if args.experts:
        wgu = (torch.randn(E, L, 2 * F, generator=g, **f32) * 0.05).to(BF)
        wd = (torch.randn(E, F, L, generator=g, **f32) * 0.05).to(BF)
        call("lmoe_gather_rows", p(x_latent), p(route.row_src), K, P, L, p(route.n_tiles), p(x_sorted), st)
        hidden = torch.empty(P, F, **bf)
        d_x = torch.empty(P, L, **bf)
        call("lmoe_combine_bwd", shape, p(d_routed), p(y_sorted), p(weights), route.struct, p(d_y_sorted), p(d_weights), st)
        te, nt, po = p(route.tile_expert), p(route.n_tiles), p(route.pad_offsets)

        def fwd(pairs):
            call("lmoe_grouped_fwd", P, E, L, F, p(x_sorted), p(wgu), p(wd), te, nt, po if pairs else None, p(h1), p(hidden),
                 p(y_sorted), p(status), st)

        def bwd(pairs, scratch):
            call("lmoe_grouped_bwd_dgrad", P, E, L, F, p(d_y_sorted), p(h1), p(wgu), p(wd), te, nt, po if pairs else None,
                 p(d_hidden) if scratch else None, p(d_h1), p(d_x), p(status), st)

        status = torch.zeros(1, dtype=torch.int32, device=dev)
        fb = used * (L * 2 + 2 * F * 2 + F * 2 + L * 2)          # x_sorted in; h1, hidden, y_sorted out
        bb = used * (L * 2 + 2 * F * 2 + 2 * F * 2 + L * 2)      # d_y_sorted, h1 in; d_h1, d_x_sorted out
        flops_f, flops_b = used * 6 * L * F, used * 6 * L * F
        print(f"# Routed expert stage at {w.name}: {used} padded rows ({used // 128} tiles), E={E} L={L} F={F}; algorithmic "
              f"bytes forward {fb / 1e6:.0f} MB, backward (data gradients) {bb / 1e6:.0f} MB; {flops_f / 1e9:.1f} GFLOP each\n")
        print("| variant | forward us | GB/s | TFLOP/s | backward us | GB/s | TFLOP/s |")
        print("|---|---|---|---|---|---|---|")
        variants = [("separate grouped GEMMs, SwiGLU adjoint as a streaming kernel", 0, True, True),
                    ("separate grouped GEMMs, SwiGLU adjoint in the d_hidden GEMM's epilogue (default)", 0, True, False),
                    ("chain kernel, one CTA per tile", 1, False, False),
                    ("chain kernel, CTA pairs of one expert", 1, True, False)]
        for name, chain, pairs, scratch in variants:
            prev = lib.lmoe_chain_enable(chain)
            try:
                if chain and not lib.lmoe_chain_applies(L, F):
                    continue
                tf = median_us(lambda: fwd(pairs))
                tb = median_us(lambda: bwd(pairs, scratch))
            finally:
                lib.lmoe_chain_enable(prev)
            print(f"| {name} | {tf:.1f} | {fb / tf / 1e3:.0f} | {flops_f / tf / 1e6:.0f} | {tb:.1f} | {bb / tb / 1e3:.0f} | "
                  f"{flops_b / tb / 1e6:.0f} |")
        torch.cuda.synchronize()
        assert status.item() == 0
        return

    print(f"# HBM-bound kernels at {w.name}: T={T} E={E} K={K} L={L} F={F} Fs={Fs}, padded rows in use {used}; "
          f"HBM peak {peak:.0f} GB/s ({src} copy bandwidth)\n")
    print("| kernel | algorithmic bytes | us (median) | GB/s | frac of peak |")
    print("|---|---|---|---|---|")
    for name, nbytes, fn in kernels:
        us = median_us(fn)
        gbs = nbytes / us / 1e3
        print(f"| {name} | {nbytes / 1e6:.1f} MB | {us:.1f} | {gbs:.0f} | {gbs / peak:.2f} |")


if __name__ == "__main__":
    main()
