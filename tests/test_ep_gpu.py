"""Expert-parallel kernels and the two-GPU exchange."""
import os
import sys

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("G,E,rank", [(2, 32, 1), (8, 256, 3), (4, 128, 0), (1, 16, 0)])
def test_ep_plan_kernel_matches_reference_tables(G, E, rank):
    from oracle import ep_ref
    from swamla_b200 import _cabi
    g = torch.Generator().manual_seed(G * 1000 + E)
    counts_all = torch.randint(0, 300, (G, E), generator=g, dtype=torch.int32)
    counts_all[:, ::5] = 0                                          # some empty experts
    recv_pos, row_src, pad_offsets, tile_expert, n_tiles = ep_ref.regroup_tables(counts_all, rank)
    dev = torch.device("cuda:0")
    El = E // G
    n_recv = recv_pos.numel()
    P = (n_recv + 127) // 128 * 128 + El * 128
    i32 = dict(dtype=torch.int32, device=dev)
    d = dict(recv_pos=torch.full((max(n_recv, 1),), -9, **i32), row_src=torch.full((P,), -9, **i32),
             pad_offsets=torch.full((El + 1,), -9, **i32), tile_expert=torch.full((P // 128,), -9, **i32),
             n_tiles=torch.full((1,), -9, **i32))
    _cabi.call("lmoe_ep_plan", counts_all.to(dev).data_ptr(), G, E, rank, d["recv_pos"].data_ptr(), d["row_src"].data_ptr(),
               d["pad_offsets"].data_ptr(), d["tile_expert"].data_ptr(), d["n_tiles"].data_ptr(),
               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert d["n_tiles"].item() == n_tiles
    assert torch.equal(d["pad_offsets"].cpu().long(), pad_offsets)
    assert torch.equal(d["recv_pos"].cpu().long()[:n_recv], recv_pos)
    assert torch.equal(d["row_src"].cpu().long()[:n_tiles * 128], row_src)
    assert torch.equal(d["tile_expert"].cpu().long()[:n_tiles], tile_expert)


def _ep_worker(rank, world, port, tmpdir, mode):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import inputs, latent_moe_ref as R
        from swamla_b200.layer import LatentMoELayer
        w = inputs.WORKLOADS["tiny_ragged"]
        params, buffers, _, _ = inputs.make_inputs(w, seed=0)
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(1, 200 + 57 * rank, w.D, generator=g)
        dy = torch.randn(1, 200 + 57 * rank, w.D, generator=g)
        dev = torch.device("cuda", rank)
        El = w.E // world

        def build(ep):
            cfg = w.config()
            if ep:
                cfg.ep_group = dist.group.WORLD
                cfg.ep_mode = mode
            layer = LatentMoELayer(cfg)
            state = {**params, **buffers}
            if ep:
                state["experts.gate_up_weight"] = params["experts.gate_up_weight"][rank * El:(rank + 1) * El]
                state["experts.down_weight"] = params["experts.down_weight"][rank * El:(rank + 1) * El]
            layer.load_state_dict(state, strict=True)
            return layer.to(dev).to(torch.bfloat16).train()

        single, ep = build(False), build(True)
        outs = []
        for layer in (single, ep):
            for _ in range(2):                      # twice: the second step reuses the exchange buffers
                for p_ in layer.parameters():
                    p_.grad = None
                xg = x.to(dev).to(torch.bfloat16).requires_grad_(True)
                y = layer(xg)
                (y.float() * dy.to(dev).to(torch.bfloat16).float()).sum().backward()
            outs.append((y.detach(), xg.grad, layer))
        torch.cuda.synchronize()
        (y1, dx1, l1), (y2, dx2, l2) = outs
        l2.check_status()                           # no overflow (201), no expired wait (101-103) on any step
        # routing is local and identical; a row's result does not depend on where it sits in an expert's segment
        assert torch.equal(l1.router._last_selected_experts, l2.router._last_selected_experts)
        dense = ("router.gate.weight", "down_proj.weight", "up_proj.weight", "shared_experts.0.gate_up_proj.weight",
                 "shared_experts.0.down_proj.weight")
        if mode == "p2p_dedup":
            # partial sums per owner travel in bf16: one more rounding than the single-GPU combine, so the comparison
            # is within the bf16 tolerance of the path (rtol 2e-2) instead of bit for bit
            for a, b, what in [(y2, y1, "y"), (dx2, dx1, "dx")] + [
                    (dict(l2.named_parameters())[n].grad, dict(l1.named_parameters())[n].grad, n) for n in dense]:
                ok, rep = R.within_tolerance(a.float().cpu(), b.float().cpu(), 2e-2)
                assert ok, (what, rep)
                assert R.closeness(a.float().cpu(), b.float().cpu(), 2e-2)["rel_fro"] < 5e-3, what
        else:
            assert torch.equal(y1, y2), (y1.float() - y2.float()).abs().max().item()
            assert torch.equal(dx1, dx2)
            for name in dense:
                a, b = dict(l1.named_parameters())[name].grad, dict(l2.named_parameters())[name].grad
                assert torch.equal(a, b), name
        # expert shard gradients: the owner sums over the tokens of ALL ranks
        for name in ("experts.gate_up_weight", "experts.down_weight"):
            full = dict(l1.named_parameters())[name].grad.float()          # this rank's tokens, all experts
            dist.all_reduce(full)                                            # all ranks' tokens
            shard = dict(l2.named_parameters())[name].grad.float()
            ok, rep = R.within_tolerance(shard.cpu(), full[rank * El:(rank + 1) * El].cpu(), 2e-2)
            assert ok, (name, rep)
        # global load histogram for the bias update
        c1 = l1.router._last_counts.clone()
        dist.all_reduce(c1)
        assert torch.equal(c1, l2.router._last_counts)
        # the ranks hold different token counts (200 vs 257): the bias update takes the expected load from the summed
        # histogram, so the replicated selection bias stays identical on every rank
        l2.router.update_bias_from_last_forward()
        biases = [torch.empty_like(l2.router.expert_bias) for _ in range(world)]
        dist.all_gather(biases, l2.router.expert_bias)
        assert all(torch.equal(b_, biases[0]) for b_ in biases) and biases[0].abs().max().item() > 0
        open(os.path.join(tmpdir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["nccl", "p2p", "p2p_dedup"])
def test_expert_parallel_layer_matches_single_gpu_layer(tmp_path, mode):
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 300) + {"nccl": 0, "p2p": 7, "p2p_dedup": 13}[mode]
    mp.spawn(_ep_worker, args=(2, port, str(tmp_path), mode), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
