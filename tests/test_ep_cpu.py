"""Expert-parallel host logic on CPU: two gloo ranks exchange rows exactly as the GPU path does (same split
sizes, same receive order, same regroup contract) and must reproduce the single-rank oracle."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import inputs, latent_moe_ref as R, ep_ref
        from swamla_b200.ep import splits_from_counts
        w = inputs.WORKLOADS["tiny_ragged"]                         # E = 32, K = 8, L = 64
        params, buffers, _, _ = inputs.make_inputs(w, seed=0)       # same parameters on every rank
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(1, 50 + 13 * rank, w.D, generator=g)        # different token counts per rank
        E, K, L, El = w.E, w.K, w.L, w.E // world
        with torch.no_grad():
            ref = R.layer_forward(params, buffers, x, K)            # all experts local: the expected result
        # --- what the GPU path does, in torch ---
        counts_all = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(counts_all, ref["counts"].to(torch.int32))
        counts_all = torch.stack(counts_all)
        send_splits, recv_splits = splits_from_counts(counts_all, rank)
        assert sum(send_splits) == x.shape[1] * K
        send_rows = ref["x_sorted"].contiguous()                    # expert order = destination order
        recv_rows = torch.empty(sum(recv_splits), L)
        dist.all_to_all_single(recv_rows, send_rows, recv_splits, send_splits)
        recv_pos, row_src, pad_offsets, tile_expert, n_tiles = ep_ref.regroup_tables(counts_all, rank)
        x_sorted = torch.zeros(n_tiles * 128, L)
        valid = row_src >= 0
        x_sorted[valid] = recv_rows[row_src[valid]]
        # local experts over the padded layout
        lo, hi = rank * El, (rank + 1) * El
        wgu, wd = params["experts.gate_up_weight"][lo:hi], params["experts.down_weight"][lo:hi]
        h1 = R.grouped_gemm(x_sorted, wgu, pad_offsets)
        gate, up = h1.chunk(2, -1)
        y_sorted = R.grouped_gemm(torch.nn.functional.silu(gate) * up, wd, pad_offsets)
        y_recv = y_sorted[recv_pos]
        y_back = torch.empty(sum(send_splits), L)
        dist.all_to_all_single(y_back, y_recv, send_splits, recv_splits)
        torch.testing.assert_close(y_back, ref["y_sorted"], rtol=1e-5, atol=1e-6)
        inv = torch.empty_like(ref["perm"])
        inv[ref["perm"]] = torch.arange(inv.numel())
        T = x.shape[1]
        routed = (ref["weights"].reshape(T, K, 1) * y_back[inv].view(T, K, L)).sum(1)
        torch.testing.assert_close(routed, ref["routed"], rtol=1e-5, atol=1e-6)
        # every received row sits in the segment of its expert, sources in rank order
        assert torch.equal(tile_expert, torch.repeat_interleave(torch.arange(El), (pad_offsets[1:] - pad_offsets[:-1]) // 128))
        open(os.path.join(tmpdir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_exchange_reproduces_single_rank_oracle(tmp_path):
    port = 29500 + (os.getpid() % 500)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_splits_from_counts():
    from swamla_b200.ep import splits_from_counts
    counts_all = torch.tensor([[1, 2, 3, 4], [5, 6, 7, 8]], dtype=torch.int32)      # G = 2, E = 4
    assert splits_from_counts(counts_all, 0) == ([3, 7], [3, 11])
    assert splits_from_counts(counts_all, 1) == ([11, 15], [7, 15])


def test_regroup_tables_contract():
    from oracle import ep_ref
    counts_all = torch.tensor([[3, 0, 130, 1], [2, 0, 5, 0]], dtype=torch.int32)
    recv_pos, row_src, pad_offsets, tile_expert, n_tiles = ep_ref.regroup_tables(counts_all, 1)   # experts 2, 3
    assert pad_offsets.tolist() == [0, 256, 384] and n_tiles == 3 and tile_expert.tolist() == [0, 0, 1]
    # receive order: (s0,e2) x130, (s0,e3) x1, (s1,e2) x5 ; padded: e2: s0 rows, s1 rows ; e3: s0 row
    assert recv_pos[:130].tolist() == list(range(130)) and recv_pos[130].item() == 256
    assert recv_pos[131:].tolist() == list(range(130, 135))
    assert (row_src[135:256] == -1).all() and row_src[256].item() == 130 and (row_src[257:] == -1).all()


def _ckpt_worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import inputs
        from swamla_b200.ep import ddp_ignore_expert_shards, expert_shard_parameter_names
        from swamla_b200.layer import LatentMoELayer
        w = inputs.WORKLOADS["tiny_ragged"]
        params, buffers, _, _ = inputs.make_inputs(w, seed=0)
        full_state = {**params, **buffers}                                     # the reference's state_dict layout
        cfg = w.config()
        cfg.ep_group = dist.group.WORLD
        layer = LatentMoELayer(cfg)
        El = w.E // world
        assert layer.experts.gate_up_weight.shape[0] == El
        # a reference checkpoint (all experts) loads into the sharded layer: every rank takes its block
        layer.load_state_dict(full_state, strict=True)
        for name in ("gate_up_weight", "down_weight"):
            assert torch.equal(getattr(layer.experts, name), params["experts." + name][rank * El:(rank + 1) * El])
        assert full_state["experts.gate_up_weight"].shape[0] == w.E              # the caller's dict is untouched
        # state_dict() is local (no collective: a rank-0-only save cannot hang) and returns this rank's block
        local = layer.state_dict()
        assert set(local) == set(full_state)
        assert torch.equal(local["experts.down_weight"], params["experts.down_weight"][rank * El:(rank + 1) * El])
        # the collective helper gathers the blocks back into the reference layout, identical on every rank
        from swamla_b200.ep import gather_full_state_dict
        saved = gather_full_state_dict(layer)
        assert set(saved) == set(full_state)
        for k, v in full_state.items():
            assert saved[k].shape == v.shape and torch.equal(saved[k].to(v.dtype), v), k
        # block-shaped tensors load as well (a checkpoint written per rank)
        shard_state = dict(full_state)
        for name in ("experts.gate_up_weight", "experts.down_weight"):
            shard_state[name] = full_state[name][rank * El:(rank + 1) * El] + 1.0
        layer.load_state_dict(shard_state, strict=True)
        assert torch.equal(layer.experts.down_weight, shard_state["experts.down_weight"])
        # DDP: the shards are ignored, their gradients scaled like DDP's average
        model = torch.nn.Sequential(layer)
        names = ddp_ignore_expert_shards(model)
        assert names == ["0.experts.gate_up_weight", "0.experts.down_weight"] == expert_shard_parameter_names(model)
        assert model._ddp_params_and_buffers_to_ignore == names
        ddp = torch.nn.parallel.DistributedDataParallel(model)
        reduced = {n for n, p_ in ddp.module.named_parameters()} - set(ddp.parameters_to_ignore)
        assert "0.experts.gate_up_weight" not in reduced and "0.router.gate.weight" in reduced
        layer.experts.gate_up_weight.grad = None
        (layer.experts.gate_up_weight.sum() * 3.0).backward()
        assert torch.allclose(layer.experts.gate_up_weight.grad, torch.full_like(layer.experts.gate_up_weight, 3.0 / world))
        open(os.path.join(tmpdir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_expert_shards_keep_the_reference_state_dict_layout_and_stay_out_of_ddp(tmp_path):
    port = 29500 + ((os.getpid() + 211) % 500)
    mp.spawn(_ckpt_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def _dedup_worker(rank, world, port, tmpdir):
    """The de-duplicated exchange in torch over gloo: one row per (token, destination rank) out, one partial-sum row
    per (token, owner) back; must reproduce the single-rank oracle's routed output."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import inputs, latent_moe_ref as R, ep_ref
        w = inputs.WORKLOADS["tiny_ragged"]
        params, buffers, _, _ = inputs.make_inputs(w, seed=0)
        g = torch.Generator().manual_seed(300 + rank)
        T = 40 + 9 * rank
        x = torch.randn(1, T, w.D, generator=g)
        E, K, L, El = w.E, w.K, w.L, w.E // world
        with torch.no_grad():
            ref = R.layer_forward(params, buffers, x, K)
        counts_all = [torch.zeros(E, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(counts_all, ref["counts"])
        counts_all = torch.stack(counts_all)
        tables = ep_ref.dedup_send_tables(ref["sel"], ref["weights"], counts_all, rank)
        # fewer rows than one per (token, expert) travel, and every routed row is described exactly once
        assert sum(len(t["tokens"]) for t in tables) <= T * min(K, world)
        assert sum(len(t["meta_rows"]) for t in tables) == T * K
        # "stores": every rank hands each destination its rows and routing words (object all-to-all stands in for NVLink)
        send = [dict(src=rank, tok=t["tokens"], rows=ref["x_latent"][t["tokens"]], mask=t["mask"], slots=t["slots"],
                     meta_rows=t["meta_rows"], meta_tok=t["meta_tok"], meta_w=t["meta_w"]) for t in tables]
        gathered = [None] * world
        dist.all_gather_object(gathered, send)
        incoming = [gathered[s][rank] for s in range(world)]                    # what every source wrote into this rank
        # owner: padded layout from the staged rows
        _, _, pad_offsets, tile_expert, n_tiles = ep_ref.regroup_tables(counts_all.to(torch.int32), rank)
        P = n_tiles * 128
        x_in = torch.zeros(P, L)
        w_row = torch.zeros(P)
        filled = torch.zeros(P, dtype=torch.bool)
        for m in incoming:
            stage = torch.zeros(int(m["mask"].numel()), L)
            stage[m["tok"]] = m["rows"]
            assert not filled[m["meta_rows"]].any()                              # no two routed rows share a padded row
            x_in[m["meta_rows"]] = stage[m["meta_tok"]]
            w_row[m["meta_rows"]] = m["meta_w"]
            filled[m["meta_rows"]] = True
        tot = counts_all[:, rank * El:(rank + 1) * El].sum(0)
        for j in range(El):                                                      # exactly the valid rows are filled
            seg = filled[pad_offsets[j]:pad_offsets[j + 1]]
            assert seg[:tot[j]].all() and not seg[tot[j]:].any()
        lo, hi = rank * El, (rank + 1) * El
        h1 = R.grouped_gemm(x_in, params["experts.gate_up_weight"][lo:hi], pad_offsets)
        gate, up = h1.chunk(2, -1)
        y_sorted = R.grouped_gemm(torch.nn.functional.silu(gate) * up, params["experts.down_weight"][lo:hi], pad_offsets)
        # owner: one weighted partial sum per (source, token)
        back = []
        for m in incoming:
            part = torch.zeros(int(m["mask"].numel()), L)
            for t in m["tok"].tolist():
                for k in range(K):
                    if (int(m["mask"][t]) >> k) & 1:
                        p = int(m["slots"][t, k])
                        part[t] += w_row[p] * y_sorted[p]
            back.append(dict(tok=m["tok"], rows=part[m["tok"]]))
        returned = [None] * world
        dist.all_gather_object(returned, back)
        routed = torch.zeros(T, L)
        for owner in range(world):                                               # source: add the owners' partial sums
            r = returned[owner][rank]
            routed[r["tok"]] += r["rows"]
        torch.testing.assert_close(routed, ref["routed"], rtol=1e-5, atol=1e-6)
        open(os.path.join(tmpdir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_dedup_exchange_reproduces_single_rank_oracle(tmp_path):
    port = 29500 + ((os.getpid() + 97) % 500)
    mp.spawn(_dedup_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
