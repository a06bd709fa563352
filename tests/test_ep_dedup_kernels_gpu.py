"""The kernels of the de-duplicated expert-parallel exchange on ONE GPU: the G ranks are G sets of buffers on the same
device and the "peer pointers" point at them, the kernels run rank after rank (none of them waits for another).
Checked against the CPU statement of the contract (oracle/ep_ref.py: dedup_send_tables) and plain torch arithmetic."""
import pytest
import torch

from oracle import ep_ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _ptrs(tensors, dev):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=dev)


class _Ranks:
    """G ranks' inputs, tables and exchange buffers on one device."""

    def __init__(self, G, E, K, L, tokens, seed, capacity_factor=2.0):
        from swamla_b200 import _cabi
        from swamla_b200.functional import RouteTables, make_shape
        self.G, self.E, self.K, self.L, self.El = G, E, K, L, E // G
        dev = self.dev = torch.device("cuda:0")
        self.st = torch.cuda.current_stream().cuda_stream
        g = torch.Generator().manual_seed(seed)
        i32, f32 = dict(dtype=torch.int32, device=dev), dict(dtype=torch.float32, device=dev)
        self.T = tokens
        self.stride = max(tokens)
        self.P = (int(capacity_factor * self.stride * K) + 127) // 128 * 128 + self.El * 128
        self.sel = [torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(t)]).to(torch.int32) for t in tokens]
        self.w = [torch.rand(t, K, generator=g) + 0.1 for t in tokens]
        self.x = [torch.randn(t, L, generator=g).to(BF) for t in tokens]
        self.d_routed = [torch.randn(t, L, generator=g).to(BF) for t in tokens]
        self.counts_all_cpu = torch.stack([torch.bincount(s.reshape(-1).long(), minlength=E) for s in self.sel])
        self.counts_all = self.counts_all_cpu.to(**i32)
        self.status = torch.zeros(1, **i32)
        lib = _cabi.load()
        self.route, self.inv, self.tab = [], [], []
        n = G * self.stride
        mk = lambda *shape, dtype: [torch.zeros(*shape, dtype=dtype, device=dev) for _ in range(G)]
        self.stage_x, self.stage_dy = mk(n, L, dtype=BF), mk(n, L, dtype=BF)
        self.ret_y, self.ret_dx = mk(n, L, dtype=BF), mk(n, L, dtype=BF)
        self.meta = [torch.full((self.P,), -1, dtype=torch.int64, device=dev) for _ in range(G)]
        self.mask, self.slots = mk(n, dtype=torch.int32), mk(n * K, dtype=torch.int32)
        self.dw = mk(self.stride * K, dtype=torch.float32)
        for r in range(G):
            shape = make_shape(tokens[r], 8 * L, L, E, K, 64, 8)
            route = RouteTables(shape, dev)
            ws = torch.empty(max(16, lib.lmoe_route_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
            sel_d = self.sel[r].to(dev)
            _cabi.call("lmoe_route_permute", shape, sel_d.data_ptr(), route.struct, ws.data_ptr(), ws.numel(), self.st)
            inv = torch.empty(tokens[r] * K, **i32)
            _cabi.call("lmoe_invert_perm", route.perm.data_ptr(), tokens[r] * K, inv.data_ptr(), self.st)
            t = dict(src_off=torch.empty(G * E, **i32), dst_base=torch.empty(E, **i32), seg_cum=torch.empty(self.El * G, **i32),
                     pad_offsets=torch.empty(self.El + 1, **i32), tile_expert=torch.empty(self.P // 128, **i32),
                     n_tiles=torch.empty(1, **i32), sel=sel_d, w=self.w[r].to(dev), x=self.x[r].to(dev),
                     d_routed=self.d_routed[r].to(dev))
            _cabi.call("lmoe_ep_tables", self.counts_all.data_ptr(), G, E, r, self.P, t["src_off"].data_ptr(),
                       t["dst_base"].data_ptr(), t["seg_cum"].data_ptr(), t["pad_offsets"].data_ptr(),
                       t["tile_expert"].data_ptr(), t["n_tiles"].data_ptr(), self.status.data_ptr(), self.st)
            self.route.append(route)
            self.inv.append(inv)
            self.tab.append(t)
        self.cpu_tables = None
        if capacity_factor >= 2.0:       # the CPU statement of the contract describes layouts that fit
            self.cpu_tables = [ep_ref.dedup_send_tables(self.sel[r].long(), self.w[r], self.counts_all_cpu, r)
                               for r in range(G)]

    def send(self, with_meta, expect_status=0):
        from swamla_b200 import _cabi
        G, E, K, L = self.G, self.E, self.K, self.L
        stage = self.stage_x if with_meta else self.stage_dy
        p_stage, p_meta = _ptrs(stage, self.dev), _ptrs(self.meta, self.dev)
        p_mask, p_slots = _ptrs(self.mask, self.dev), _ptrs(self.slots, self.dev)
        for r in range(G):
            t, route = self.tab[r], self.route[r]
            if with_meta:
                _cabi.call("lmoe_epd_send", t["x"].data_ptr(), t["sel"].data_ptr(), self.inv[r].data_ptr(),
                           route.offsets.data_ptr(), t["dst_base"].data_ptr(), t["w"].data_ptr(), self.T[r], K, E, G, r, L,
                           self.P, self.stride, p_stage.data_ptr(), p_meta.data_ptr(), p_mask.data_ptr(), p_slots.data_ptr(),
                           self.status.data_ptr(), self.st)
            else:
                _cabi.call("lmoe_epd_send", t["d_routed"].data_ptr(), t["sel"].data_ptr(), None, None, None, None, self.T[r],
                           K, E, G, r, L, self.P, self.stride, p_stage.data_ptr(), None, None, None, self.status.data_ptr(),
                           self.st)
        torch.cuda.synchronize()
        assert self.status.item() == expect_status

    def gather(self, r, y_sorted=None):
        from swamla_b200 import _cabi
        t = self.tab[r]
        out = torch.full((self.P, self.L), 7.0, dtype=BF, device=self.dev)
        d_w_row = None if y_sorted is None else torch.zeros(self.P, dtype=torch.float32, device=self.dev)
        stage = self.stage_x[r] if y_sorted is None else self.stage_dy[r]
        _cabi.call("lmoe_epd_gather", stage.data_ptr(), self.meta[r].data_ptr(), t["tile_expert"].data_ptr(),
                   t["n_tiles"].data_ptr(), t["pad_offsets"].data_ptr(), t["seg_cum"].data_ptr(), self.counts_all.data_ptr(),
                   self.G, self.E, r, self.L, self.P, self.G * self.stride, None if y_sorted is None else y_sorted.data_ptr(),
                   out.data_ptr(), None if d_w_row is None else d_w_row.data_ptr(), self.st)
        torch.cuda.synchronize()
        return out, d_w_row

    def expected_layout(self, r, rows_of_source):
        """Padded layout of owner r on the CPU: (rows [P, L] fp32, weight per row, filled mask, (source, token) per row)."""
        rows = torch.zeros(self.P, self.L)
        w_row = torch.zeros(self.P)
        filled = torch.zeros(self.P, dtype=torch.bool)
        origin = torch.full((self.P, 2), -1, dtype=torch.long)
        for s in range(self.G):
            m = self.cpu_tables[s][r]
            rows[m["meta_rows"]] = rows_of_source[s].float()[m["meta_tok"]]
            w_row[m["meta_rows"]] = m["meta_w"]
            filled[m["meta_rows"]] = True
            origin[m["meta_rows"], 0] = s
            origin[m["meta_rows"], 1] = m["meta_tok"]
        return rows, w_row, filled, origin


@pytest.mark.parametrize("G,E,K,L,tokens", [(2, 32, 8, 128, (150, 97)), (4, 64, 6, 256, (64, 33, 80, 5)),
                                            (8, 256, 16, 256, (40, 40, 17, 40, 3, 40, 40, 25))])
def test_dedup_exchange_kernels_match_contract(G, E, K, L, tokens):
    from swamla_b200 import _cabi
    R = _Ranks(G, E, K, L, tokens, seed=G * 100 + K)
    # ---- forward send: masks, slot tables, routing words, staged rows ----
    R.send(with_meta=True)
    for r in range(G):
        used = int(R.tab[r]["n_tiles"].item()) * 128
        exp_rows, exp_w, filled, origin = R.expected_layout(r, R.x)
        meta = R.meta[r].cpu()
        slot = (meta & 0xffffffff).to(torch.int32).long()
        wbits = (meta >> 32).to(torch.int32)
        assert torch.equal(slot[filled], origin[filled, 0] * R.stride + origin[filled, 1])
        assert torch.equal(wbits[filled].view(torch.float32), exp_w[filled])
        for s in range(G):
            m = R.cpu_tables[s][r]
            lo = s * R.stride
            assert torch.equal(R.mask[r][lo:lo + tokens[s]].cpu().long() & ((1 << K) - 1), m["mask"])
            got = R.slots[r].view(-1, K)[lo:lo + tokens[s]].cpu().long()
            live = m["mask"] != 0                                   # slot lines are written for tokens that use this rank
            assert torch.equal(got[live], m["slots"][live])
        x_in, _ = R.gather(r)
        assert torch.equal(x_in[:used].float().cpu(), exp_rows[:used])          # pad rows zero, valid rows exact copies
        assert (x_in[used:].float() == 7.0).all()                                # nothing beyond the tiles in use
    # ---- forward return: weighted partial sums per (token, owner), summed at the source ----
    g = torch.Generator().manual_seed(9)
    y_sorted = [torch.randn(R.P, L, generator=g).to(BF) for _ in range(G)]
    y_dev = [y.to(R.dev) for y in y_sorted]
    p_ret, p_dw = _ptrs(R.ret_y, R.dev), _ptrs(R.dw, R.dev)
    for r in range(G):
        t = R.tab[r]
        _cabi.call("lmoe_epd_reduce_return", y_dev[r].data_ptr(), R.meta[r].data_ptr(), R.mask[r].data_ptr(),
                   R.slots[r].data_ptr(), None, t["src_off"].data_ptr(), R.counts_all.data_ptr(), G, E, r, K, L, R.stride,
                   R.P, p_ret.data_ptr(), None, R.st)
    torch.cuda.synchronize()
    for s in range(G):
        out = torch.zeros(tokens[s], L, dtype=BF, device=R.dev)
        _cabi.call("lmoe_epd_sum", R.ret_y[s].data_ptr(), R.tab[s]["sel"].data_ptr(), tokens[s], K, E, G, L, R.stride,
                   out.data_ptr(), L, R.st)
        torch.cuda.synchronize()
        exp = torch.zeros(tokens[s], L)
        for r in range(G):                                          # owners ascending, slots ascending inside an owner
            m = R.cpu_tables[s][r]
            part = torch.zeros(tokens[s], L)
            for k in range(K):
                rows = m["slots"][:, k]
                on = rows >= 0
                part[on] += R.w[s][on, k, None] * y_sorted[r].float()[rows[on]]
            exp += part.to(BF).float() * (m["mask"] != 0)[:, None]
        err = (out.float().cpu() - exp.to(BF).float()).abs().max().item()
        assert err <= 2.0 ** -7 * exp.abs().max().item(), err                     # one bf16 ulp (fma vs mul+add)
    # ---- backward send + owner-side adjoint of the combine ----
    R.send(with_meta=False)
    d_x_sorted = [torch.randn(R.P, L, generator=g).to(BF) for _ in range(G)]
    p_ret_dx = _ptrs(R.ret_dx, R.dev)
    d_w_rows = []
    for r in range(G):
        used = int(R.tab[r]["n_tiles"].item()) * 128
        dy_in, d_w_row = R.gather(r, y_sorted=y_dev[r])
        exp_rows, exp_w, filled, _ = R.expected_layout(r, R.d_routed)
        exp_dy = (exp_w[:, None] * exp_rows).to(BF).float()
        assert (dy_in[:used].float().cpu() - exp_dy[:used]).abs().max().item() <= 2.0 ** -8 * exp_dy.abs().max().item()
        exp_dw = (exp_rows * y_sorted[r].float()).sum(-1) * filled
        torch.testing.assert_close(d_w_row[:used].cpu(), exp_dw[:used], rtol=1e-4, atol=1e-4)
        d_w_rows.append(d_w_row)
        t = R.tab[r]
        dxs = d_x_sorted[r].to(R.dev)
        _cabi.call("lmoe_epd_reduce_return", dxs.data_ptr(), R.meta[r].data_ptr(), R.mask[r].data_ptr(),
                   R.slots[r].data_ptr(), d_w_row.data_ptr(), t["src_off"].data_ptr(), R.counts_all.data_ptr(), G, E, r, K, L,
                   R.stride, R.P, p_ret_dx.data_ptr(), p_dw.data_ptr(), R.st)
    torch.cuda.synchronize()
    for s in range(G):
        out = torch.zeros(tokens[s], L, dtype=BF, device=R.dev)
        _cabi.call("lmoe_epd_sum", R.ret_dx[s].data_ptr(), R.tab[s]["sel"].data_ptr(), tokens[s], K, E, G, L, R.stride,
                   out.data_ptr(), L, R.st)
        torch.cuda.synchronize()
        exp = torch.zeros(tokens[s], L)
        exp_dw = torch.zeros(tokens[s], K)
        for r in range(G):
            m = R.cpu_tables[s][r]
            part = torch.zeros(tokens[s], L)
            for k in range(K):
                rows = m["slots"][:, k]
                on = rows >= 0
                part[on] += d_x_sorted[r].float()[rows[on]]
                exp_dw[on, k] = d_w_rows[r].cpu()[rows[on]]
            exp += part.to(BF).float() * (m["mask"] != 0)[:, None]
        err = (out.float().cpu() - exp.to(BF).float()).abs().max().item()
        assert err <= 2.0 ** -7 * exp.abs().max().item(), err
        assert torch.equal(R.dw[s][:tokens[s] * K].view(tokens[s], K).cpu(), exp_dw)   # gating gradients are copies
    assert R.status.item() == 0


def test_shard_overflow_raises_status_201_and_drops_rows_without_faulting():
    """A shard that receives more rows than its static capacity: the tables kernel and the send kernel both raise
    device status 201, every access stays inside the buffers (excess rows are dropped by bounds checks), and the host
    side turns the status into an exception."""
    from swamla_b200 import _cabi, status as status_monitor
    G, E, K, L = 2, 16, 8, 128
    tokens = (600, 500)                                     # ~550 rows per expert -> 5120 padded rows per shard
    R = _Ranks(G, E, K, L, tokens, seed=5, capacity_factor=0.3)
    assert R.P < 5120                                       # capacity 2560 rows: the layout cannot fit
    assert R.status.item() == 201                           # raised by lmoe_ep_tables already
    R.status.zero_()
    R.send(with_meta=True, expect_status=201)               # ... and by the send kernel for the rows it drops
    for r in range(G):
        used = int(R.tab[r]["n_tiles"].item()) * 128
        assert used <= R.P
        x_in, _ = R.gather(r)                               # bounded by the capacity; rows that fit are exact copies
        meta = R.meta[r].cpu()
        slot = (meta & 0xffffffff).to(torch.int32).long()
        ok = (slot >= 0)[:used]
        assert ok.any()
        stage = R.stage_x[r].float().cpu()
        assert torch.equal(x_in[:used].float().cpu()[ok], stage[slot[:used][ok]])
    assert "more rows than its buffers hold" in _cabi.status_string(201)
    status_monitor.post(R.status, "overflow test")
    with pytest.raises(_cabi.LmoeError, match="201"):
        status_monitor.poll(block=True)
    assert status_monitor.pending() == 0


@pytest.mark.gpu
def test_flag_barrier_passes_when_every_peer_has_arrived_and_reports_a_missing_one():
    """``lmoe_ep_flag_barrier`` with two ranks whose flag words live on this one GPU.  Only rank 0's kernel ever runs (two
    kernels that wait for each other must not be separate launches on one GPU): first with rank 1's arrival written
    by hand, which must pass at once and leave rank 0's own arrival in rank 1's word; then with an epoch nobody
    announces, where the bounded wait must give up with status 202 and leave the context usable."""
    import time
    from swamla_b200 import _cabi
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    flags = [torch.zeros(32, dtype=torch.int32, device=dev) for _ in range(2)]
    peers = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)      # rank 0's barrier counter
    flags[0][1] = 1                                            # "rank 1 has reached barrier 1"
    _cabi.call("lmoe_ep_flag_barrier", peers.data_ptr(), epoch.data_ptr(), 0, 2, status.data_ptr(), st)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert flags[1][0].item() == 1 and flags[0][0].item() == 1  # rank 0 told rank 1 and itself
    t0 = time.time()
    _cabi.call("lmoe_ep_flag_barrier", peers.data_ptr(), epoch.data_ptr(), 0, 2, status.data_ptr(), st)   # rank 1 never arrives
    torch.cuda.synchronize()
    assert status.item() == 202
    assert time.time() - t0 < 10.0
    assert flags[1][0].item() == 2 and epoch.item() == 2
    # the context is intact: an ordinary kernel still runs
    assert torch.ones(8, device=dev).sum().item() == 8.0
