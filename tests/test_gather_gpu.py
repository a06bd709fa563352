"""Routed expert GEMMs with the A operand gathered by the TMA unit (lmoe_grouped_fwd_gather,
lmoe_grouped_bwd_wgrad_gather) against the same GEMMs on a materialised x_sorted: bit for bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(T, E, K, L, F, seed, skew=False):
    from swamla_b200 import _cabi
    from swamla_b200.functional import RouteTables, make_shape
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(seed)
    scores = torch.rand(T, E, generator=g)
    if skew:                                   # a few hot experts, some empty ones
        scores[:, : E // 4] += 0.5
        scores[:, E // 2:: 3] -= 2.0
    sel = scores.topk(K, dim=1).indices.to(torch.int32).to(dev)
    shape = make_shape(T, 8 * L, L, E, K, F, 8)
    lib = _cabi.load()
    route = RouteTables(shape, dev)
    st = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(max(16, lib.lmoe_route_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
    _cabi.call("lmoe_route_permute", shape, sel.data_ptr(), route.struct, ws.data_ptr(), ws.numel(), st)
    x_ext = torch.randn(T + 1, L, generator=g).to(dev).to(torch.bfloat16)
    x_ext[T].zero_()
    P = route.padded_rows
    x_sorted = torch.empty(P, L, dtype=torch.bfloat16, device=dev)
    _cabi.call("lmoe_gather_rows", x_ext.data_ptr(), route.row_src.data_ptr(), K, P, L, route.n_tiles.data_ptr(),
               x_sorted.data_ptr(), st)
    return dev, g, shape, route, x_ext, x_sorted, P, st


@pytest.mark.parametrize("T,E,K,L,F,skew", [(300, 16, 4, 128, 64, False), (1000, 32, 6, 256, 128, True),
                                            (4096, 128, 12, 256, 256, False)])
def test_gathered_gate_up_forward_equals_materialised(T, E, K, L, F, skew):
    from swamla_b200 import _cabi
    dev, g, shape, route, x_ext, x_sorted, P, st = _setup(T, E, K, L, F, seed=T + E, skew=skew)
    bf = dict(dtype=torch.bfloat16, device=dev)
    wgu = (torch.randn(E, L, 2 * F, generator=g) * 0.05).to(**bf)
    wde = (torch.randn(E, F, L, generator=g) * 0.05).to(**bf)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    outs = []
    for gathered in (False, True):
        h1, hidden, y = (torch.zeros(P, 2 * F, **bf), torch.zeros(P, F, **bf), torch.zeros(P, L, **bf))
        tail = (wgu.data_ptr(), wde.data_ptr(), route.tile_expert.data_ptr(), route.n_tiles.data_ptr(), h1.data_ptr(),
                hidden.data_ptr(), y.data_ptr(), status.data_ptr(), st)
        if gathered:
            _cabi.call("lmoe_grouped_fwd_gather", P, E, L, F, x_ext.data_ptr(), T + 1, route.row_src.data_ptr(), 1, K, T,
                       *tail)
        else:
            _cabi.call("lmoe_grouped_fwd", P, E, L, F, x_sorted.data_ptr(), *tail[:4], route.pad_offsets.data_ptr(), *tail[4:])
        outs.append((h1, hidden, y))
    torch.cuda.synchronize()
    assert status.item() == 0
    used = int(route.n_tiles.item()) * 128
    for a, b, name in zip(outs[0], outs[1], ("h1", "hidden", "y_sorted")):
        assert a[:used].float().abs().sum().item() > 0, name
        assert torch.equal(a[:used], b[:used]), name


@pytest.mark.parametrize("T,E,K,L,F,skew", [(300, 16, 4, 128, 64, False), (1000, 32, 6, 256, 128, True),
                                            (4096, 128, 12, 256, 256, False)])
def test_gathered_gate_up_weight_gradient_equals_materialised(T, E, K, L, F, skew):
    from swamla_b200 import _cabi
    dev, g, shape, route, x_ext, x_sorted, P, st = _setup(T, E, K, L, F, seed=7 * T + E, skew=skew)
    bf = dict(dtype=torch.bfloat16, device=dev)
    used = int(route.n_tiles.item()) * 128
    valid = (route.row_src[:used] >= 0).to(torch.bfloat16)[:, None]

    def rows(width):                              # pad rows zero, as the layer's kernels leave them
        t = torch.zeros(P, width, **bf)
        t[:used] = torch.randn(used, width, generator=g).to(**bf) * valid
        return t

    d_h1, hidden, d_y = rows(2 * F), rows(F), rows(L)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    outs = []
    for gathered in (False, True):
        dwgu, dwd = torch.zeros(E, L, 2 * F, **bf), torch.zeros(E, F, L, **bf)
        tail = (d_h1.data_ptr(), hidden.data_ptr(), d_y.data_ptr(), route.pad_offsets.data_ptr(), dwgu.data_ptr(),
                dwd.data_ptr(), status.data_ptr(), st)
        if gathered:
            _cabi.call("lmoe_grouped_bwd_wgrad_gather", P, E, L, F, x_ext.data_ptr(), T + 1, route.row_src.data_ptr(), 1, K,
                       T, *tail)
        else:
            _cabi.call("lmoe_grouped_bwd_wgrad", P, E, L, F, x_sorted.data_ptr(), *tail)
        outs.append((dwgu, dwd))
    torch.cuda.synchronize()
    assert status.item() == 0
    assert outs[0][0].float().abs().sum().item() > 0
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])


def test_gather_arguments_are_checked():
    from swamla_b200 import _cabi
    ERR_ARG = -1                                   # LMOE_ERR_ARG
    dev, g, shape, route, x_ext, x_sorted, P, st = _setup(256, 16, 2, 128, 64, seed=3)
    lib = _cabi.load()
    bf = dict(dtype=torch.bfloat16, device=dev)
    w1, w2 = torch.zeros(16, 128, 128, **bf), torch.zeros(16, 64, 128, **bf)
    h1, hid, y = torch.zeros(P, 128, **bf), torch.zeros(P, 64, **bf), torch.zeros(P, 128, **bf)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def call(n_src, stride, div, zero_row, index=route.row_src.data_ptr()):
        return lib.lmoe_grouped_fwd_gather(P, 16, 128, 64, x_ext.data_ptr(), n_src, index, stride, div, zero_row,
                                           w1.data_ptr(), w2.data_ptr(), route.tile_expert.data_ptr(),
                                           route.n_tiles.data_ptr(), h1.data_ptr(), hid.data_ptr(), y.data_ptr(),
                                           status.data_ptr(), st)

    assert call(257, 1, 2, 256) == 0
    assert call(257, 1, 2, 257) == ERR_ARG      # the zero row must exist
    assert call(257, 0, 2, 256) == ERR_ARG
    assert call(257, 1, 0, 256) == ERR_ARG
    assert call(0, 1, 2, 0) == ERR_ARG
    assert call(257, 1, 2, 256, index=None) == ERR_ARG
    torch.cuda.synchronize()
