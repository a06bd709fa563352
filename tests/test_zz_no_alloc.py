"""lmoe_route_permute_static: the routing tables without any caller-provided scratch.

Some hosts cannot give this library device memory when they call it: a plugin interface that passes
input and output buffers only, or a process whose allocator already owns the whole GPU.  For them the
library keeps the scratch of the routing kernels in a fixed 4 MiB array inside its own image.  This
file checks, through the C ABI, that the entry point returns exactly what lmoe_route_permute returns
-- twice in a row with different inputs, because the array is shared and keeps the previous call's
contents -- and that a problem beyond the fixed capacity is refused before anything is launched.

The file name sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tables(shape, device):
    from swamla_b200 import _cabi
    T, K, E = shape.T, shape.K, shape.E
    P = _cabi.load().lmoe_padded_rows(shape)
    i32 = dict(dtype=torch.int32, device=device)
    bufs = dict(counts=torch.full((E,), -3, **i32), offsets=torch.full((E + 1,), -3, **i32),
                perm=torch.full((T * K,), -3, **i32), pad_offsets=torch.full((E + 1,), -3, **i32),
                pos=torch.full((T * K,), -3, **i32), row_src=torch.full((P,), -3, **i32),
                tile_expert=torch.full((P // 128,), -3, **i32), n_tiles=torch.full((1,), -3, **i32))
    return bufs, _cabi.Route(**{k: v.data_ptr() for k, v in bufs.items()})


def _random_selection(T, E, K, seed, device):
    g = torch.Generator().manual_seed(seed)
    scores = torch.rand(T, E, generator=g)
    return scores.topk(K, dim=1).indices.to(torch.int32).to(device).contiguous()


@pytest.mark.parametrize("T,E,K", [(1024, 128, 12), (777, 32, 8)])
def test_static_scratch_variant_matches_workspace_variant_twice(T, E, K):
    from swamla_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda:0")
    shape = _cabi.Shape(T=T, D=1024, L=256, E=E, K=K, F=256, Fs=1024, n_shared=1)
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(max(16, lib.lmoe_route_workspace_bytes(shape)), dtype=torch.uint8, device=dev)
    for call, seed in enumerate((11, 12)):           # two calls in a row, different routing each time
        sel = _random_selection(T, E, K, seed, dev)
        want, want_struct = _tables(shape, dev)
        _cabi.call("lmoe_route_permute", shape, sel.data_ptr(), want_struct, ws.data_ptr(), ws.numel(), stream)
        got, got_struct = _tables(shape, dev)
        _cabi.call("lmoe_route_permute_static", shape, sel.data_ptr(), got_struct, stream)
        torch.cuda.synchronize()
        used = int(want["n_tiles"].item()) * 128
        for name in ("counts", "offsets", "perm", "pad_offsets", "pos", "n_tiles"):
            assert torch.equal(got[name], want[name]), f"call {call}: {name} differs"
        # rows and tiles beyond the part in use are not written by either entry point
        assert torch.equal(got["row_src"][:used], want["row_src"][:used]), f"call {call}: row_src differs"
        assert torch.equal(got["tile_expert"][:used // 128], want["tile_expert"][:used // 128])


def test_static_scratch_variant_refuses_problems_beyond_its_capacity():
    from swamla_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda:0")
    # ceil(T*K/256) * E * 4 bytes > 4 MiB: 2**20 tokens x top-32 over 256 experts
    big = _cabi.Shape(T=1 << 20, D=1024, L=256, E=256, K=32, F=256, Fs=1024, n_shared=1)
    assert lib.lmoe_route_workspace_bytes(big) > (4 << 20)
    dummy = torch.zeros(64, dtype=torch.int32, device=dev)
    route = _cabi.Route(**{k: dummy.data_ptr() for k in ("counts", "offsets", "perm", "pad_offsets", "pos", "row_src",
                                                          "tile_expert", "n_tiles")})
    before = lib.lmoe_launch_count()
    rc = lib.lmoe_route_permute_static(big, dummy.data_ptr(), route, torch.cuda.current_stream().cuda_stream)
    assert rc == -6 and "capacity" in _cabi.status_string(rc)
    assert lib.lmoe_launch_count() == before          # refused on the host, nothing was launched
