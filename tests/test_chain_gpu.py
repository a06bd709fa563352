"""The chained routed-expert kernel (gate_up -> SwiGLU -> down in one launch, and its backward counterpart) through
the C ABI, against the separate grouped GEMMs (+ streaming SwiGLU adjoint) it replaces and against fp32 torch."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _layout(counts, capacity_tiles, dev):
    """Padded expert layout for the given rows per expert: (P, pad_offsets, tile_expert, n_tiles, valid-row mask)."""
    tiles = [(c + 127) // 128 for c in counts]
    n_tiles = sum(tiles)
    assert n_tiles <= capacity_tiles
    P = capacity_tiles * 128
    tile_expert = torch.zeros(capacity_tiles, dtype=torch.int32)
    valid = torch.zeros(P, dtype=torch.bool)
    row_expert = torch.full((P,), -1, dtype=torch.long)
    t0 = 0
    for e, (c, nt) in enumerate(zip(counts, tiles)):
        tile_expert[t0:t0 + nt] = e
        valid[t0 * 128:t0 * 128 + c] = True
        row_expert[t0 * 128:(t0 + nt) * 128] = e
        t0 += nt
    pad_offsets = torch.tensor([0] + [128 * sum(tiles[:e + 1]) for e in range(len(counts))], dtype=torch.int32, device=dev)
    return (P, tile_expert.to(dev), torch.tensor([n_tiles], dtype=torch.int32, device=dev), pad_offsets, valid, row_expert,
            n_tiles)


CASES = [
    # E, L, F, rows per expert, capacity in tiles
    (4, 64, 64, [100, 0, 129, 5], 6),
    (3, 128, 192, [300, 17, 128], 8),
    (5, 192, 128, [1, 255, 0, 130, 64], 8),
    (8, 256, 256, [200, 0, 513, 90, 128, 7, 260, 1], 20),
    (6, 256, 768, [140, 260, 3, 0, 129, 400], 14),
    (16, 256, 256, [2500 + 37 * i for i in range(16)], 16 * 23),      # ~350 tiles: several tiles per SM
]


@pytest.mark.parametrize("E,L,F,counts,cap", CASES)
def test_chain_forward_and_backward_match_the_separate_kernels(E, L, F, counts, cap):
    from swamla_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    prev = lib.lmoe_chain_enable(1)
    assert lib.lmoe_chain_applies(L, F) == 1
    lib.lmoe_chain_enable(prev)
    P, tile_expert, n_tiles, pad_offsets, valid, row_expert, nt = _layout(counts, cap, dev)
    used = nt * 128
    g = torch.Generator().manual_seed(E * 1000 + L + F)
    x = torch.randn(P, L, generator=g)
    dy = torch.randn(P, L, generator=g)
    x[~valid] = 0
    dy[~valid] = 0
    wgu = (torch.randn(E, L, 2 * F, generator=g) * 0.05).to(BF).to(dev)
    wd = (torch.randn(E, F, L, generator=g) * 0.05).to(BF).to(dev)
    x, dy = x.to(BF).to(dev), dy.to(BF).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def run(chain, pairs=True, fused_adjoint=False):
        # pairs: the pad_offsets table lets the launcher put two tiles of an expert on a CTA pair (L a multiple of 128)
        po = pad_offsets.data_ptr() if pairs else None
        prev = lib.lmoe_chain_enable(1 if chain else 0)
        try:
            o = dict(h1=torch.full((P, 2 * F), 3.0, dtype=BF, device=dev), hidden=torch.full((P, F), 3.0, dtype=BF, device=dev),
                     y=torch.full((P, L), 3.0, dtype=BF, device=dev), d_h1=torch.full((P, 2 * F), 3.0, dtype=BF, device=dev),
                     d_x=torch.full((P, L), 3.0, dtype=BF, device=dev))
            # no d_hidden scratch: the SwiGLU adjoint runs in the epilogue of the d_hidden GEMM (gate / up staged by TMA)
            d_hidden = None if (chain or fused_adjoint) else torch.empty(P, F, dtype=BF, device=dev)
            _cabi.call("lmoe_grouped_fwd", P, E, L, F, x.data_ptr(), wgu.data_ptr(), wd.data_ptr(), tile_expert.data_ptr(),
                       n_tiles.data_ptr(), po, o["h1"].data_ptr(), o["hidden"].data_ptr(), o["y"].data_ptr(), status.data_ptr(), st)
            _cabi.call("lmoe_grouped_bwd_dgrad", P, E, L, F, dy.data_ptr(), o["h1"].data_ptr(), wgu.data_ptr(), wd.data_ptr(),
                       tile_expert.data_ptr(), n_tiles.data_ptr(), po, _cabi.ptr(d_hidden), o["d_h1"].data_ptr(),
                       o["d_x"].data_ptr(), status.data_ptr(), st)
            torch.cuda.synchronize()
            assert status.item() == 0
            return o
        finally:
            lib.lmoe_chain_enable(prev)

    a, b, single, fused = run(True), run(False), run(True, pairs=False), run(False, fused_adjoint=True)
    # with the per-expert offsets the separate grouped GEMMs run on CTA pairs too (gemm_pair.cuh, grouped form); without
    # them, one CTA per tile: the same products summed in the same order
    # (the grouped form of the pair kernel is opt-in, LMOE_PAIR_GROUPED=1, read once per process: without it both runs
    #  use one CTA per tile and the comparison is trivially true)
    plain = run(False, pairs=False)
    for k in b:
        assert torch.equal(b[k][:used], plain[k][:used]), k
    for k in ("d_h1", "d_x"):      # the same arithmetic on the same d_hidden, then the very same second GEMM: at most a
        ta, tb = fused[k][:used].float(), b[k][:used].float()          # last-bit difference where the compiler fuses
        assert ((ta - tb).norm() / tb.norm().clamp_min(1e-30)).item() <= 1e-3, k   # multiplies and adds differently
        assert ((ta - tb).abs() <= 2.0 ** -7 * (tb.abs() + tb.pow(2).mean().sqrt())).all(), k
    for k, t in fused.items():
        assert (t[used:].float() == 3.0).all(), k
    for k in ("h1", "hidden", "y"):                      # same MMAs in the same order: identical bits
        assert torch.equal(a[k][:used], b[k][:used]), k
    for k in a:                                          # one CTA per tile or CTA pairs: the same arithmetic
        assert torch.equal(a[k], single[k]), k
    for k in ("d_h1", "d_x"):                            # d_x sums its 2F products in another order
        ta, tb = a[k][:used].float(), b[k][:used].float()
        rel = ((ta - tb).norm() / tb.norm().clamp_min(1e-30)).item()
        assert rel <= 2e-3, (k, rel)
        bound = 2.0 ** -7 * (tb.abs() + tb.pow(2).mean().sqrt())
        assert ((ta - tb).abs() <= 2 * bound).all(), k
    for k, t in a.items():                               # nothing beyond the tiles in use; pad rows stay zero
        assert (t[used:].float() == 3.0).all(), k
        assert t[:used][~valid[:used].to(dev)].float().abs().max().item() == 0 if (~valid[:used]).any() else True, k

    # fp32 torch on the same bf16 inputs (the expert of each valid row), bf16 tolerance
    re = row_expert.to(dev)
    rows = valid.to(dev).nonzero().flatten()
    if rows.numel() > 2048:                              # a sample keeps the per-row weight gather small
        rows = rows[torch.randperm(rows.numel(), generator=g)[:2048].to(dev)]
    xe, dye, ee = x[rows].float(), dy[rows].float(), re[rows]
    h1 = torch.einsum("rl,rlf->rf", xe, wgu.float()[ee])
    gate, up = h1.chunk(2, -1)
    hidden = torch.nn.functional.silu(gate) * up
    y = torch.einsum("rf,rfl->rl", hidden, wd.float()[ee])
    for k, ref in (("h1", h1), ("hidden", hidden), ("y", y)):
        rel = ((a[k][rows].float() - ref).norm() / ref.norm()).item()
        assert rel < 1e-2, (k, rel)
    gb, ub = a["h1"][rows].float().chunk(2, -1)          # the adjoint uses the saved (bf16) gate / up
    d_hidden = torch.einsum("rl,rfl->rf", dye, wd.float()[ee]).to(BF).float()
    sg = torch.sigmoid(gb)
    d_h1 = torch.cat([d_hidden * ub * sg * (1 + gb * (1 - sg)), d_hidden * gb * sg], -1)
    d_x = torch.einsum("rf,rlf->rl", d_h1.to(BF).float(), wgu.float()[ee])
    for k, ref in (("d_h1", d_h1), ("d_x", d_x)):
        rel = ((a[k][rows].float() - ref).norm() / ref.norm()).item()
        assert rel < 1e-2, (k, rel)
