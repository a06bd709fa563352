"""Router kernels through the C ABI against the CPU oracle: indices and permutation bit-exact."""
import pytest
import torch

from oracle import latent_moe_ref as R

pytestmark = pytest.mark.gpu


def _shape(T, E, K):
    from swamla_b200 import _cabi
    return _cabi.Shape(T=T, D=1024, L=256, E=E, K=K, F=256, Fs=1024, n_shared=1)


def run_topk(logits, bias, K, z_coef=0.001):
    from swamla_b200 import _cabi
    dev = torch.device("cuda:0")
    T, E = logits.shape
    s = _shape(T, E, K)
    lg, bs = logits.to(dev), bias.to(dev)
    sel = torch.empty(T, K, dtype=torch.int32, device=dev)
    w = torch.empty(T, K, dtype=torch.float32, device=dev)
    lse = torch.empty(T, dtype=torch.float32, device=dev)
    zp = torch.empty((T + 7) // 8, dtype=torch.float32, device=dev)
    z = torch.empty(1, dtype=torch.float32, device=dev)
    _cabi.call("lmoe_gate_topk_fwd", s, lg.data_ptr(), bs.data_ptr(), z_coef, sel.data_ptr(), w.data_ptr(),
               lse.data_ptr(), zp.data_ptr(), z.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return sel.cpu(), w.cpu(), lse.cpu(), z.cpu()


def run_route(sel, E):
    from swamla_b200 import _cabi
    dev = torch.device("cuda:0")
    T, K = sel.shape
    s = _shape(T, E, K)
    lib = _cabi.load()
    P = lib.lmoe_padded_rows(s)
    i32 = dict(dtype=torch.int32, device=dev)
    bufs = dict(counts=torch.empty(E, **i32), offsets=torch.empty(E + 1, **i32), perm=torch.empty(T * K, **i32),
                pad_offsets=torch.empty(E + 1, **i32), pos=torch.empty(T * K, **i32),
                row_src=torch.full((P,), -7, **i32), tile_expert=torch.full((P // 128,), -7, **i32),
                n_tiles=torch.empty(1, **i32))
    r = _cabi.Route(**{k: v.data_ptr() for k, v in bufs.items()})
    ws = torch.empty(lib.lmoe_route_workspace_bytes(s), dtype=torch.uint8, device=dev)
    _cabi.call("lmoe_route_permute", s, sel.to(dev).to(torch.int32).data_ptr(), r, ws.data_ptr(), ws.numel(),
               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return {k: v.cpu() for k, v in bufs.items()}


def near_tie_rows(scores, sel_a, sel_b):
    """Rows whose index mismatch is explained by two candidates within 2 ulp of each other."""
    bad = (sel_a != sel_b).any(dim=1).nonzero().flatten().tolist()
    unexplained = []
    for t in bad:
        a = set(sel_a[t].tolist()) ^ set(sel_b[t].tolist())
        vals = scores[t, sorted(a)] if a else scores[t, sel_a[t]]
        spread = (vals.max() - vals.min()).item()
        if spread > 2 * torch.finfo(torch.float32).eps * vals.abs().max().item():
            unexplained.append(t)
    return bad, unexplained


@pytest.mark.parametrize("T,E,K", [(1024, 128, 12), (131, 32, 8), (1, 16, 4), (4096, 256, 16), (777, 8, 8),
                                   (65, 256, 32), (200, 64, 32), (33, 32, 32), (500, 48, 7)])   # top-k and expert limits
def test_topk_matches_oracle(T, E, K):
    g = torch.Generator().manual_seed(T + E)
    logits = torch.randn(T, E, generator=g) * 0.7
    bias = torch.randn(E, generator=g) * 0.05 if T != 1024 else torch.zeros(E)
    _, sel_ref, w_ref, z_ref = R.router_forward(None, None, bias, K, 0.001, logits=logits)
    sel, w, lse, z = run_topk(logits, bias, K)
    scores = torch.sigmoid(logits) + bias
    bad, unexplained = near_tie_rows(scores, sel_ref, sel.long())
    assert not unexplained, f"{len(unexplained)} rows differ beyond a 2-ulp near-tie"
    assert len(bad) <= max(1, T // 1000)
    good = torch.ones(T, dtype=torch.bool)
    good[bad] = False
    torch.testing.assert_close(w[good], w_ref[good], rtol=2e-6, atol=1e-7)
    torch.testing.assert_close(lse, torch.logsumexp(logits, -1), rtol=2e-6, atol=2e-6)
    torch.testing.assert_close(z[0], z_ref, rtol=1e-5, atol=1e-9)


def test_topk_tie_rule_lower_index_first():
    logits = torch.zeros(64, 32)                      # all scores equal
    sel, w, _, _ = run_topk(logits, torch.zeros(32), 5)
    assert torch.equal(sel, torch.arange(5, dtype=torch.int32).repeat(64, 1))
    torch.testing.assert_close(w, torch.full((64, 5), 0.2))
    bias = torch.zeros(32)
    bias[7] = 0.25                                    # bias steers selection, not the weights
    sel, w, _, _ = run_topk(logits, bias, 3)
    assert sel[0].tolist() == [7, 0, 1]
    torch.testing.assert_close(w[0], torch.full((3,), 1 / 3))
    # ties inside one lane's block of experts and across lanes (256 experts: 8 per lane)
    logits = torch.zeros(9, 256)
    logits[:, [13, 14, 200, 8]] = 1.0
    sel, _, _, _ = run_topk(logits, torch.zeros(256), 6)
    assert sel[3].tolist() == [8, 13, 14, 200, 0, 1]


@pytest.mark.parametrize("T,E,K", [(1024, 128, 12), (131, 32, 8), (1, 16, 4), (5000, 256, 16), (3, 8, 8), (700, 256, 32)])
def test_route_permute_matches_oracle_bit_exact(T, E, K):
    g = torch.Generator().manual_seed(T * 3 + K)
    sel = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    counts, offsets, perm = R.route_permute(sel, E)
    out = run_route(sel, E)
    assert torch.equal(out["counts"].long(), counts)
    assert torch.equal(out["offsets"].long(), offsets)
    assert torch.equal(out["perm"].long(), perm)
    # padded layout is derived from the canonical one
    padded = (counts + 127) // 128 * 128
    poff = torch.cat([torch.zeros(1, dtype=torch.long), padded.cumsum(0)])
    assert torch.equal(out["pad_offsets"].long(), poff)
    assert out["n_tiles"].item() == poff[-1].item() // 128
    flat = sel.reshape(-1)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel())
    expect_pos = poff[flat] + (inv - offsets[flat])
    assert torch.equal(out["pos"].long(), expect_pos)
    used = poff[-1].item()
    row_src = out["row_src"][:used].long()
    expect_src = torch.full((used,), -1, dtype=torch.long)
    expect_src[expect_pos] = torch.arange(flat.numel())
    assert torch.equal(row_src, expect_src)
    te = out["tile_expert"][: used // 128].long()
    assert torch.equal(te, torch.repeat_interleave(torch.arange(E), padded // 128))


def test_route_permute_all_tokens_to_one_expert_and_empty_experts():
    T, E, K = 700, 16, 1
    sel = torch.full((T, K), 5)
    out = run_route(sel, E)
    assert out["counts"].tolist() == [0] * 5 + [700] + [0] * 10
    assert out["n_tiles"].item() == 6
    assert torch.equal(out["perm"].long(), torch.arange(700))


def test_bias_update_matches_oracle():
    from swamla_b200 import _cabi
    dev = torch.device("cuda:0")
    T, E, K = 131, 32, 8
    g = torch.Generator().manual_seed(5)
    sel = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    buffers = {"router.expert_bias": torch.randn(E, generator=g) * 0.01, "router.load_history": torch.rand(E, generator=g),
               "router.update_count": torch.tensor(0)}
    bias, hist = buffers["router.expert_bias"].clone().to(dev), buffers["router.load_history"].clone().to(dev)
    R.update_bias(sel, T, buffers, K)
    counts = torch.bincount(sel.reshape(-1), minlength=E).to(torch.int32).to(dev)
    _cabi.call("lmoe_router_bias_update", _shape(T, E, K), counts.data_ptr(), 0.001, bias.data_ptr(), hist.data_ptr(),
               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    torch.testing.assert_close(bias.cpu(), buffers["router.expert_bias"], rtol=0, atol=0)
    torch.testing.assert_close(hist.cpu(), buffers["router.load_history"], rtol=1e-6, atol=1e-7)
