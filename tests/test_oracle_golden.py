"""The CPU oracle against the frozen outputs of the reference module (CPU only)."""
import pytest
import torch

from oracle import inputs, latent_moe_ref as R, ref_shim
from conftest import golden_path


def _check_digest(t: torch.Tensor, d: dict, rtol=1e-5, atol=1e-6):
    assert tuple(t.shape) == tuple(d["shape"])
    flat = t.detach().reshape(-1).float()
    torch.testing.assert_close(flat[::d["step"]], d["sample"], rtol=rtol, atol=atol)
    assert abs(flat.double().pow(2).sum().sqrt().item() - d["l2"]) <= rtol * max(d["l2"], 1e-12) + atol


@pytest.mark.parametrize("name", ["tiny", "tiny_ragged", "tiny_shared2", "cfg1", "tiny_moe", "tiny_moe_ragged"])
def test_oracle_matches_reference_fixture(name):
    fx = torch.load(golden_path(name), weights_only=False)
    w = inputs.WORKLOADS[name]
    params, buffers, x, dy = inputs.make_inputs(w, seed=fx["seed"])
    # seeded inputs reproduce bit-for-bit
    for k, d in fx["inputs"].items():
        _check_digest(x if k == "x" else params[k], d, rtol=0, atol=0)
    if "grads" in fx:
        out, grads = R.layer_forward_backward(params, buffers, x, dy, w.K, aux_grad=fx["aux_grad"])
    else:
        with torch.no_grad():
            out = R.layer_forward(params, buffers, x, w.K)
        grads = None
    # integer results: bit-exact
    assert torch.equal(out["sel"].to(torch.int16), fx["sel"])
    assert torch.equal(out["counts"].to(torch.int32), fx["counts"])
    assert torch.equal(out["offsets"].to(torch.int32), fx["offsets"])
    assert torch.equal(out["perm"].to(torch.int32), fx["perm"])
    # float results
    assert abs(out["aux_loss"].item() - fx["aux_loss"]) <= 1e-6 * abs(fx["aux_loss"])
    _check_digest(out["y"], fx["y"])
    if grads is not None:
        for k, d in fx["grads"].items():
            _check_digest(grads[k], d)
    # bias update after backward
    R.update_bias(out["sel"], w.T, buffers, w.K)
    torch.testing.assert_close(buffers["router.expert_bias"], fx["expert_bias_after_update"])
    torch.testing.assert_close(buffers["router.load_history"], fx["load_history_after_update"])


def test_canonical_topk_is_lower_index_first_on_ties():
    s = torch.tensor([[0.5, 0.9, 0.9, 0.1, 0.9, 0.5]])
    assert R.canonical_topk(s, 4).tolist() == [[1, 2, 4, 0]]


def test_canonical_topk_agrees_with_torch_topk_without_ties():
    g = torch.Generator().manual_seed(1)
    s = torch.rand(512, 128, generator=g)
    assert torch.equal(R.canonical_topk(s, 12), torch.topk(s, 12, dim=-1).indices)


def test_route_permute_is_stable_and_grouped():
    g = torch.Generator().manual_seed(2)
    sel = torch.stack([torch.randperm(16, generator=g)[:4] for _ in range(100)])
    counts, offsets, perm = R.route_permute(sel, 16)
    flat = sel.reshape(-1)
    assert counts.sum().item() == flat.numel() and offsets[-1].item() == flat.numel()
    sorted_e = flat[perm]
    assert torch.all(sorted_e[1:] >= sorted_e[:-1])
    for e in range(16):
        seg = perm[offsets[e]:offsets[e + 1]]
        assert torch.all(seg[1:] > seg[:-1])           # ascending flat index inside an expert
        assert torch.all(flat[seg] == e)


def test_grouped_gemm_matches_dense_masked_einsum():
    g = torch.Generator().manual_seed(3)
    E, Kd, N = 5, 8, 6
    counts = torch.tensor([3, 0, 7, 1, 4])
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)])
    a = torch.randn(int(counts.sum()), Kd, generator=g)
    b = torch.randn(E, Kd, N, generator=g)
    eid = torch.repeat_interleave(torch.arange(E), counts)
    ref = torch.einsum("tk,tkn->tn", a, b[eid])
    torch.testing.assert_close(R.grouped_gemm(a, b, offsets), ref)


@pytest.mark.skipif(not ref_shim.available(), reason="reference source tree not present")
@pytest.mark.parametrize("name", ["tiny", "tiny_moe"])
def test_oracle_matches_live_reference_module(name):
    w = inputs.WORKLOADS[name]
    params, buffers, x, dy = inputs.make_inputs(w, seed=7)
    ro, rg, _ = ref_shim.run_reference(w, params, buffers, x, dy, aux_grad=0.5)
    o, g = R.layer_forward_backward(params, buffers, x, dy, w.K, aux_grad=0.5)
    assert torch.equal(o["sel"], ro["sel"])
    torch.testing.assert_close(o["y"], ro["y"])
    for k in rg:
        torch.testing.assert_close(g[k], rg[k])
