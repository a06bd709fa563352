"""Fused RMSNorm / residual kernels and the NormedResidualFFN block on the GPU against the CPU oracle and the fixture
generated from the reference's RMSNorm class."""
import pytest
import torch

from oracle import block_ref, inputs, latent_moe_ref as R
from conftest import golden_path

pytestmark = pytest.mark.gpu
RTOL_BF16 = 2e-2


def _close(name, test, ref, rtol=RTOL_BF16):
    ok, rep = R.within_tolerance(test.detach().float().cpu(), ref, rtol)
    assert ok, f"{name}: {rep}"


@pytest.mark.parametrize("T,D", [(37, 256), (1000, 1024), (515, 2048), (64, 8)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_rmsnorm_kernels_match_oracle(T, D, with_residual):
    from swamla_b200 import _cabi
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(T + D)
    rb = inputs.round_to_bf16
    x, w = rb(torch.randn(T, D, generator=g) * 1.7), 1.0 + 0.1 * torch.randn(D, generator=g)
    d_xn, d_res = rb(torch.randn(T, D, generator=g)), rb(torch.randn(T, D, generator=g))
    st = torch.cuda.current_stream().cuda_stream
    bf = dict(dtype=torch.bfloat16, device=dev)
    xd, wd = x.to(**bf), w.to(dev)
    xn, rstd = torch.empty(T, D, **bf), torch.empty(T, dtype=torch.float32, device=dev)
    _cabi.call("lmoe_rmsnorm_fwd", xd.data_ptr(), wd.data_ptr(), 1e-6, T, D, xn.data_ptr(), rstd.data_ptr(), st)
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    ref = block_ref.rmsnorm(xr, wr, 1e-6)
    # one rounding of an fp32 result: half a bf16 ulp
    assert (xn.float().cpu() - ref.detach()).abs().max().item() <= 2.0 ** -8 * ref.detach().abs().max().item() + 1e-6
    torch.testing.assert_close(rstd.cpu(), torch.rsqrt(x.pow(2).mean(-1) + 1e-6), rtol=1e-5, atol=1e-6)
    (ref * d_xn).sum().backward()
    dx, dw = torch.empty(T, D, **bf), torch.empty(D, dtype=torch.float32, device=dev)
    ws = torch.empty(_cabi.load().lmoe_rmsnorm_workspace_bytes(D), dtype=torch.uint8, device=dev)
    gd, rd = d_xn.to(**bf), d_res.to(**bf)
    for _ in range(2):                                   # twice: the weight gradient is deterministic
        _cabi.call("lmoe_rmsnorm_bwd", xd.data_ptr(), wd.data_ptr(), rstd.data_ptr(), gd.data_ptr(),
                   rd.data_ptr() if with_residual else None, T, D, dx.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws.numel(), st)
        torch.cuda.synchronize()
        if _ == 0:
            dw0 = dw.clone()
    assert torch.equal(dw, dw0)
    ref_dx = xr.grad + (d_res if with_residual else 0.0)
    _close("dx", dx, ref_dx, 1e-2)
    torch.testing.assert_close(dw.cpu(), wr.grad, rtol=2e-4, atol=2e-4 * wr.grad.abs().max().item())
    out = torch.empty(T, D, **bf)
    _cabi.call("lmoe_add_bf16", xd.data_ptr(), gd.data_ptr(), out.data_ptr(), T * D, st)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), (x + d_xn).to(torch.bfloat16))


def test_rmsnorm_kernels_match_reference_fixture():
    from swamla_b200.block import _NormAndPass
    fx = torch.load(golden_path("rmsnorm"), weights_only=False)
    g = torch.Generator().manual_seed(fx["seed"])
    x = torch.randn(fx["T"], fx["D"], generator=g)
    w = 1.0 + 0.1 * torch.randn(fx["D"], generator=g)
    dy = torch.randn(fx["T"], fx["D"], generator=g)
    xg = x.to("cuda:0").requires_grad_(True)                  # fp32 in -> fp32 out (bf16 arithmetic on the rows)
    wg = w.to("cuda:0").requires_grad_(True)
    y, x_pass = _NormAndPass.apply(xg, wg, fx["eps"])
    assert y.dtype == torch.float32
    (y * dy.to("cuda:0")).sum().backward()
    _close("y", y, fx["y"])
    _close("dx", xg.grad, fx["dx"])
    _close("dw", wg.grad, fx["dw"])


def test_norm_arguments_are_checked():
    from swamla_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda:0")
    x = torch.zeros(4, 4096, dtype=torch.bfloat16, device=dev)
    w = torch.ones(4096, device=dev)
    r = torch.zeros(4, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.lmoe_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), 1e-6, 4, 4096, x.data_ptr(), r.data_ptr(), st) == -2   # D > 2048
    assert lib.lmoe_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), 1e-6, 4, 12, x.data_ptr(), r.data_ptr(), st) == -2     # D % 8
    assert lib.lmoe_rmsnorm_fwd(None, w.data_ptr(), 1e-6, 4, 64, x.data_ptr(), r.data_ptr(), st) == -1
    assert lib.lmoe_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), r.data_ptr(), x.data_ptr(), None, 4, 64, x.data_ptr(),
                                w.data_ptr(), x.data_ptr(), 16, st) == -4                                          # workspace
    assert lib.lmoe_add_bf16(x.data_ptr(), x.data_ptr(), x.data_ptr(), 12, st) == -2


@pytest.mark.parametrize("name", ["tiny", "tiny_moe"])
def test_block_with_moe_layer_matches_oracle(name):
    """x + moe(rmsnorm(x)) with the drop-in layers, forward and backward, against the fp32 oracle composition."""
    from swamla_b200 import functional
    from swamla_b200.block import NormedResidualFFN
    from swamla_b200.layer import create_moe_layer
    w = inputs.WORKLOADS[name]
    params, buffers, x, dy = inputs.make_inputs(w)
    g = torch.Generator().manual_seed(3)
    nw = 1.0 + 0.1 * torch.randn(w.D, generator=g)
    layer = create_moe_layer(w.config())
    layer.load_state_dict({**params, **buffers}, strict=True)
    block = NormedResidualFFN(layer, w.D, eps=1e-6)
    with torch.no_grad():
        block.ffn_norm.weight.copy_(nw)
    assert set(block.state_dict()) == {"ffn_norm.weight"} | {"ffn." + k for k in list(params) + list(buffers)}
    block = block.to("cuda:0").to(torch.bfloat16).train()
    rb = inputs.round_to_bf16
    pr = {k: rb(v) for k, v in params.items()}

    def oracle(sel_override=None):
        xr = rb(x).clone().requires_grad_(True)
        p = {k: v.clone().requires_grad_(True) for k, v in pr.items()}
        nwr = rb(nw).clone().requires_grad_(True)
        cache = {}

        def ffn(xn):
            cache.update(R.layer_forward(p, buffers, xn, w.K, w.router_z_loss_coef, sel_override=sel_override))
            return cache["y"]

        out = block_ref.ffn_block_residual(xr, nwr, 1e-6, ffn)
        (out * rb(dy)).sum().backward()
        grads = {"ffn." + k: v.grad for k, v in p.items()}
        grads["ffn_norm.weight"] = nwr.grad
        return out.detach(), xr.grad, grads, cache["sel"]

    def run(force=None):
        for p_ in block.parameters():
            p_.grad = None
        xg = x.to("cuda:0").to(torch.bfloat16).requires_grad_(True)
        functional._testing.FORCE_SEL = force
        try:
            out = block(xg)
            (out.float() * dy.to("cuda:0").to(torch.bfloat16).float()).sum().backward()
            torch.cuda.synchronize()
        finally:
            functional._testing.FORCE_SEL = None
        return out, xg

    ref_out, ref_dx, ref_grads, ref_sel = oracle()
    out, xg = run()
    sel = layer.router._last_selected_experts.cpu().long()
    if not torch.equal(sel, ref_sel):            # bf16-rounded normed activations flip near-ties: compare on one selection
        assert (sel != ref_sel).any(dim=1).float().mean().item() < 0.3
        out, xg = run(force=ref_sel)
    assert out.dtype == torch.bfloat16 and out.shape == x.shape
    _close("out", out, ref_out)
    _close("dx", xg.grad, ref_dx)
    named = dict(block.named_parameters())
    for k, ref in ref_grads.items():
        assert named[k].grad is not None, k
        _close(f"grad {k}", named[k].grad, ref)


def test_fp32_residual_stream_is_not_rounded_to_bf16():
    """Under the reference's autocast training the residual stream is fp32 (train.py:1195): the block must add the
    feed-forward output to x in fp32 and hand the residual branch's gradient back unrounded.  With a feed-forward
    branch a thousand times smaller than x, any bf16 rounding of the residual (2^-9 relative) would dwarf the error of
    the branch itself."""
    from swamla_b200.block import NormedResidualFFN

    class Scale(torch.nn.Module):            # a stand-in feed-forward so that only the block's own arithmetic is seen
        def forward(self, t):
            return t * 1e-3

    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(4)
    x = torch.randn(2, 33, 256, generator=g) * 3.0
    dy = torch.randn(2, 33, 256, generator=g) * 3.0
    block = NormedResidualFFN(Scale(), 256).to(dev)
    xg = x.to(dev).requires_grad_(True)
    out = block(xg)
    assert out.dtype == torch.float32
    out.backward(dy.to(dev))
    xr = x.clone().requires_grad_(True)
    ref = xr + 1e-3 * block_ref.rmsnorm(xr, torch.ones(256), 1e-6)
    ref.backward(dy)
    assert (out.detach().cpu() - ref.detach()).abs().max().item() <= 2e-5          # bf16 rounding of x would be ~2e-2
    assert (xg.grad.cpu() - xr.grad).abs().max().item() <= 2e-5
    assert (x.to(torch.bfloat16).float() - x).abs().max().item() > 1e-3            # (what a bf16 residual would lose)
