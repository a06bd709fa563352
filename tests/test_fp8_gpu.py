"""FP8 (e4m3) expert path: quantisation kernel, e4m3 tcgen05 GEMM in every operand major-ness, and the layer with
`moe_fp8` against the fp32 oracle (tolerance 6e-2) and against the CPU model of the same recipe."""
import pytest
import torch

from oracle import inputs, latent_moe_ref as R, bf16_pipeline as BP

pytestmark = pytest.mark.gpu
RTOL_FP8 = 6e-2


def _quantize_gpu(t_bf16):
    from swamla_b200 import fp8
    rows, cols = t_bf16.shape
    q, deq = fp8.quantize(t_bf16.contiguous(), rows, cols, None, torch.cuda.current_stream().cuda_stream)
    return q, deq


def test_quantize_matches_torch_cast():
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(300, 256, generator=g) * 3).to(torch.bfloat16)
    q, deq = _quantize_gpu(x.cuda())
    torch.cuda.synchronize()
    amax = x.float().abs().max()
    ref = (x.float() * (448.0 / amax)).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert torch.equal(q.cpu().view(torch.float8_e4m3fn).float(), ref.float())
    assert abs(deq.item() - (amax / 448.0).item()) <= 1e-7 * amax.item()
    z, dz = _quantize_gpu(torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda"))
    assert z.abs().max().item() == 0 and dz.item() == 1.0


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("shape", [(128, 128, 128), (384, 272, 512), (1024, 512, 384)])
def test_gemm_fp8_majors(shape, a_mn, b_mn):
    from swamla_b200 import _cabi
    M, N, K = shape
    if (a_mn and M % 16) or (b_mn and N % 16):
        pytest.skip("leading dimension must be a multiple of 16 bytes")
    g = torch.Generator().manual_seed(M + N + K)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    B = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    Aq, da = _quantize_gpu(A)
    Bq, db = _quantize_gpu(B)
    ref = (Aq.view(torch.float8_e4m3fn).float() @ Bq.view(torch.float8_e4m3fn).float().t()) * (da * db)
    A_dev = Aq.t().contiguous() if a_mn else Aq
    B_dev = Bq.t().contiguous() if b_mn else Bq
    C = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _cabi.call("lmoe_gemm_fp8", M, N, K, A_dev.data_ptr(), M if a_mn else K, a_mn, B_dev.data_ptr(), N if b_mn else K, b_mn,
               da.data_ptr(), db.data_ptr(), C.data_ptr(), N, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status.item() == 0
    err = (C.float() - ref).abs().max().item()
    assert err <= 1e-2 * ref.abs().max().item(), err      # exact products, fp32 accumulation, bf16 output rounding


@pytest.mark.parametrize("aux_grad", [0.0, 2.0])
def test_layer_fp8_experts(aux_grad):
    from swamla_b200 import functional
    from swamla_b200.layer import LatentMoELayer
    w = inputs.WORKLOADS["tiny_fp8"]
    params, buffers, x, dy = inputs.make_inputs(w)
    cfg = w.config()
    cfg.moe_fp8 = True
    layer = LatentMoELayer(cfg)
    layer.load_state_dict({**params, **buffers}, strict=True)
    layer = layer.to("cuda:0").to(torch.bfloat16).train()
    xg = x.to("cuda:0").to(torch.bfloat16).requires_grad_(True)
    sink = {}
    functional._testing.SINK = sink
    try:
        y = layer(xg)
        ((y.float() * dy.to("cuda:0").to(torch.bfloat16).float()).sum() + aux_grad * layer.get_aux_loss()).backward()
        torch.cuda.synchronize()
    finally:
        functional._testing.SINK = None
    assert sink["status"].item() == 0
    sel = sink["sel"].cpu().long()
    pr = {k: inputs.round_to_bf16(v) for k, v in params.items()}
    out, grads = R.layer_forward_backward(pr, buffers, inputs.round_to_bf16(x), inputs.round_to_bf16(dy), w.K,
                                          aux_grad=aux_grad, sel_override=sel)
    model, model_grads = BP.forward_backward(params, buffers, x, dy, w.K, aux_grad=aux_grad, sel_override=sel, fp8=True)
    named = dict(layer.named_parameters())
    got = {"x": xg.grad, **{k: named[k].grad for k in grads if k != "x"}}

    # (1) the layer's outputs, y and dx, against the fp32 oracle at the FP8 tolerance
    for name, t, ref in (("y", y, out["y"]), ("grad x", xg.grad, grads["x"])):
        ok, rep = R.within_tolerance(t.detach().float().cpu(), ref, RTOL_FP8)
        assert ok, (name, rep)
    # (2) every gradient: as close to the fp32 oracle as the CPU model of the recipe itself is.  (Three chained
    #     e4m3 GEMMs put the routed-path parameter gradients at ~6.5 % relative Frobenius error in that model.)
    for k, ref in grads.items():
        mine = R.closeness(got[k].detach().float().cpu(), ref, RTOL_FP8)["rel_fro"]
        recipe = R.closeness(model_grads[k], ref, RTOL_FP8)["rel_fro"]
        assert mine <= 1.15 * recipe + 1e-3, (k, mine, recipe)
        assert mine <= 8e-2, (k, mine)
    # (3) against the CPU model of the same recipe: well inside the recipe's own error (amax differences of one
    #     bf16 ulp move the e4m3 rounding boundaries of a few percent of the elements)
    rows = sink["route"].pos.cpu().long()[out["perm"]]
    for k in ("h1", "y_sorted"):
        rep = R.closeness(sink[k].cpu()[rows].float(), model[k], RTOL_FP8)
        assert rep["rel_fro"] <= 2e-2, (k, rep)
    for k in grads:
        rep = R.closeness(got[k].detach().float().cpu(), model_grads[k], RTOL_FP8)
        assert rep["rel_fro"] <= 2.5e-2, (k, rep)
    rep = R.closeness(y.detach().float().cpu(), model["y"], RTOL_FP8)
    assert rep["rel_fro"] <= 5e-3, rep
