"""The CTA-pair GEMM kernel (tcgen05 cta_group::2) through the C ABI against a torch fp32 matmul and against the
single-CTA kernel."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def pair_kernel():
    from swamla_b200 import _cabi
    lib = _cabi.load()
    before = lib.lmoe_pair_gemm_enable(1)
    yield lib
    lib.lmoe_pair_gemm_enable(before)


def _gemm(M, N, K, a_mn, b_mn, c_f32, split_k=1, seed=0):
    from swamla_b200 import _cabi
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(seed)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16)
    B = torch.randn(N, K, generator=g).to(torch.bfloat16)
    ref = (A.float().to(dev) @ B.float().to(dev).t())
    A_dev = (A.t().contiguous() if a_mn else A.contiguous()).to(dev)
    B_dev = (B.t().contiguous() if b_mn else B.contiguous()).to(dev)
    C = torch.zeros(M, N, dtype=torch.float32 if c_f32 else torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ws_bytes = _cabi.load().lmoe_gemm_workspace_bytes(M, N, split_k)
    ws = torch.empty(max(16, ws_bytes), dtype=torch.uint8, device=dev)
    _cabi.call("lmoe_gemm_bf16", M, N, K, A_dev.data_ptr(), M if a_mn else K, int(a_mn), B_dev.data_ptr(),
               N if b_mn else K, int(b_mn), C.data_ptr(), N, _cabi.F32 if c_f32 else _cabi.BF16, split_k, ws.data_ptr(),
               ws_bytes, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status.item() == 0, _cabi.status_string(status.item())
    return C, ref


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 256, 256), (1024, 512, 1024), (640, 264, 200), (2048 + 136, 1024, 520)])
def test_pair_gemm_bf16_out(pair_kernel, shape, a_mn, b_mn):
    M, N, K = shape
    C, ref = _gemm(M, N, K, a_mn, b_mn, c_f32=False)
    err = (C.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item(), err
    # same operands on the single-CTA kernel: fp32 accumulation of the same products, rounded once
    pair_kernel.lmoe_pair_gemm_enable(0)
    C1, _ = _gemm(M, N, K, a_mn, b_mn, c_f32=False)
    pair_kernel.lmoe_pair_gemm_enable(1)
    assert (C.float() - C1.float()).abs().max().item() <= 2.0 ** -7 * ref.abs().max().item()


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (1, 1)])
def test_pair_gemm_f32_out_many_tiles(pair_kernel, a_mn, b_mn):
    C, ref = _gemm(256 * 90, 512, 320, a_mn, b_mn, c_f32=True)          # more tiles than SM pairs: several per pair
    assert (C - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()


@pytest.mark.parametrize("split_k", [2, 5])
def test_pair_gemm_split_k(pair_kernel, split_k):
    for M, N, K, f32 in [(512, 256, 64 * 37, True), (384, 320, 64 * 9 + 8, False)]:
        C, ref = _gemm(M, N, K, 1, 1, c_f32=f32, split_k=split_k)
        assert (C.float() - ref).abs().max().item() <= (2e-3 if f32 else 2e-2) * ref.abs().max().item()


def test_pair_swiglu_epilogue_matches_single_cta(pair_kernel):
    from swamla_b200 import _cabi
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(4)
    M, H, K = 1000, 384, 256
    A = (torch.randn(M, K, generator=g)).to(torch.bfloat16).to(dev)
    W = (torch.randn(2 * H, K, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    st = torch.cuda.current_stream().cuda_stream
    outs = []
    for on in (1, 0):
        pair_kernel.lmoe_pair_gemm_enable(on)
        h1 = torch.zeros(M, 2 * H, dtype=torch.bfloat16, device=dev)
        hid = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        _cabi.call("lmoe_gemm_swiglu_bf16", M, H, K, A.data_ptr(), K, W.data_ptr(), K, h1.data_ptr(), 2 * H, hid.data_ptr(),
                   H, status.data_ptr(), st)
        torch.cuda.synchronize()
        assert status.item() == 0
        outs.append((h1, hid))
    pair_kernel.lmoe_pair_gemm_enable(1)
    ref = A.float() @ W.float().t()
    assert (outs[0][0].float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    gate, up = outs[0][0].float().chunk(2, -1)
    ref_hid = torch.nn.functional.silu(gate) * up
    assert (outs[0][1].float() - ref_hid).abs().max().item() <= 2e-2 * ref_hid.abs().max().item()
    assert (outs[0][0].float() - outs[1][0].float()).abs().max().item() <= 2.0 ** -7 * ref.abs().max().item()
