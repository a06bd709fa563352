"""tcgen05 GEMM core through the C ABI against a torch fp32 matmul of the same bf16 operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(M, N, K, a_mn, b_mn, c_f32, split_k=1, seed=0):
    from swamla_b200 import _cabi
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(seed)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16)
    B = torch.randn(N, K, generator=g).to(torch.bfloat16)
    ref = (A.float().to(dev) @ B.float().to(dev).t())
    A_dev = (A.t().contiguous() if a_mn else A.contiguous()).to(dev)
    B_dev = (B.t().contiguous() if b_mn else B.contiguous()).to(dev)
    lda = M if a_mn else K
    ldb = N if b_mn else K
    C = torch.zeros(M, N, dtype=torch.float32 if c_f32 else torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ws_bytes = _cabi.load().lmoe_gemm_workspace_bytes(M, N, split_k)
    ws = torch.empty(max(16, ws_bytes), dtype=torch.uint8, device=dev)
    _cabi.call("lmoe_gemm_bf16", M, N, K, A_dev.data_ptr(), lda, int(a_mn), B_dev.data_ptr(), ldb, int(b_mn),
               C.data_ptr(), N, _cabi.F32 if c_f32 else _cabi.BF16, split_k, ws.data_ptr(), ws_bytes,
               status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status.item() == 0, _cabi.status_string(status.item())
    # bf16 operands, fp32 accumulation: error is accumulation order (+ bf16 rounding of C)
    tol = 2e-2 if not c_f32 else 2e-3
    err = (C.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= tol * scale, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 256, 256), (384, 136, 200), (1024, 384, 1024)])
def test_gemm_majors_bf16_out(shape, a_mn, b_mn):
    M, N, K = shape
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("leading dimension must be a multiple of 8")
    _run(M, N, K, a_mn, b_mn, c_f32=False)


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1)])
def test_gemm_wide_tiles_f32_out(a_mn, b_mn):
    # enough tiles that the launcher picks 256-wide accumulators
    _run(128 * 160, 512, 320, a_mn, b_mn, c_f32=True)


@pytest.mark.parametrize("split_k", [2, 5])
def test_gemm_split_k(split_k):
    _run(256, 128, 64 * 37, 1, 1, c_f32=True, split_k=split_k)
    _run(384, 320, 64 * 9 + 8, 1, 1, c_f32=False, split_k=split_k)


def test_gemm_ragged_rows_and_small_k():
    _run(200, 64, 16, 0, 1, c_f32=True)
    _run(72, 256, 40, 0, 0, c_f32=False)


def test_gemm_rejects_bad_arguments():
    from swamla_b200 import _cabi
    lib = _cabi.load()
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    p = x.data_ptr()
    assert lib.lmoe_gemm_bf16(128, 128, 128, None, 128, 0, p, 128, 0, p, 128, 0, 1, None, 0, None, st) == -1
    assert lib.lmoe_gemm_bf16(128, 100, 128, p, 128, 0, p, 128, 0, p, 100, 0, 1, None, 0, None, st) == -2
    assert lib.lmoe_gemm_bf16(128, 128, 128, p + 2, 128, 0, p, 128, 0, p, 128, 0, 1, None, 0, None, st) == -3
    assert lib.lmoe_gemm_bf16(128, 128, 128, p, 128, 0, p, 128, 0, p, 128, 1, 4, None, 0, None, st) == -4
