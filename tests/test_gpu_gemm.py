"""tcgen05 GEMM kernel against an fp32 PyTorch reference (needs a B200)."""
import pytest
import torch

from common import assert_tensors_equal

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().transpose(-1, -2) if a_mn else a.float()
    B = b.float().transpose(-1, -2) if b_mn else b.float()
    return A @ B.transpose(-1, -2)


def _check_flag():
    from catch_b200.ops import capi

    torch.cuda.synchronize()
    assert capi.read_error_flag() == 0, "kernel reported a bounded-wait timeout"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (300, 1000, 2048), (4096, 768, 3072), (77, 40, 136)])
def test_gemm_k_major(shape, dtype):
    from catch_b200.ops import capi

    M, N, K = shape
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    b = torch.randn(N, K, device="cuda", dtype=dtype)
    d = capi.gemm(a, b, out_dtype=torch.float32)
    _check_flag()
    assert_tensors_equal(d, _ref(a, b, False, False), prec=3e-3, use_MSE=True)


@pytest.mark.parametrize("a_mn,b_mn", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("shape", [(256, 256, 128), (384, 320, 200), (2048, 1000, 256)])
def test_gemm_mn_major(shape, a_mn, b_mn):
    from catch_b200.ops import capi

    M, N, K = shape
    torch.manual_seed(1)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    d = capi.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out_dtype=torch.float32)
    _check_flag()
    assert_tensors_equal(d, _ref(a, b, a_mn, b_mn), prec=3e-3, use_MSE=True)


def test_gemm_epilogue_bias_relu_residual():
    from catch_b200.ops import capi

    torch.manual_seed(2)
    M, N, K = 512, 384, 320
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.float32)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    d = capi.gemm(a, b, bias=bias, residual=res, alpha=0.5, beta=2.0, act=1)
    _check_flag()
    ref = torch.relu(0.5 * _ref(a, b, False, False) + bias + 2.0 * res.float())
    assert d.dtype == torch.bfloat16
    assert_tensors_equal(d, ref, prec=2e-2, use_MSE=True)


def test_gemm_batched():
    from catch_b200.ops import capi

    torch.manual_seed(3)
    a = torch.randn(24, 128, 64, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(24, 128, 64, device="cuda", dtype=torch.bfloat16)
    d = capi.gemm(a, b, out_dtype=torch.float32)
    _check_flag()
    assert_tensors_equal(d, _ref(a, b, False, False), prec=3e-3, use_MSE=True)


def test_gemm_tf32():
    from catch_b200.ops import capi

    torch.manual_seed(4)
    a = torch.randn(256, 192, device="cuda")
    b = torch.randn(320, 192, device="cuda")
    d = capi.gemm(a, b)
    _check_flag()
    assert_tensors_equal(d, a @ b.t(), prec=3e-3, use_MSE=True)
