"""Implicit-GEMM convolution kernels (forward, data gradient, weight gradient)
against an fp32 CPU reference (needs a B200)."""
import pytest
import torch
import torch.nn.functional as F

from common import assert_tensors_equal

pytestmark = pytest.mark.gpu
DEV = "blackwell"

CASES = [
    # N, C, H, W, K, R, stride, pad
    (4, 64, 56, 56, 256, 1, 1, 0),
    (4, 64, 56, 56, 64, 3, 1, 1),
    (2, 128, 56, 56, 128, 3, 2, 1),
    (2, 256, 56, 56, 512, 1, 2, 0),
    (3, 72, 13, 9, 40, 3, 1, 1),
    (2, 512, 7, 7, 512, 3, 1, 1),
    (2, 3, 224, 224, 64, 7, 2, 3),
    (2, 64, 15, 15, 64, 3, 2, 1),
    # large enough for the resident-weight / halo-tile mode of the single-channel-block 3x3 layers
    (16, 64, 56, 56, 64, 3, 1, 1),
    (24, 32, 30, 27, 64, 3, 1, 1),
    (40, 64, 20, 36, 128, 3, 1, 1),
]


@pytest.fixture(scope="module", autouse=True)
def _backend():
    import catch_b200  # noqa: F401

    assert torch.b200.backend_name() == "cuda"
    torch.b200.set_flag("op_trycatch", False)  # a failing device kernel must not be masked by the CPU fallback
    yield
    torch.b200.set_flag("op_trycatch", True)


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dtype,channels_last", [(torch.bfloat16, True), (torch.float32, False)])
def test_conv_forward_backward(case, dtype, channels_last):
    N, C, H, W, K, R, stride, pad = case
    torch.manual_seed(0)
    x = torch.randn(N, C, H, W)
    w = torch.randn(K, C, R, R) / (C * R * R) ** 0.5
    xq, wq = x.to(dtype).float(), w.to(dtype).float()
    xr, wr = xq.clone().requires_grad_(C >= 8), wq.clone().requires_grad_()
    ref = F.conv2d(xr, wr, None, stride, pad)
    gy = torch.randn_like(ref)
    gyq = gy.to(dtype).float()
    ref.backward(gyq)

    xd = xq.to(dtype).to(DEV)
    wd = wq.to(dtype).to(DEV)
    if channels_last:
        xd = xd.contiguous(memory_format=torch.channels_last)
        wd = wd.contiguous(memory_format=torch.channels_last)
    xd.requires_grad_(C >= 8)
    wd.requires_grad_()
    out = F.conv2d(xd, wd, None, stride, pad)
    assert out.device.type == DEV and out.dtype == dtype
    prec = 2e-2 if dtype == torch.bfloat16 else 3e-3
    assert_tensors_equal(out, ref, prec=prec, use_MSE=True, msg="fprop")
    out.backward(gyq.to(dtype).to(DEV))
    assert_tensors_equal(wd.grad, wr.grad, prec=prec, use_MSE=True, msg="wgrad")
    if C >= 8:
        assert_tensors_equal(xd.grad, xr.grad, prec=prec, use_MSE=True, msg="dgrad")
    from catch_b200.ops import capi

    torch.b200.synchronize()
    assert capi.read_error_flag() == 0


def test_conv_bias():
    torch.manual_seed(1)
    x = torch.randn(2, 64, 10, 10).bfloat16()
    conv = torch.nn.Conv2d(64, 96, 3, padding=1).bfloat16()
    ref = conv(x).float()
    dconv = torch.nn.Conv2d(64, 96, 3, padding=1).bfloat16()
    dconv.load_state_dict(conv.state_dict())
    out = dconv.to(DEV)(x.to(DEV))
    assert_tensors_equal(out, ref, prec=2e-2, use_MSE=True)


@pytest.mark.parametrize("case", [(8, 64, 56, 56, 64, 3, 1, 1), (8, 64, 28, 28, 256, 1, 1, 0), (4, 128, 30, 30, 128, 3, 2, 1),
                                  (3, 256, 14, 14, 320, 1, 1, 0), (64, 512, 7, 7, 512, 3, 1, 1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_conv2d_stats_matches_output(case, dtype):
    """The channel sums accumulated in the epilogue equal sums over the stored output."""
    N, C, H, W, K, R, stride, pad = case
    torch.manual_seed(1)
    x = (torch.randn(N, C, H, W) + 0.3).to(dtype).to(DEV).contiguous(memory_format=torch.channels_last)
    w = (torch.randn(K, C, R, R) / (C * R * R) ** 0.5).to(dtype).to(DEV).contiguous(memory_format=torch.channels_last)
    y, sums = torch.ops.catch_b200.conv2d_stats(x, w, [stride, stride], [pad, pad])
    ref = F.conv2d(x.cpu().float(), w.cpu().float(), None, stride, pad)
    assert_tensors_equal(y, ref, prec=2e-2, use_MSE=True, msg="fprop")
    yd = y.cpu().double()
    s_ref = torch.cat([yd.sum((0, 2, 3)), (yd * yd).sum((0, 2, 3))])
    assert sums.dtype == torch.float64 and sums.shape == (2 * K,)
    rel = (sums.cpu() - s_ref).abs() / (s_ref.abs() + 1e-2 * s_ref.abs().max())
    assert rel.max().item() < 5e-5, rel.max().item()


def test_conv_backward_with_fp32_weight_gradient():
    """conv2d_backward_fp32w: data gradient in the activation dtype, weight gradient in fp32 straight from the
    accumulation buffer, laid out like a channels-last weight."""
    torch.manual_seed(3)
    N, C, H, W, K, R = 8, 64, 28, 28, 128, 3
    x = torch.randn(N, C, H, W).bfloat16()
    w = (torch.randn(K, C, R, R) / (C * R * R) ** 0.5).bfloat16()
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    y = F.conv2d(xr, wr, None, 1, 1)
    gy = torch.randn_like(y).bfloat16()
    y.backward(gy.float())
    xd = x.to(DEV).contiguous(memory_format=torch.channels_last)
    wd = w.to(DEV).contiguous(memory_format=torch.channels_last)
    gd = gy.to(DEV).contiguous(memory_format=torch.channels_last)
    dx, dw = torch.ops.catch_b200.conv2d_backward_fp32w(gd, xd, wd, [1, 1], [1, 1], True, True)
    assert dx.dtype == torch.bfloat16 and dw.dtype == torch.float32 and dw.shape == w.shape
    assert dw.is_contiguous(memory_format=torch.channels_last)
    assert_tensors_equal(dx, xr.grad, prec=2e-2, use_MSE=True, msg="dx")
    assert_tensors_equal(dw, wr.grad, prec=3e-3, use_MSE=True, msg="dw")  # fp32 accumulation, no 16-bit rounding
    dx2, dw2 = torch.ops.catch_b200.conv2d_backward_fp32w(gd, xd, wd, [1, 1], [1, 1], False, True)
    assert_tensors_equal(dw2, wr.grad, prec=3e-3, use_MSE=True, msg="dw only")


HALO_WGRAD_CASES = [
    # N, C, H, W, K: stride-1 3x3 layers whose weight gradient takes the shared-window kernel
    (8, 64, 56, 56, 64),     # one channel block, half-empty M tile
    (6, 128, 28, 28, 128),   # two channel blocks per item (N = 384), W = 28 -> a partly empty column tile
    (5, 256, 14, 14, 256),   # two M tiles, two channel groups, odd batch
    (3, 512, 7, 7, 512),     # 7 rows per image: K steps straddle images, batch not a multiple of the chunk
    (4, 192, 20, 12, 72),    # three channel blocks (last group has one), Cout not a multiple of 64
]


@pytest.mark.parametrize("mode", [1, 2, 0])
@pytest.mark.parametrize("case", HALO_WGRAD_CASES)
def test_wgrad_shared_window_kernel(case, mode):
    """conv_wgrad_halo_kernel (mode 1: one N = 192 MMA over three overlapping windows; mode 2: one MMA per window)
    and the plain kernel (mode 0) against the fp32 CPU gradient, added into an fp32 buffer that already holds
    values (the bucket accumulation path) and returned as a tensor."""
    import catch_b200

    N, C, H, W, K = case
    torch.manual_seed(2)
    x = torch.randn(N, C, H, W).bfloat16()
    w = (torch.randn(K, C, 3, 3) / (C * 9) ** 0.5).bfloat16()
    gy = torch.randn(N, K, H, W).bfloat16()
    wr = w.float().requires_grad_()
    F.conv2d(x.float(), wr, None, 1, 1).backward(gy.float())
    cl = torch.channels_last
    xd, wd, gd = (t.to(DEV).contiguous(memory_format=cl) for t in (x, w, gy))
    prev = catch_b200._C._conv_wgrad_halo_mode(mode)
    try:
        _, dw = torch.ops.catch_b200.conv2d_backward_fp32w(gd, xd, wd, [1, 1], [1, 1], False, True, None)
        acc = torch.full((K * 9 * C,), 0.5, device=DEV)
        torch.ops.catch_b200.conv2d_backward_fp32w(gd, xd, wd, [1, 1], [1, 1], False, True, acc)
    finally:
        catch_b200._C._conv_wgrad_halo_mode(prev)
    assert dw.dtype == torch.float32
    assert_tensors_equal(dw.cpu(), wr.grad, prec=1e-2, use_MSE=True, msg=f"mode {mode}")
    got = acc.cpu().view(K, 3, 3, C).permute(0, 3, 1, 2) - 0.5
    assert_tensors_equal(got, wr.grad, prec=1e-2, use_MSE=True, msg=f"mode {mode} accumulate")
    from catch_b200.ops import capi

    torch.b200.synchronize()
    assert capi.read_error_flag() == 0
