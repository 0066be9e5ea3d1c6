"""int8 tcgen05 convolution / linear and the quantization kernels on a B200."""
import pytest
import torch

from common import assert_tensors_equal

pytestmark = pytest.mark.gpu
DEV = "blackwell"


@pytest.fixture(scope="module", autouse=True)
def _backend():
    import catch_b200  # noqa: F401

    assert torch.b200.backend_name() == "cuda"
    torch.b200.set_flag("op_trycatch", False)
    yield
    torch.b200.set_flag("op_trycatch", True)


def _fq(t, s):
    return torch.clamp(torch.round(t * s), -127, 127) / s


def _fq_rows(w):
    f = w.reshape(w.shape[0], -1)
    s = 127.0 / f.abs().max(1, keepdim=True).values
    return (torch.clamp(torch.round(f * s), -127, 127) / s).reshape(w.shape)


@pytest.mark.parametrize("shape", [(4, 64, 28, 28, 128, 3, 1, 1), (2, 128, 14, 14, 256, 1, 1, 0), (2, 32, 17, 13, 48, 3, 2, 1)])
def test_int8_conv_matches_fake_quant(shape):
    N, C, H, W, K, R, s, p = shape
    torch.manual_seed(0)
    x = torch.randn(N, C, H, W).half()
    w = (torch.randn(K, C, R, R) / (C * R * R) ** 0.5).half()
    b = torch.randn(K).half()
    s_in = 127.0 / x.float().abs().max().item()
    ref = torch.nn.functional.conv2d(_fq(x.float(), s_in), _fq_rows(w.float()), b.float(), s, p)
    q_scale = torch.tensor([s_in, 1.0])
    q_mode = torch.tensor([3], dtype=torch.int32)
    out = torch.ops.catch_b200.conv2d(x.to(DEV), w.to(DEV), b.to(DEV), [p, p], [s, s], [1, 1], 1, q_scale, q_mode)
    assert out.dtype == torch.float16 and out.device.type == DEV
    assert_tensors_equal(out, ref, prec=3e-3, use_MSE=True)
    # and the quantized result stays close to the floating-point convolution
    fp = torch.nn.functional.conv2d(x.float(), w.float(), b.float(), s, p)
    assert_tensors_equal(out, fp, prec=2e-2, use_MSE=True)


def test_int8_linear_matches_fake_quant():
    torch.manual_seed(1)
    x = torch.randn(300, 512).bfloat16()
    w = (torch.randn(1000, 512) / 512 ** 0.5).bfloat16()
    b = torch.randn(1000).bfloat16()
    s_in = 127.0 / x.float().abs().max().item()
    ref = torch.nn.functional.linear(_fq(x.float(), s_in), _fq_rows(w.float()), b.float())
    out = torch.ops.catch_b200.linear(x.to(DEV), w.to(DEV), b.to(DEV), torch.tensor([s_in, 1.0]), torch.tensor([3], dtype=torch.int32))
    assert_tensors_equal(out, ref, prec=1e-2, use_MSE=True)


def test_quantize_tool_on_device():
    from catch_b200.quantize import quantize_dynamic

    torch.manual_seed(2)
    net = torch.nn.Sequential(torch.nn.Conv2d(16, 32, 3, padding=1), torch.nn.ReLU(), torch.nn.Conv2d(32, 64, 3, stride=2, padding=1),
                              torch.nn.ReLU(), torch.nn.AdaptiveAvgPool2d(1), torch.nn.Flatten(), torch.nn.Linear(64, 16)).eval()
    calib = quantize_dynamic(net, {"per_channel": True}, dtype="int8", gen_quant=True).to(DEV)
    g = torch.Generator().manual_seed(3)
    for _ in range(4):
        calib(torch.randn(8, 16, 20, 20, generator=g).to(DEV))
    sd = {k: v.cpu() for k, v in calib.state_dict().items()}
    infer = quantize_dynamic(net)
    infer.load_state_dict(sd, strict=False)
    x = torch.randn(8, 16, 20, 20, generator=g)
    ref = net(x)
    out = infer.half().to(DEV)(x.half().to(DEV))
    assert_tensors_equal(out, ref, prec=2e-2, use_MSE=True)
