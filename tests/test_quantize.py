"""Quantization tool on the host-simulated device: calibrate -> state_dict -> load ->
quantized inference close to floating point (tolerance 2e-2 relative RMS, the
reference's int8 bound)."""
import torch

import catch_b200  # noqa: F401
from catch_b200.quantize import QuantConv2d, QuantLinear, quantize_dynamic
from common import assert_tensors_equal


class Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1 = torch.nn.Conv2d(3, 16, 3, padding=1)
        self.conv2 = torch.nn.Conv2d(16, 32, 3, stride=2, padding=1)
        self.fc = torch.nn.Linear(32, 10)

    def forward(self, x):
        x = torch.relu(self.conv1(x))
        x = torch.relu(self.conv2(x))
        return self.fc(x.mean((2, 3)))


def test_calibrate_save_load_infer():
    torch.manual_seed(0)
    net = Net().eval()
    calib = quantize_dynamic(net, {"per_channel": True, "iteration": 4}, dtype="int8", gen_quant=True,
                             mixed_layer={"conv1": "float"})
    assert isinstance(calib.conv2, QuantConv2d) and isinstance(calib.fc, QuantLinear)
    assert isinstance(calib.conv1, torch.nn.Conv2d) and not isinstance(calib.conv1, QuantConv2d)
    g = torch.Generator().manual_seed(1)
    for _ in range(4):
        calib(torch.randn(8, 3, 16, 16, generator=g))
    sd = calib.state_dict()
    assert {"conv2.scale", "conv2.quantized_mode", "conv2.scale_weight_per_channel", "conv2.quantized_by_channel",
            "fc.scale", "fc.quantized_mode"} <= set(sd)
    assert sd["conv2.quantized_mode"].item() == 3 and sd["conv2.scale"].numel() == 2
    assert sd["conv2.scale_weight_per_channel"].shape == (32,)

    infer = quantize_dynamic(net, mixed_layer={"conv1": "float"})
    missing, unexpected = infer.load_state_dict(sd, strict=False)
    assert not missing and not unexpected
    assert infer.conv2.is_quantized() and infer.fc.is_quantized()
    x = torch.randn(8, 3, 16, 16, generator=g)
    ref = net(x)
    out_cpu = infer(x)
    assert_tensors_equal(out_cpu, ref, prec=2e-2, use_MSE=True)
    out_dev = infer.to("blackwell")(x.to("blackwell"))
    assert out_dev.device.type == "blackwell"
    assert_tensors_equal(out_dev, ref, prec=2e-2, use_MSE=True)
    # the exported dict round-trips through torch.save / torch.load
    import io

    buf = io.BytesIO()
    torch.save(infer.state_dict(), buf)
    buf.seek(0)
    sd2 = torch.load(buf)
    assert torch.equal(sd2["fc.scale"].cpu(), sd["fc.scale"])


def test_unquantized_module_runs_float():
    lin = quantize_dynamic(torch.nn.Sequential(torch.nn.Linear(16, 4)))
    x = torch.randn(3, 16)
    assert not lin[0].is_quantized()
    assert torch.allclose(lin(x), torch.nn.functional.linear(x, lin[0].weight, lin[0].bias))


def test_conv1d_conv3d_view_custom_ops():
    """The remaining custom ops of the reference's namespace (torch.ops.torch_mlu.{conv1d,conv3d,view})."""
    import torch.nn.functional as F

    d = "blackwell"
    torch.manual_seed(0)
    x, w, b = torch.randn(2, 16, 20), torch.randn(8, 16, 3), torch.randn(8)
    y = torch.ops.catch_b200.conv1d(x.to(d), w.to(d), b.to(d), [1], [2], [1], 1, None, None)
    assert torch.allclose(y.cpu(), F.conv1d(x, w, b, 2, 1), atol=1e-5)
    qs, qm = torch.tensor([127.0 / x.abs().max().item(), 127.0 / w.abs().max().item()]), torch.tensor([1])
    yq = torch.ops.catch_b200.conv1d(x.to(d), w.to(d), b.to(d), [1], [2], [1], 1, qs, qm)
    rel = (yq.cpu() - y.cpu()).norm() / y.cpu().norm()
    assert 0 < rel < 5e-2  # quantized, close to the float result
    x3, w3 = torch.randn(1, 4, 5, 6, 7), torch.randn(6, 4, 3, 3, 3)
    y3 = torch.ops.catch_b200.conv3d(x3.to(d), w3.to(d), None, [1, 1, 1], [1, 1, 1], [1, 1, 1], 1, None, None)
    assert torch.allclose(y3.cpu(), F.conv3d(x3, w3, None, 1, 1), atol=1e-4)
    v = torch.ops.catch_b200.view(x.to(d), [2, 320])
    assert v.shape == (2, 320) and v.data_ptr() == v._base.data_ptr() if v._base is not None else True


def test_torchvision_nms_dispatches_to_the_backend():
    import torchvision

    torch.manual_seed(1)
    xy, wh = torch.rand(40, 2) * 50, torch.rand(40, 2) * 20 + 1
    boxes, scores = torch.cat([xy, xy + wh], 1), torch.rand(40)
    keep = torchvision.ops.nms(boxes.to("blackwell"), scores.to("blackwell"), 0.4)
    assert keep.device.type == "blackwell"
    assert torch.equal(keep.cpu(), torchvision.ops.nms(boxes, scores, 0.4))
