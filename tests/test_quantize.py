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


def test_data_scale_widens_the_range_like_the_reference():
    from catch_b200.quantize import LrnObserver, MinMaxObserver

    x = torch.tensor([-2.0, 0.5, 4.0])
    plain, wide, lrn = MinMaxObserver(), MinMaxObserver(data_scale=2.0), LrnObserver()
    for o in (plain, wide, lrn):
        o(x)
    assert abs(plain.scale().item() - 127.0 / 4.0) < 1e-6
    assert abs(wide.scale().item() - 127.0 / 8.0) < 1e-6      # min / max are multiplied by data_scale
    assert abs(lrn.scale().item() - 127.0 / 16.0) < 1e-6      # the LRN input is squared by the layer


def test_conv1d_conv3d_modules_and_first_conv():
    """Conv1d / Conv3d are swapped like Conv2d; the first Conv2d carries input_mean / input_std (x 255) through
    the state dict and normalises raw inputs itself at inference time."""
    import pytest
    from catch_b200.quantize import QuantConv1d, QuantConv2d, QuantConv3d

    class Multi(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c1 = torch.nn.Conv1d(8, 8, 3, padding=1)
            self.c3 = torch.nn.Conv3d(4, 8, 3, padding=1)

        def forward(self, a, b):
            return self.c1(a).mean(), self.c3(b).mean()

    torch.manual_seed(0)
    m = Multi().eval()
    calib = quantize_dynamic(m, {"iteration": 2}, gen_quant=True)
    assert isinstance(calib.c1, QuantConv1d) and isinstance(calib.c3, QuantConv3d)
    a, b = torch.randn(2, 8, 16), torch.randn(1, 4, 5, 6, 7)
    calib(a, b)
    sd = calib.state_dict()
    infer = quantize_dynamic(m)
    infer.load_state_dict(sd, strict=False)
    assert infer.c1.is_quantized() and infer.c3.is_quantized()
    out = infer.to("blackwell")(a.to("blackwell"), b.to("blackwell"))
    ref = m(a, b)
    for o, r in zip(out, ref):
        assert abs(o.item() - r.item()) < 5e-2 * (abs(r.item()) + 1e-2) + 2e-3

    net = Net().eval()
    with pytest.raises(AssertionError, match="firstconv"):
        quantize_dynamic(net, {"firstconv": True}, gen_quant=True)
    mean, std = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]
    calib = quantize_dynamic(net, {"firstconv": True, "mean": mean, "std": std, "iteration": 2}, gen_quant=True)
    g = torch.Generator().manual_seed(3)
    raw = torch.rand(4, 3, 16, 16, generator=g) * 255.0
    norm = (raw / 255.0 - torch.tensor(mean).view(1, 3, 1, 1)) / torch.tensor(std).view(1, 3, 1, 1)
    calib(norm)                                   # calibration sees normalised inputs
    sd = calib.state_dict()
    assert torch.allclose(sd["conv1.input_mean"].flatten(), torch.tensor(mean) * 255)
    assert torch.allclose(sd["conv1.input_std"].flatten(), torch.tensor(std) * 255)
    assert "conv2.input_mean" not in sd           # only the first convolution
    infer = quantize_dynamic(net)
    missing, unexpected = infer.load_state_dict(sd, strict=False)
    assert not missing and not unexpected
    assert isinstance(infer.conv1, QuantConv2d) and infer.conv1.input_std is not None
    out = infer.to("blackwell")(raw.to("blackwell"))  # inference takes the raw 0..255 image
    assert_tensors_equal(out, net(norm), prec=3e-2, use_MSE=True)
    sd2 = infer.state_dict()                      # an inference module saves the values as loaded
    assert torch.allclose(sd2["conv1.input_mean"].cpu().flatten(), torch.tensor(mean) * 255)


class ResBlockNet(torch.nn.Module):
    """stem (float) -> [conv-relu-conv-relu-conv + skip, relu] -> conv -> pooled linear: every quantized chain shape."""

    def __init__(self):
        super().__init__()
        self.stem = torch.nn.Conv2d(3, 16, 3, padding=1)
        self.a = torch.nn.Conv2d(16, 16, 1)
        self.b = torch.nn.Conv2d(16, 16, 3, padding=1)
        self.c = torch.nn.Conv2d(16, 16, 1)
        self.d = torch.nn.Conv2d(16, 32, 3, stride=2, padding=1)
        self.fc = torch.nn.Linear(32, 10)
        self.relu = torch.nn.ReLU(inplace=True)

    def forward(self, x):
        x = self.relu(self.stem(x))
        y = self.relu(self.a(x))
        y = self.relu(self.b(y))
        y = self.c(y)
        y += x
        y = self.relu(y)
        y = self.d(y)
        return self.fc(y.mean((2, 3)))


def test_quantized_trace_fuses_chains_and_requantizes_between_layers():
    """Reference flow test/magicmind/test_quantization.py:44-75: calibrate -> state dict -> load -> trace -> compare;
    the fusion pass folds conv + add + relu and hands int8 from layer to layer."""
    from catch_b200 import jit

    torch.manual_seed(0)
    net = ResBlockNet().eval()
    mixed = {"stem": "float"}
    calib = quantize_dynamic(net, {"per_channel": True, "iteration": 4}, dtype="int8", gen_quant=True, mixed_layer=mixed)
    g = torch.Generator().manual_seed(1)
    for _ in range(4):
        calib(torch.randn(8, 3, 16, 16, generator=g))
    infer = quantize_dynamic(net, mixed_layer=mixed)
    infer.load_state_dict(calib.state_dict(), strict=False)
    infer = infer.eval().to("blackwell")
    x = torch.randn(8, 3, 16, 16, generator=g)
    xd = x.to("blackwell")
    eager = infer(xd)
    assert_tensors_equal(eager, net(x), prec=3e-2, use_MSE=True)
    opt = jit.optimize(torch.jit.trace(infer, xd))
    text = str(opt.graph)  # prints the groups' subgraphs as well
    assert "catch_b200::FusionGroup" in text
    assert text.count("catch_b200::qconv_act(") == 4 and "catch_b200::conv2d" not in text
    assert "aten::relu" not in text.replace("relu_", "") and "aten::add(" not in text
    # a -> b and b -> c hand over int8 (non-zero output scale); c feeds the skip connection and d the pooling: float
    import re

    scales = [float(v) for v in re.findall(r"float = prim::Constant\[value=([0-9.eE+-]+)\]", text)]
    assert sum(1 for v in scales if v > 0) >= 2
    out = opt(xd)
    # same quantization points as the eager quantized model: only rounding-order differences remain
    assert_tensors_equal(out, eager, prec=1e-2, use_MSE=True)
    assert_tensors_equal(out, net(x), prec=3e-2, use_MSE=True)
