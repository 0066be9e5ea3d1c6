"""ResNet-18 eager fp32 inference through the backend with no GPU: batch 4,
N(0,1) inputs from seed 0, Kaiming-normal conv weights, BN gamma=1 / beta=0 /
running stats 0 / 1; logits must match CPU torch at atol 1e-4."""
import torch
import torchvision

import catch_b200  # noqa: F401


def _make_model():
    torch.manual_seed(0)
    m = torchvision.models.resnet18(weights=None)
    for mod in m.modules():
        if isinstance(mod, torch.nn.Conv2d):
            torch.nn.init.kaiming_normal_(mod.weight, mode="fan_out", nonlinearity="relu")
        elif isinstance(mod, torch.nn.BatchNorm2d):
            torch.nn.init.ones_(mod.weight)
            torch.nn.init.zeros_(mod.bias)
            mod.running_mean.zero_()
            mod.running_var.fill_(1.0)
    return m.eval()


def test_resnet18_logits_match_cpu():
    model = _make_model()
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 3, 224, 224, generator=g)
    with torch.no_grad():
        ref = model(x)
        dev_model = _make_model().to("blackwell")
        out = dev_model(x.to("blackwell"))
    assert out.device.type == "blackwell"
    assert out.shape == (4, 1000)
    assert torch.allclose(out.cpu(), ref, atol=1e-4), (out.cpu() - ref).abs().max()
