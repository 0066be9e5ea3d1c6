"""Graph rewrites on model families other than ResNet (host-simulated device: the passes are the same code on a GPU).

``jit.optimize`` (freeze, lower, fuse, partition into groups) must reproduce the eager result, and ``fuse_bn_act`` (fx)
must reproduce the unfused module in training and in evaluation mode with an unchanged state dict.  ShuffleNet has
shape arithmetic and a view() behind a contiguous() (channel shuffle), MobileNetV3 hard-swish and squeeze-excitation,
GoogLeNet concatenations, EfficientNet stochastic depth (a module whose behaviour depends on ``self.training``)."""
import copy

import pytest
import torch
import torchvision

import catch_b200  # noqa: F401
from catch_b200 import jit
from catch_b200.fusion import fuse_bn_act

FAMILIES = ["shufflenet_v2_x0_5", "mobilenet_v3_small", "googlenet", "efficientnet_b0", "densenet121", "squeezenet1_1"]


def _model(name):
    torch.manual_seed(0)
    kw = {"aux_logits": False, "init_weights": False} if name == "googlenet" else {}
    return getattr(torchvision.models, name)(num_classes=10, **kw)


@pytest.mark.parametrize("name", FAMILIES)
def test_fusion_mode_reproduces_eager(name):
    m = _model(name).eval()
    x = torch.randn(2, 3, 64, 64)
    with torch.no_grad():
        ref = m(x)
        dev = copy.deepcopy(m).to("blackwell")
        xd = x.to("blackwell")
        fused = jit.optimize(torch.jit.trace(dev, xd))
        out, again = fused(xd), fused(xd)
    assert "catch_b200::FusionGroup" in str(fused.graph)
    assert (out.cpu() - ref).abs().max().item() <= 1e-4 * (ref.abs().max().item() + 1e-6)
    assert torch.equal(out.cpu(), again.cpu())


@pytest.mark.parametrize("name", FAMILIES)
def test_training_time_fusion_reproduces_the_module(name):
    m = _model(name)
    x = torch.randn(2, 3, 64, 64)
    fused, plain = fuse_bn_act(copy.deepcopy(m).train()), copy.deepcopy(m).train()
    assert set(fused.state_dict()) == set(m.state_dict())
    torch.manual_seed(1)
    a = fused(x)
    torch.manual_seed(1)
    b = plain(x)
    assert (a - b).abs().max().item() <= 1e-5 * (b.abs().max().item() + 1e-6)
    fused.eval(); plain.eval()   # fused in training mode, evaluated afterwards: nothing of the mode may be frozen
    with torch.no_grad():
        assert (fused(x) - plain(x)).abs().max().item() <= 1e-5 * (plain(x).abs().max().item() + 1e-6)
