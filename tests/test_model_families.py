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


@pytest.mark.parametrize("name", ["resnet18", "mobilenet_v2", "densenet121", "efficientnet_b0"])
def test_fused_operators_train_then_evaluate_like_the_stock_layers(name):
    """The fused convolution / batch-norm functions themselves (host paths of their operators): two training
    passes, then evaluation: outputs and every buffer (running statistics, batch counters) equal the stock model's."""
    from catch_b200 import fusion

    m = _model(name)
    for mod in m.modules():
        if isinstance(mod, torch.nn.Dropout) or type(mod).__name__ == "StochasticDepth":
            mod.p = 0.0
    fusion.fused_ops_on_host(True)
    try:
        fused = fuse_bn_act(copy.deepcopy(m)).to("blackwell").to(memory_format=torch.channels_last)
        plain = copy.deepcopy(m)
        fused.train(); plain.train()
        for _ in range(2):
            xb = torch.randn(4, 3, 64, 64)
            plain(xb)
            fused(xb.to("blackwell"))
        for (k, a), (_, b) in zip(fused.named_buffers(), plain.named_buffers()):
            assert (a.cpu().float() - b.float()).abs().max().item() <= 1e-4, k
        fused.eval(); plain.eval()
        x = torch.randn(2, 3, 64, 64)
        with torch.no_grad():
            a, b = fused(x.to("blackwell")).cpu(), plain(x)
        assert (a - b).abs().max().item() <= 1e-4 * (b.abs().max().item() + 1e-6)
    finally:
        fusion.fused_ops_on_host(False)


def test_batch_norm_updates_running_statistics_on_the_host_path():
    """The boxed CPU fallback would update copies of the running statistics and drop them (their arguments are not
    marked as written in the operator's schema): batch norm has a host path of its own."""
    bn, ref = torch.nn.BatchNorm2d(5).to("blackwell").train(), torch.nn.BatchNorm2d(5).train()
    for _ in range(3):
        x = torch.randn(8, 5, 6, 6) * 2 + 3
        a, b = bn(x.to("blackwell")), ref(x)
        assert torch.allclose(a.cpu(), b, atol=1e-5)
    assert torch.allclose(bn.running_mean.cpu(), ref.running_mean, atol=1e-6) and ref.running_mean.abs().min() > 0.1
    assert torch.allclose(bn.running_var.cpu(), ref.running_var, atol=1e-5)
    assert int(bn.num_batches_tracked) == 3
    bn1 = torch.nn.BatchNorm1d(10).to("blackwell").train()
    bn1(torch.randn(16, 10).to("blackwell") + 2)
    assert bn1.running_mean.cpu().abs().min() > 0.05
