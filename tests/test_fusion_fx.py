"""fx fusion of BN(+add)+ReLU: same results and state dict as the unfused model (CPU path)."""
import copy

import torch
import torchvision

import catch_b200  # noqa: F401
from catch_b200.fusion import BatchNormAct2d, StatsConv2d, fuse_bn_act


def test_fuse_resnet_keeps_semantics_and_state_dict():
    torch.manual_seed(0)
    ref = torchvision.models.resnet18(num_classes=10)
    fused = fuse_bn_act(copy.deepcopy(ref))
    assert fused.fused_bn_act_count == 1 + 8 + 8  # stem + conv1 of every block + the residual joins
    assert set(fused.state_dict()) == set(ref.state_dict())
    # the three downsample batch norms have no ReLU but still take their statistics from the convolution
    assert sum(isinstance(m, BatchNormAct2d) for m in fused.modules()) == 20
    assert sum(isinstance(m, BatchNormAct2d) and m.act == 0 for m in fused.modules()) == 3
    assert sum(isinstance(m, StatsConv2d) for m in fused.modules()) == 20
    x = torch.randn(4, 3, 64, 64)
    y_ref, y = ref(x), fused(x)
    assert torch.allclose(y, y_ref, atol=1e-5)
    y_ref.sum().backward(); y.sum().backward()
    for (n, a), (_, b) in zip(ref.named_parameters(), fused.named_parameters()):
        assert torch.allclose(a.grad, b.grad, atol=1e-4), n
    for (n, a), (_, b) in zip(ref.named_buffers(), fused.named_buffers()):
        assert torch.allclose(a.float(), b.float(), atol=1e-6), n
    ref.eval(); fused.eval()
    assert torch.allclose(fused(x), ref(x), atol=1e-5)
    # also on the (host-simulated) device
    d = copy.deepcopy(fused).to("blackwell")
    assert torch.allclose(d(x.to("blackwell")).cpu(), ref(x), atol=1e-4)
