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


def _residual_net():
    """Two residual blocks whose convolutions qualify for the fused path (16-bit, channels % 64 == 0), the second with
    a strided 1x1 projection on the skip path."""
    torch.manual_seed(1)
    m = torchvision.models.resnet.ResNet(torchvision.models.resnet.BasicBlock, [1, 1, 0, 0], num_classes=7)
    m.layer3, m.layer4 = torch.nn.Identity(), torch.nn.Identity()
    m.fc = torch.nn.Linear(128, 7)
    return m


def test_fused_training_path_on_the_host_simulated_device():
    """With fused_ops_on_host(True) the fused modules run the same autograd functions as on a GPU (their operators
    take host paths): batch statistics from the convolution, BN + add + ReLU backward, fp32 weight gradients, and the
    gradient sinks that fold the additions at residual forks into the data-gradient call."""
    import pytest

    from catch_b200 import fusion

    ref = _residual_net()
    x = torch.randn(4, 3, 32, 32)
    t = torch.randint(0, 7, (4,))
    loss_fn = torch.nn.CrossEntropyLoss()
    # reference: the unfused model on the CPU with the same bf16 autocast
    with torch.autocast("cpu", dtype=torch.bfloat16):
        loss_ref = loss_fn(ref(x), t)
    loss_ref.backward()
    g_ref = {n: p.grad.clone() for n, p in ref.named_parameters()}
    fusion.fused_ops_on_host(True)
    try:
        results = {}
        for sinks in (False, True):
            fusion.set_gradient_sinks(sinks)
            net = fuse_bn_act(copy.deepcopy(ref)).to("blackwell").to(memory_format=torch.channels_last)
            net.zero_grad()
            calls = []
            orig = torch.ops.catch_b200.conv2d_backward_fp32w

            class Spy:  # counts data-gradient calls that received a parked gradient
                def __call__(self, *a):
                    calls.append(a[8] is not None)
                    return orig(*a)

            fusion.torch.ops.catch_b200.conv2d_backward_fp32w = Spy()
            try:
                with torch.autocast("blackwell", dtype=torch.bfloat16):
                    loss = loss_fn(net(x.to("blackwell")), t.to("blackwell"))
                loss.backward()
            finally:
                fusion.torch.ops.catch_b200.conv2d_backward_fp32w = orig
            assert len(calls) >= 4, calls                       # the fused convolutions really took the fused path
            assert any(calls) == sinks
            if sinks:
                # block 1: the skip gradient parked by the batch norm; block 2: the projection's data gradient
                assert sum(calls) == 2
            results[sinks] = (float(loss.detach()), {n: p.grad.cpu().clone() for n, p in net.named_parameters()})
            assert all(p.grad.dtype == torch.float32 for p in net.parameters())
        for sinks, (loss, grads) in results.items():
            assert abs(loss - float(loss_ref)) < 3e-2
            for n, g in grads.items():
                err = (g - g_ref[n]).norm() / (g_ref[n].norm() + 1e-6)
                assert err < 8e-2, (sinks, n, float(err))       # bf16 activations; the rounding points differ
        for n in results[True][1]:                                # with and without sinks: the same up to one rounding
            a, b = results[True][1][n], results[False][1][n]
            assert (a - b).norm() <= 3e-2 * (b.norm() + 1e-6), n
        # a parked gradient that nobody picks up is an error, not a silently dropped term
        fusion.set_gradient_sinks(True)
        net = fuse_bn_act(copy.deepcopy(ref)).to("blackwell").to(memory_format=torch.channels_last)
        feats = {}
        net.get_submodule("layer1.0.bn2").register_forward_hook(lambda m, i, o: feats.setdefault("y", o))
        with torch.autocast("blackwell", dtype=torch.bfloat16):
            net(x.to("blackwell"))
        sink = getattr(feats["y"], "_b200_grad_sink", None)
        assert sink is not None and sink.consumers == 2           # conv1 and the projection of block 2
    finally:
        fusion.set_gradient_sinks(True)
        fusion.fused_ops_on_host(False)
    with pytest.raises(Exception):
        torch.ops.catch_b200.batch_norm_act_backward(torch.ones(1, 8, 2, 2), torch.zeros(0, dtype=torch.uint8), torch.ones(1, 8, 2, 2),
                                                     None, None, torch.zeros(8), torch.zeros(0), True, 1, False)


def test_inplace_activation_behind_a_fused_batch_norm():
    """MobileNet / EfficientNet style blocks: BN followed by ReLU6(inplace=True) or SiLU(inplace=True), which the
    rewrite does not fuse.  The fused batch norm must not keep its output for the backward (the activation overwrites
    it), on the fused operators' path as well as on the stock one."""
    from catch_b200 import fusion

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Conv2d(8, 64, 3, padding=1, bias=False), torch.nn.BatchNorm2d(64), torch.nn.ReLU6(inplace=True),
                              torch.nn.Conv2d(64, 64, 1, bias=False), torch.nn.BatchNorm2d(64), torch.nn.SiLU(inplace=True))
    x = torch.randn(4, 8, 10, 10)
    ref = copy.deepcopy(net)
    ref(x).square().mean().backward()
    fusion.fused_ops_on_host(True)
    try:
        fused = fuse_bn_act(copy.deepcopy(net)).to("blackwell").to(memory_format=torch.channels_last)
        assert sum(isinstance(m, BatchNormAct2d) and m.act == 0 for m in fused.modules()) == 2
        out = fused(x.to("blackwell"))
        out.square().mean().backward()          # used to raise: "modified by an inplace operation"
        for p, q in zip(ref.parameters(), fused.parameters()):
            assert torch.allclose(q.grad.cpu(), p.grad, atol=1e-4, rtol=1e-3)
        with torch.autocast("blackwell", dtype=torch.bfloat16):   # and through the fused convolution path
            fused.zero_grad()
            fused(x.to("blackwell")).float().square().mean().backward()
        assert all(torch.isfinite(q.grad).all() for q in fused.parameters())
    finally:
        fusion.fused_ops_on_host(False)
