"""FusedDataParallel on one GPU (world size one: the same bucket bookkeeping, fused single-device
optimizer kernels): 16-bit parameter copies, convolution weight gradients added straight into the
buckets, gradient accumulation under no_sync(), bucket launch order with unused parameters, and an
optimizer state dict that torch.optim.SGD / AdamW can load."""
import copy

import pytest
import torch
import torch.nn.functional as F

from common import assert_tensors_equal

pytestmark = pytest.mark.gpu
DEV = "blackwell"


def _small_convnet():
    import torchvision

    torch.manual_seed(3)
    return torchvision.models.resnet18(num_classes=16)


def test_direct_weight_gradients_and_lowp_copies_match_plain_training():
    """The fused wrapper (weight gradients added into the buckets by the kernel, bf16 weight copies written
    by the optimizer kernel) must take the same steps as FusedSGD on the plain fused model."""
    from catch_b200.fusion import StatsConv2d, fuse_bn_act
    from catch_b200.optim import FusedSGD
    from catch_b200.parallel import FusedDataParallel

    ref = _small_convnet()
    a = fuse_bn_act(copy.deepcopy(ref)).to(DEV).to(memory_format=torch.channels_last)
    b = fuse_bn_act(copy.deepcopy(ref)).to(DEV).to(memory_format=torch.channels_last)
    opt = FusedSGD(a.parameters(), lr=0.01, momentum=0.9, weight_decay=1e-4)
    fdp = FusedDataParallel(b, "sgd", lr=0.01, momentum=0.9, weight_decay=1e-4, bucket_mb=1.0)
    assert len(fdp.buckets) > 2
    convs = [m for m in b.modules() if isinstance(m, StatsConv2d)]
    assert all(hasattr(m.weight, "_b200_lowp") and m.weight._b200_lowp.dtype == torch.bfloat16 for m in convs)
    start = {n: p.detach().cpu().clone() for n, p in a.named_parameters()}
    g = torch.Generator().manual_seed(5)
    for it in range(3):
        x = torch.randn(8, 3, 64, 64, generator=g).to(DEV)
        t = torch.randint(0, 16, (8,), generator=g).to(DEV)
        with torch.autocast(DEV, dtype=torch.bfloat16):
            la = F.cross_entropy(a(x), t)
            lb = F.cross_entropy(fdp(x), t)
        opt.zero_grad()
        la.backward(); opt.step()
        lb.backward(); fdp.step()
        if it == 0:
            # the sharp check: both runs start from the same weights, so their first updates (learning rate times
            # gradient) agree up to the order of the fp32 reduce-adds in the weight-gradient kernels
            assert abs(la.item() - lb.item()) < 1e-3, (la.item(), lb.item())
            for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
                da, db = p.detach().cpu() - start[n], q.detach().cpu() - start[n]
                assert float((da - db).norm()) <= 1e-2 * float(da.norm()) + 1e-7, n
        # later steps: a batch of 8 with batch norm over as few as 32 values amplifies those rounding differences,
        # so the trajectories are only compared loosely
        assert abs(la.item() - lb.item()) < 1e-1 * max(1.0, abs(la.item())), (la.item(), lb.item())
    # (per tensor the comparison would be dominated by the noisiest gradients, e.g. of biases that start at zero)
    flat_a = torch.cat([p.detach().cpu().flatten() for p in a.parameters()])
    flat_b = torch.cat([q.detach().cpu().flatten() for q in b.parameters()])
    assert_tensors_equal(flat_b, flat_a, prec=3e-2, use_MSE=True, msg="all parameters")
    for m in convs:  # the 16-bit copies follow the masters
        assert torch.equal(m.weight._b200_lowp.cpu(), m.weight.detach().to(torch.bfloat16).cpu())
    for bk in fdp.buckets:  # gradients are cleared for the next step
        assert float(bk.grads.abs().max()) == 0.0


def test_no_sync_accumulates_and_second_backward_raises():
    from catch_b200.parallel import FusedDataParallel

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 4))
    ref = copy.deepcopy(net)
    fdp = FusedDataParallel(net.to(DEV), "sgd", lr=0.1, momentum=0.9, bucket_mb=0.001, lowp_dtype=None)
    opt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    g = torch.Generator().manual_seed(1)
    for _ in range(3):
        xs = [torch.randn(8, 32, generator=g) for _ in range(2)]
        opt.zero_grad()
        for x in xs:
            ref(x).pow(2).mean().backward()
        opt.step()
        with fdp.no_sync():
            fdp(xs[0].to(DEV)).pow(2).mean().backward()
        fdp(xs[1].to(DEV)).pow(2).mean().backward()
        fdp.step()
    for p, q in zip(ref.parameters(), fdp.module.parameters()):
        assert_tensors_equal(q, p, prec=3e-3)
    fdp(torch.randn(8, 32).to(DEV)).sum().backward()
    with pytest.raises(RuntimeError, match="no_sync"):
        fdp(torch.randn(8, 32).to(DEV)).sum().backward()


def test_buckets_launch_in_order_with_unused_parameters():
    from catch_b200.parallel import FusedDataParallel

    class Two(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(16, 16)
            self.unused = torch.nn.Linear(16, 16)
            self.b = torch.nn.Linear(16, 4)

        def forward(self, x):
            return self.b(torch.tanh(self.a(x)))

    torch.manual_seed(0)
    net = Two()
    before = copy.deepcopy(net.state_dict())
    fdp = FusedDataParallel(net.to(DEV), "sgd", lr=0.1, bucket_mb=0.0005, lowp_dtype=None)
    order = []
    launch = fdp._launch
    fdp._launch = lambda b: (order.append(b.index), launch(b))[1]
    fdp(torch.randn(4, 16).to(DEV)).sum().backward()
    fdp.step()
    assert order == sorted(order) and len(order) == len(fdp.buckets), order
    after = fdp.module.state_dict()
    assert torch.equal(after["unused.weight"].cpu(), before["unused.weight"])   # zero gradient, no weight decay
    assert not torch.equal(after["a.weight"].cpu(), before["a.weight"])


@pytest.mark.parametrize("kind", ["sgd", "adamw"])
def test_optimizer_state_dict_loads_into_stock_optimizer(kind):
    from catch_b200.parallel import FusedDataParallel

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 4))
    ref = copy.deepcopy(net)
    if kind == "sgd":
        fdp = FusedDataParallel(net.to(DEV), "sgd", lr=0.05, momentum=0.9, weight_decay=1e-4, bucket_mb=0.001)
        mk = lambda ps: torch.optim.SGD(ps, lr=0.05, momentum=0.9, weight_decay=1e-4)  # noqa: E731
    else:
        fdp = FusedDataParallel(net.to(DEV), "adamw", lr=1e-2, weight_decay=0.01, bucket_mb=0.001)
        mk = lambda ps: torch.optim.AdamW(ps, lr=1e-2, weight_decay=0.01)  # noqa: E731
    opt = mk(ref.parameters())
    g = torch.Generator().manual_seed(2)
    data = [torch.randn(8, 32, generator=g) for _ in range(6)]
    for x in data[:3]:
        opt.zero_grad(); ref(x).pow(2).mean().backward(); opt.step()
        fdp(x.to(DEV)).pow(2).mean().backward(); fdp.step()
    # the wrapper's state loads into a fresh stock optimizer, which then continues identically
    sd = fdp.optimizer_state_dict()
    resumed = copy.deepcopy(ref)
    resumed.load_state_dict({k: v.cpu() for k, v in fdp.module.state_dict().items()})
    opt2 = mk(resumed.parameters())
    opt2.load_state_dict(sd)
    # ... and the stock optimizer's state loads into a fresh wrapper
    net3 = copy.deepcopy(ref)
    fdp3 = FusedDataParallel(net3.to(DEV), kind, **({"lr": 0.05, "momentum": 0.9, "weight_decay": 1e-4} if kind == "sgd"
                                                    else {"lr": 1e-2, "weight_decay": 0.01}), bucket_mb=0.002)
    fdp3.load_optimizer_state_dict(opt.state_dict())
    for x in data[3:]:
        opt.zero_grad(); ref(x).pow(2).mean().backward(); opt.step()
        opt2.zero_grad(); resumed(x).pow(2).mean().backward(); opt2.step()
        fdp3(x.to(DEV)).pow(2).mean().backward(); fdp3.step()
    # fp32 linears run as TF32 on the device: where a gradient is within rounding of zero Adam's normalised step
    # can take the other sign (a difference of 2 * lr in that element), so AdamW is compared by relative RMS
    kw = dict(prec=3e-3) if kind == "sgd" else dict(prec=1e-2, use_MSE=True)
    for p, q, r in zip(ref.parameters(), resumed.parameters(), fdp3.module.parameters()):
        assert_tensors_equal(q, p, **kw)
        assert_tensors_equal(r, p, **kw)


def test_gradient_sinks_fold_the_fork_additions():
    """The gradients that reach a residual block's input over the skip connection and over the first convolution are
    added in that convolution's data-gradient epilogue (no element-wise add per fork): same parameter and input
    gradients as with the additions left to autograd, also for a second backward pass over a retained graph."""
    import copy

    import catch_b200
    import torchvision
    from catch_b200 import fusion

    torch.manual_seed(5)
    ref = torchvision.models.resnet50(num_classes=8)
    x = torch.randn(4, 3, 64, 64)
    t = torch.randint(0, 8, (4,))
    grads = {}
    for sinks in (False, True):
        fusion.set_gradient_sinks(sinks)
        try:
            m = fusion.fuse_bn_act(copy.deepcopy(ref)).to(DEV).to(memory_format=torch.channels_last)
            xd = x.to(DEV).contiguous(memory_format=torch.channels_last).requires_grad_()
            catch_b200._C._reset_kernel_launch_count()
            with torch.autocast(DEV, dtype=torch.bfloat16):
                loss = F.cross_entropy(m(xd), t.to(DEV))
            loss.backward(retain_graph=sinks)
            launches = catch_b200._C._kernel_launch_count()
            g1 = {n: p.grad.detach().float().cpu().clone() for n, p in m.named_parameters()}
            g1["input"] = xd.grad.detach().float().cpu().clone()
            if sinks:  # a second pass over the same graph accumulates the same gradients again
                loss.backward()
                for n, p in m.named_parameters():
                    assert_tensors_equal(p.grad.float().cpu(), 2 * g1[n], prec=2e-2, use_MSE=True, msg=f"second pass {n}")
            grads[sinks] = (g1, launches, loss.item())
        finally:
            fusion.set_gradient_sinks(True)
    assert abs(grads[True][2] - grads[False][2]) < 1e-3
    assert grads[True][1] <= grads[False][1] - 12, (grads[True][1], grads[False][1])  # 16 fork additions are gone
    for n, a in grads[False][0].items():
        b = grads[True][0][n]
        cos = (a.double().flatten() @ b.double().flatten() / (a.double().norm() * b.double().norm() + 1e-30)).item()
        assert cos > 0.995, (n, cos)


def test_parked_gradient_that_nobody_consumes_is_an_error():
    from catch_b200 import fusion

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.unused = fusion.StatsConv2d(64, 64, 1, bias=False)
            self.conv = fusion.StatsConv2d(64, 64, 3, padding=1, bias=False)
            self.bn = fusion.BatchNormAct2d(64)

        def forward(self, x):
            self.unused(x)  # reads x, but its result never reaches the loss
            return self.bn(self.conv(x), x)

    net = Net().to(DEV).to(memory_format=torch.channels_last).train()
    x = torch.randn(2, 64, 8, 8).to(DEV).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_()
    with torch.autocast(DEV, dtype=torch.bfloat16):
        y = net(x)
    with pytest.raises(RuntimeError, match="parked"):
        y.float().sum().backward()
    # the next iteration starts clean
    fusion.set_gradient_sinks(False)
    try:
        with torch.autocast(DEV, dtype=torch.bfloat16):
            net(x).float().sum().backward()
        assert x.grad is not None
    finally:
        fusion.set_gradient_sinks(True)
