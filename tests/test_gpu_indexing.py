"""Indexing, sorting, resampling, NMS, losses and the non-dense convolution paths on the
device against the same PyTorch ops on the CPU (needs a B200)."""
import pytest
import torch
import torch.nn.functional as F

from common import assert_tensors_equal

pytestmark = pytest.mark.gpu
DEV = "blackwell"


@pytest.fixture(scope="module", autouse=True)
def _backend():
    import catch_b200  # noqa: F401

    assert torch.b200.backend_name() == "cuda"
    torch.b200.set_flag("op_trycatch", False)  # a failing device kernel must not be masked by the CPU fallback
    torch.b200.set_flag("fallback_to_cpu", False)  # nor may an op silently be unregistered
    yield
    torch.b200.set_flag("op_trycatch", True)
    torch.b200.set_flag("fallback_to_cpu", True)


def dev(t):
    return t.to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
def test_gather_scatter(dtype):
    torch.manual_seed(0)
    x = (torch.randn(5, 7, 6) * 10).to(dtype)
    idx = torch.randint(0, 7, (5, 4, 6))
    assert torch.equal(dev(x).gather(1, dev(idx)).cpu(), x.gather(1, idx))
    assert torch.equal(dev(x).gather(-1, dev(idx[:, :, :3] % 6)).cpu(), x.gather(-1, idx[:, :, :3] % 6))
    # transposed (strided) source
    xt = x.transpose(0, 2)
    it = torch.randint(0, 5, (6, 7, 2))
    assert torch.equal(dev(x).transpose(0, 2).gather(2, dev(it)).cpu(), xt.gather(2, it))
    src = (torch.randn(5, 4, 6) * 10).to(dtype)
    perm = torch.stack([torch.stack([torch.randperm(7)[:4] for _ in range(6)], 1) for _ in range(5)])  # unique targets
    assert torch.equal(dev(x).scatter(1, dev(perm), dev(src)).cpu(), x.scatter(1, perm, src))
    assert torch.equal(dev(x).scatter(1, dev(perm), 3).cpu(), x.scatter(1, perm, 3))
    if dtype != torch.int64:
        got = dev(x).scatter_add(1, dev(idx), dev(src)).cpu()
        ref = x.float().scatter_add(1, idx, src.float())
        # 16-bit inputs are accumulated in fp32 and rounded once at the end
        assert_tensors_equal(got, ref.to(dtype).float(), prec=0.3 if dtype == torch.bfloat16 else 1e-5)


def test_gather_backward_runs_on_device():
    x = torch.randn(4, 9, requires_grad=True)
    idx = torch.randint(0, 9, (4, 5))
    x.gather(1, idx).pow(2).sum().backward()
    xd = x.detach().to(DEV).requires_grad_()
    xd.gather(1, dev(idx)).pow(2).sum().backward()
    assert_tensors_equal(xd.grad, x.grad, prec=1e-5)


def test_advanced_indexing():
    torch.manual_seed(1)
    x = torch.randn(6, 5, 4, 3)
    xd = dev(x)
    i0 = torch.tensor([0, 5, -1, 2])
    i1 = torch.tensor([[1], [4]])
    assert torch.equal(xd[dev(i0)].cpu(), x[i0])
    assert torch.equal(xd[:, dev(i0) % 5].cpu(), x[:, i0 % 5])
    assert torch.equal(xd[dev(i1), dev(i0) % 5].cpu(), x[i1, i0 % 5])
    assert torch.equal(xd[:, :, dev(i0) % 4, dev(i0) % 3].cpu(), x[:, :, i0 % 4, i0 % 3])
    m = x[:, :, 0, 0] > 0
    assert torch.equal(xd[dev(m)].cpu(), x[m])
    assert torch.equal(xd[xd > 0.5].cpu(), x[x > 0.5])
    assert torch.equal(xd.masked_select(dev(m)[:, :, None, None]).cpu(), x.masked_select(m[:, :, None, None]))
    # strided input
    assert torch.equal(xd.permute(1, 0, 2, 3)[dev(i0) % 5].cpu(), x.permute(1, 0, 2, 3)[i0 % 5])


def test_index_put():
    torch.manual_seed(2)
    x = torch.randn(8, 5, 3)
    i0 = torch.tensor([0, 7, 3])
    v = torch.randn(3, 5, 3)
    a, b = x.clone(), dev(x.clone())
    a[i0] = v; b[dev(i0)] = dev(v)
    assert torch.equal(b.cpu(), a)
    a[:, i0 % 5] = 2.5; b[:, dev(i0) % 5] = 2.5
    assert torch.equal(b.cpu(), a)
    dup = torch.tensor([1, 1, 1, 4])
    a.index_put_((dup,), torch.ones(4, 5, 3), accumulate=True)
    b.index_put_((dev(dup),), dev(torch.ones(4, 5, 3)), accumulate=True)
    assert_tensors_equal(b, a, prec=1e-5)
    hb = dev(x.bfloat16())
    ha = x.bfloat16().index_put((dup,), torch.ones(4, 5, 3).bfloat16(), accumulate=True)
    assert_tensors_equal(hb.index_put((dev(dup),), dev(torch.ones(4, 5, 3).bfloat16()), accumulate=True), ha.float(), prec=2e-2)
    m = x > 1.0
    a[m] = 0.0; b[dev(m)] = 0.0
    assert torch.equal(b.cpu(), a)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.bool, torch.int64, torch.uint8])
def test_nonzero(dtype):
    torch.manual_seed(3)
    x = (torch.randn(37, 65, 3) > 0.8).to(dtype) if dtype in (torch.bool, torch.uint8) else (torch.randn(37, 65, 3) * (torch.rand(37, 65, 3) > 0.7)).to(dtype)
    assert torch.equal(dev(x).nonzero().cpu(), x.nonzero())
    z = torch.zeros(10, dtype=dtype)
    assert dev(z).nonzero().shape == (0, 1)
    if dtype == torch.float32:
        assert dev(torch.tensor([-0.0, 0.0, 1.0])).nonzero().cpu().tolist() == [[2]]
    big = torch.zeros(300000, dtype=dtype)
    big[[5, 1024, 299999]] = 1
    assert dev(big).nonzero().cpu().flatten().tolist() == [5, 1024, 299999]


def test_arange_tril_triu():
    for args in [(10,), (2, 11), (0, 1, 0.125), (5, -5, -2)]:
        for dt in (torch.float32, torch.int64, torch.bfloat16):
            if dt == torch.int64 and any(isinstance(a, float) for a in args):
                continue
            assert torch.equal(torch.arange(*args, dtype=dt, device=DEV).cpu(), torch.arange(*args, dtype=dt)), (args, dt)
    x = torch.randn(3, 6, 9)
    for k in (-2, 0, 1):
        assert torch.equal(dev(x).tril(k).cpu(), x.tril(k))
        assert torch.equal(dev(x).triu(k).cpu(), x.triu(k))
    y = dev(x.clone()); y.tril_()
    assert torch.equal(y.cpu(), x.tril())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sort_topk(dtype):
    torch.manual_seed(4)
    x = torch.randn(7, 1000).to(dtype)
    for desc in (False, True):
        v, i = dev(x).sort(-1, descending=desc)
        rv, _ = x.sort(dim=-1, descending=desc, stable=True)
        assert torch.equal(v.cpu(), rv)
        assert torch.equal(x.gather(-1, i.cpu()), rv)
    v, i = dev(x).topk(5, dim=-1)
    rv, _ = x.topk(5, dim=-1)
    assert torch.equal(v.cpu(), rv) and torch.equal(x.gather(-1, i.cpu()), rv)
    v, i = dev(x).topk(3, dim=0, largest=False)
    rv, _ = x.topk(3, dim=0, largest=False)
    assert torch.equal(v.cpu(), rv)
    assert dev(x).argsort(-1).cpu().shape == x.argsort(-1).shape
    t = torch.tensor([3.0, 1.0, 3.0, 1.0, 2.0])
    assert dev(t).sort(stable=True)[1].cpu().tolist() == [1, 3, 4, 0, 2]


@pytest.mark.parametrize("channels_last", [False, True])
def test_upsample(channels_last):
    torch.manual_seed(5)
    x = torch.randn(2, 8, 7, 5)
    for mode, kw in (("nearest", {}), ("bilinear", {"align_corners": False}), ("bilinear", {"align_corners": True})):
        for size_kw in ({"scale_factor": 2}, {"size": (10, 13)}):
            xr = x.clone().requires_grad_()
            ref = F.interpolate(xr, mode=mode, **size_kw, **kw)
            g = torch.randn_like(ref)
            ref.backward(g)
            xd = dev(x)
            if channels_last:
                xd = xd.contiguous(memory_format=torch.channels_last)
            xd.requires_grad_()
            out = F.interpolate(xd, mode=mode, **size_kw, **kw)
            assert_tensors_equal(out, ref, prec=1e-5, msg=f"{mode} {size_kw}")
            out.backward(dev(g))
            assert_tensors_equal(xd.grad, xr.grad, prec=1e-4, msg=f"{mode} {size_kw} backward")


def test_nms():
    torch.manual_seed(6)
    n = 300
    xy = torch.rand(n, 2) * 100
    wh = torch.rand(n, 2) * 30 + 1
    boxes = torch.cat([xy, xy + wh], 1)
    scores = torch.rand(n)
    keep = torch.ops.catch_b200.nms(dev(boxes), dev(scores), 0.5).cpu()
    ref = torch.ops.catch_b200.nms(boxes, scores, 0.5)  # host implementation of the same op
    assert torch.equal(keep, ref)
    try:
        import torchvision
        assert torch.equal(keep, torchvision.ops.nms(boxes, scores, 0.5))
    except ImportError:
        pass


def test_losses():
    torch.manual_seed(7)
    a, b = torch.randn(6, 10), torch.randn(6, 10)
    p, t = torch.rand(6, 10).clamp(0.01, 0.99), (torch.rand(6, 10) > 0.5).float()
    cases = [
        (lambda x, y, r: F.mse_loss(x, y, reduction=r), a, b),
        (lambda x, y, r: F.smooth_l1_loss(x, y, reduction=r, beta=0.7), a, b),
        (lambda x, y, r: F.huber_loss(x, y, reduction=r, delta=0.6), a, b),
        (lambda x, y, r: F.l1_loss(x, y, reduction=r), a, b),
        (lambda x, y, r: F.binary_cross_entropy(x, y, reduction=r), p, t),
        (lambda x, y, r: F.binary_cross_entropy_with_logits(x, y, reduction=r), a, t),
    ]
    for fn, x, y in cases:
        for r in ("mean", "sum", "none"):
            xr = x.clone().requires_grad_()
            ref = fn(xr, y, r)
            ref.sum().backward()
            xd = dev(x).requires_grad_()
            out = fn(xd, dev(y), r)
            out.sum().backward()
            assert_tensors_equal(out, ref, prec=1e-5)
            assert_tensors_equal(xd.grad, xr.grad, prec=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_depthwise_grouped_transposed_conv(dtype):
    torch.manual_seed(8)
    prec = 2e-2 if dtype == torch.bfloat16 else 3e-3

    def check(xs, ws, fn):
        x = torch.randn(*xs).to(dtype).float()
        w = (torch.randn(*ws) / (ws[1] * ws[2] * ws[3]) ** 0.5).to(dtype).float()
        xr, wr = x.clone().requires_grad_(), w.clone().requires_grad_()
        ref = fn(xr, wr)
        g = torch.randn_like(ref).to(dtype).float()
        ref.backward(g)
        xd = dev(x.to(dtype)).contiguous(memory_format=torch.channels_last).requires_grad_()
        wd = dev(w.to(dtype)).requires_grad_()
        out = fn(xd, wd)
        assert out.device.type == DEV
        assert_tensors_equal(out, ref, prec=prec, use_MSE=True, msg="forward")
        out.backward(dev(g.to(dtype)))
        assert_tensors_equal(xd.grad, xr.grad, prec=prec, use_MSE=True, msg="dx")
        assert_tensors_equal(wd.grad, wr.grad, prec=prec, use_MSE=True, msg="dw")

    check((3, 16, 14, 14), (16, 1, 3, 3), lambda x, w: F.conv2d(x, w, None, 1, 1, 1, 16))          # depthwise
    check((2, 8, 15, 15), (16, 1, 3, 3), lambda x, w: F.conv2d(x, w, None, 2, 1, 1, 8))            # depthwise, multiplier 2
    check((2, 32, 14, 14), (64, 16, 3, 3), lambda x, w: F.conv2d(x, w, None, 1, 1, 1, 2))          # grouped
    check((2, 16, 9, 9), (16, 24, 3, 3), lambda x, w: F.conv_transpose2d(x, w, None, 2, 1, 1))     # transposed, stride 2
    check((2, 16, 9, 9), (16, 8, 4, 4), lambda x, w: F.conv_transpose2d(x, w, None, 1, 0))         # transposed, stride 1
