"""Memory formats of results and operators composed from device kernels.

Results follow the stock rule for memory formats (a convolution result is channels-last when its input or weight is,
else contiguous; batch norm follows its input), so scripts that call ``view()`` on them behave as on other devices
(the classic ``conv -> pool -> x.view(-1, n)`` network, ``group_norm``, ``BatchNorm1d`` on [N, C, L]).  And var / std,
dot, mv, flip, roll, the ELU / hardswish gradients, logit and xlogy run on the device, with the CPU fallback disabled
here so that an unregistered operator fails the test instead of hiding behind it."""
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
    torch.b200.set_flag("op_trycatch", False)
    torch.b200.set_flag("fallback_to_cpu", False)
    yield
    torch.b200.set_flag("op_trycatch", True)
    torch.b200.set_flag("fallback_to_cpu", True)


def test_convolution_and_batch_norm_results_follow_the_input_format():
    torch.manual_seed(0)
    x = torch.randn(4, 8, 12, 12)
    conv = torch.nn.Conv2d(8, 16, 3, padding=1)
    bn = torch.nn.BatchNorm2d(16)
    ref = bn(conv(x))
    conv_d, bn_d = torch.nn.Conv2d(8, 16, 3, padding=1).to(DEV), torch.nn.BatchNorm2d(16).to(DEV)
    conv_d.load_state_dict(conv.state_dict()); bn_d.load_state_dict(bn.state_dict())
    y = conv_d(x.to(DEV))
    assert y.is_contiguous()
    z = bn_d(y)
    assert z.is_contiguous()
    assert_tensors_equal(z, ref, prec=2e-3, use_MSE=True)
    z.view(4, -1)                                          # must not raise
    xc = x.to(DEV).contiguous(memory_format=torch.channels_last)
    yc = conv_d(xc)
    assert yc.is_contiguous(memory_format=torch.channels_last) and not yc.is_contiguous()
    assert bn_d(yc).is_contiguous(memory_format=torch.channels_last)
    conv_d = conv_d.to(memory_format=torch.channels_last)  # a channels-last weight decides as well
    assert conv_d(x.to(DEV)).is_contiguous(memory_format=torch.channels_last)
    # gradients: of a contiguous input contiguous, of a channels-last input channels-last
    for inp in (x.to(DEV), xc):
        inp = inp.clone().requires_grad_()
        conv2 = torch.nn.Conv2d(8, 16, 3, padding=1).to(DEV)
        bn_d(conv2(inp)).square().mean().backward()
        assert inp.grad.stride() == inp.stride()


def test_view_after_convolution_and_pooling_network():
    """The tutorial network: the flattening view() after the last pooling layer needs a contiguous activation."""

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = torch.nn.Conv2d(8, 16, 5)
            self.conv2 = torch.nn.Conv2d(16, 24, 5)
            self.fc = torch.nn.Linear(24 * 4 * 4, 10)

        def forward(self, x):
            x = F.max_pool2d(F.relu(self.conv1(x)), 2)
            x = F.max_pool2d(F.relu(self.conv2(x)), 2)
            return self.fc(x.view(-1, 24 * 4 * 4))

    torch.manual_seed(1)
    net = Net()
    x = torch.randn(6, 8, 28, 28)
    ref = net(x)
    ref.square().mean().backward()
    g_ref = net.conv1.weight.grad.clone()
    net.zero_grad()
    net_d = Net().to(DEV)
    net_d.load_state_dict(net.state_dict())
    out = net_d(x.to(DEV))
    assert_tensors_equal(out, ref, prec=3e-3, use_MSE=True)
    out.square().mean().backward()
    assert_tensors_equal(net_d.conv1.weight.grad, g_ref, prec=3e-3, use_MSE=True)


def test_group_norm_and_batch_norm_1d_on_three_dimensions():
    torch.manual_seed(2)
    x = torch.randn(2, 8, 5, 5)
    w, b = torch.randn(8), torch.randn(8)
    xr = x.clone().requires_grad_()
    ref = F.group_norm(xr, 4, w, b)
    ref.square().sum().backward()
    xd = x.to(DEV).requires_grad_()
    out = F.group_norm(xd, 4, w.to(DEV), b.to(DEV))
    assert_tensors_equal(out, ref, prec=1e-4, use_MSE=True)
    out.square().sum().backward()
    assert_tensors_equal(xd.grad, xr.grad, prec=1e-4, use_MSE=True)
    bn = torch.nn.BatchNorm1d(8)
    seq = torch.randn(4, 8, 20)
    ref = bn(seq)
    bn_d = torch.nn.BatchNorm1d(8).to(DEV)
    got = bn_d(seq.to(DEV))
    assert got.is_contiguous()
    assert_tensors_equal(got.view(4, -1), ref.view(4, -1), prec=1e-4, use_MSE=True)
    conv1d = torch.nn.Conv1d(8, 16, 3, padding=1)
    c_d = torch.nn.Conv1d(8, 16, 3, padding=1).to(DEV)
    c_d.load_state_dict(conv1d.state_dict())
    got = c_d(seq.to(DEV))
    assert got.is_contiguous()
    assert_tensors_equal(got.view(4, -1), conv1d(seq).view(4, -1), prec=3e-3, use_MSE=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_var_std_on_the_device(dtype):
    torch.manual_seed(3)
    prec = 1e-4 if dtype == torch.float32 else 2e-2
    for shape, dims in [((3, 5), [0, 1, (0, 1), None]), ((2, 3, 4, 5), [1, -1, (0, 2), (1, 3), None]), ((1031, 17), [0, 1])]:
        x = torch.randn(shape).to(dtype)
        xd = x.to(DEV)
        for dim in dims:
            for keepdim in (False, True):
                for corr in (1, 0, 2):
                    kw = dict(dim=dim, correction=corr, keepdim=keepdim)
                    assert_tensors_equal(torch.var(xd, **kw), torch.var(x, **kw), prec=prec, use_MSE=True, msg=f"var {shape} {kw}")
                    assert_tensors_equal(torch.std(xd, **kw), torch.std(x, **kw), prec=prec, use_MSE=True, msg=f"std {shape} {kw}")
            v, m = torch.var_mean(xd, dim=dim)
            vr, mr = torch.var_mean(x, dim=dim)
            assert v.dtype == dtype and v.shape == vr.shape and m.shape == mr.shape
            assert_tensors_equal(v, vr, prec=prec, use_MSE=True); assert_tensors_equal(m, mr, prec=prec, use_MSE=True)
            s, m = torch.std_mean(xd, dim=dim, keepdim=True)
            sr, mr = torch.std_mean(x, dim=dim, keepdim=True)
            assert_tensors_equal(s, sr, prec=prec, use_MSE=True); assert_tensors_equal(m, mr, prec=prec, use_MSE=True)
    x = torch.randn(7, 9, dtype=torch.float32).to(dtype).requires_grad_()
    xd = x.detach().to(DEV).requires_grad_()
    x.std(1).sum().backward(); xd.std(1).sum().backward()
    assert_tensors_equal(xd.grad, x.grad, prec=prec, use_MSE=True)
    assert torch.isnan(torch.var(torch.randn(1, 4).to(dtype).to(DEV), dim=0).cpu()).all()   # n - correction == 0


def test_dot_mv_flip_roll_on_the_device():
    torch.manual_seed(4)
    for dtype, prec in [(torch.float32, 2e-3), (torch.bfloat16, 2e-2), (torch.float16, 5e-3)]:
        a, b = torch.randn(257).to(dtype), torch.randn(257).to(dtype)
        assert_tensors_equal(torch.dot(a.to(DEV), b.to(DEV)), torch.dot(a, b), prec=prec * 4, use_MSE=True)
        m, v = torch.randn(33, 65).to(dtype), torch.randn(65).to(dtype)
        assert_tensors_equal(torch.mv(m.to(DEV), v.to(DEV)), torch.mv(m, v), prec=prec, use_MSE=True)
        assert_tensors_equal(torch.matmul(m.to(DEV), v.to(DEV)), m @ v, prec=prec, use_MSE=True)
        c = torch.randn(33).to(dtype)
        assert_tensors_equal(torch.addmv(c.to(DEV), m.to(DEV), v.to(DEV), beta=0.5, alpha=2.0),
                             torch.addmv(c, m, v, beta=0.5, alpha=2.0), prec=prec, use_MSE=True)
    for dtype in (torch.float32, torch.bfloat16, torch.int64, torch.bool):
        x = torch.randn(3, 4, 5).to(dtype) if dtype.is_floating_point else (torch.randn(3, 4, 5) > 0).to(dtype)
        xd = x.to(DEV)
        for dims in ([0], [2], [0, 1], [-1, 0], [0, 1, 2]):
            assert torch.equal(torch.flip(xd, dims).cpu(), torch.flip(x, dims)), (dtype, dims)
        for shifts, dims in [(1, 0), (-2, 2), ((1, 2), (0, 1)), (7, 1), (0, 0)]:
            assert torch.equal(torch.roll(xd, shifts, dims).cpu(), torch.roll(x, shifts, dims)), (dtype, shifts, dims)
        assert torch.equal(torch.roll(xd, 7).cpu(), torch.roll(x, 7))          # flattened
    r = torch.flip(xd, [1])
    assert r.data_ptr() != xd.data_ptr()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_elementwise_composites_on_the_device(dtype):
    torch.manual_seed(5)
    prec = 1e-5 if dtype == torch.float32 else 2e-2
    x = (torch.randn(9, 31) * 3).to(dtype)
    x[0, :4] = torch.tensor([-3.0, 3.0, 0.0, -0.0]).to(dtype)       # the boundaries of the piecewise definitions
    for fn in (F.elu, lambda t: F.elu(t, 0.7), F.selu, F.celu, F.hardswish):
        xr = x.clone().requires_grad_()
        xd = x.to(DEV).requires_grad_()
        fn(xr).square().sum().backward(); fn(xd).square().sum().backward()
        assert_tensors_equal(xd.grad, xr.grad, prec=prec, use_MSE=True)
    xr = x.clone().requires_grad_()
    xd = x.to(DEV).requires_grad_()
    F.elu_(xr.clone()).sum().backward(); F.elu_(xd.clone()).sum().backward()        # gradient from the result
    assert_tensors_equal(xd.grad, xr.grad, prec=prec, use_MSE=True)
    p = torch.rand(9, 31).to(dtype)
    assert_tensors_equal(torch.logit(p.to(DEV), 1e-3), torch.logit(p, 1e-3), prec=prec, use_MSE=True)
    a = torch.randn(9, 31).to(dtype); a[0, :5] = 0
    b = torch.rand(9, 31).to(dtype) + 0.1; b[0, 0] = float("nan"); b[1, 1] = float("nan")
    assert_tensors_equal(torch.xlogy(a.to(DEV), b.to(DEV)), torch.xlogy(a, b), prec=prec, use_MSE=True)
    lg, tg = torch.randn(9, 11).to(dtype), torch.randn(9, 11).to(dtype)
    ref = F.kl_div(F.log_softmax(lg, 1), F.softmax(tg, 1), reduction="batchmean")
    got = F.kl_div(F.log_softmax(lg.to(DEV), 1), F.softmax(tg.to(DEV), 1), reduction="batchmean")
    assert_tensors_equal(got, ref, prec=max(prec, 1e-4) * 4)
