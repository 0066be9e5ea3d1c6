"""Operators that the reference runs on its device and that used to take the CPU fallback here:
3-D pooling, adaptive max pooling, unique, index_fill_, nll_loss2d, linspace, equal, diag, long and
64-bit sorts, dilated / stride-3 / stride-4 and wide-range fp32 convolutions.  Each is checked against
the same PyTorch op on the CPU in the layouts the reference's op tests walk through
(test/cnnl/op_test/test_conv2d.py:27-150): contiguous, channels-last, permuted (non-dense) inputs,
in-place and out= variants where the op has them, and backward."""
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
    torch.b200.set_flag("op_trycatch", False)      # a failing device kernel must not be masked by the CPU fallback
    torch.b200.set_flag("fallback_to_cpu", False)  # nor may an op silently be unregistered
    yield
    torch.b200.set_flag("op_trycatch", True)
    torch.b200.set_flag("fallback_to_cpu", True)


def dev(t):
    return t.to(DEV)


def layouts(x):
    """The same values as a contiguous, a channels-last (4-D / 5-D) and a permuted non-dense tensor."""
    out = [("contiguous", x)]
    if x.dim() == 4:
        out.append(("channels_last", x.contiguous(memory_format=torch.channels_last)))
    if x.dim() == 5:
        out.append(("channels_last_3d", x.contiguous(memory_format=torch.channels_last_3d)))
    big = torch.zeros(*[s * 2 for s in x.shape], dtype=x.dtype)
    sl = tuple(slice(0, 2 * s, 2) for s in x.shape)
    big[sl] = x
    out.append(("strided", big[sl]))
    return out


def fwd_bwd(fn, x_cpu, x_dev, prec=3e-3, check_indices=True, use_MSE=False):
    xr = x_cpu.detach().clone().requires_grad_()
    xd = x_dev.detach().clone().requires_grad_()
    yr, yd = fn(xr), fn(xd)
    outs_r = yr if isinstance(yr, tuple) else (yr,)
    outs_d = yd if isinstance(yd, tuple) else (yd,)
    for a, b in zip(outs_r, outs_d):
        if a.dtype == torch.int64:
            if check_indices:
                assert torch.equal(a, b.cpu())
        else:
            assert_tensors_equal(b, a, prec=prec, use_MSE=use_MSE)
    g = torch.randn_like(outs_r[0])
    outs_r[0].backward(g)
    outs_d[0].backward(g.to(DEV))
    assert_tensors_equal(xd.grad, xr.grad, prec=prec, use_MSE=use_MSE)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pool3d_matrix(dtype):
    torch.manual_seed(0)
    prec = 3e-3 if dtype == torch.float32 else 2e-2
    x = torch.randn(2, 8, 9, 10, 11).to(dtype)
    cases = [
        lambda t: F.max_pool3d(t, 3, 2, 1, return_indices=True),
        lambda t: F.max_pool3d(t, (2, 3, 2), (2, 1, 2), (0, 1, 1), dilation=(1, 2, 1), ceil_mode=True, return_indices=True),
        lambda t: F.avg_pool3d(t, 3, 2, 1),
        lambda t: F.avg_pool3d(t, (2, 3, 2), (1, 2, 2), (1, 1, 0), ceil_mode=True, count_include_pad=False),
        lambda t: F.avg_pool3d(t, 2, divisor_override=3),
        lambda t: F.adaptive_avg_pool3d(t, (4, 3, 5)),
        lambda t: F.adaptive_avg_pool3d(t, 1),
    ]
    for name, xl in layouts(x):
        for i, fn in enumerate(cases):
            # equal values are rare in random floats, so index ties do not arise; bf16 can tie: compare values only
            fwd_bwd(fn, xl.float() if dtype == torch.bfloat16 else xl, dev(xl), prec=prec, check_indices=dtype == torch.float32,
                    use_MSE=dtype != torch.float32)
    # unbatched (4-D) input
    fwd_bwd(lambda t: F.max_pool3d(t, 2, return_indices=True), x[0].float(), dev(x[0].float()))
    fwd_bwd(lambda t: F.avg_pool3d(t, 2), x[0].float(), dev(x[0].float()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_adaptive_max_pool2d_matrix(dtype):
    torch.manual_seed(1)
    prec = 3e-3 if dtype == torch.float32 else 2e-2
    x = torch.randn(3, 16, 13, 9).to(dtype)
    for name, xl in layouts(x):
        for size in [(5, 4), (1, 1), (13, 9), (7, 3)]:
            fwd_bwd(lambda t: F.adaptive_max_pool2d(t, size, return_indices=True), xl.float() if dtype != torch.float32 else xl,
                    dev(xl), prec=prec, check_indices=dtype == torch.float32, use_MSE=dtype != torch.float32)
    fwd_bwd(lambda t: F.adaptive_max_pool2d(t, 3, return_indices=True), x[0].float(), dev(x[0].float()))


@pytest.mark.parametrize("dtype", [torch.int64, torch.float32, torch.int32, torch.bfloat16, torch.uint8, torch.float64])
def test_unique(dtype):
    torch.manual_seed(2)
    x = torch.randint(0, 50, (7, 301)).to(dtype)
    for xl in (x, x.t()):
        for inv, cnt in ((True, True), (False, True), (True, False), (False, False)):
            ref = torch.unique(xl, sorted=True, return_inverse=inv, return_counts=cnt)
            got = torch.unique(dev(xl), sorted=True, return_inverse=inv, return_counts=cnt)
            ref = ref if isinstance(ref, tuple) else (ref,)
            got = got if isinstance(got, tuple) else (got,)
            assert len(ref) == len(got)
            for a, b in zip(ref, got):
                assert torch.equal(a, b.cpu()), (dtype, inv, cnt)
    big = torch.randint(-2 ** 40, 2 ** 40, (300000,))
    big[::7] = big[0]
    v, c = torch.unique(dev(big), return_counts=True)
    vr, cr = torch.unique(big, return_counts=True)
    assert torch.equal(v.cpu(), vr) and torch.equal(c.cpu(), cr)
    assert torch.unique(dev(torch.empty(0))).numel() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64, torch.bool])
def test_index_fill(dtype):
    torch.manual_seed(3)
    x = (torch.randn(4, 6, 5) * 10).to(dtype)
    idx = torch.tensor([4, 0, -1, 2])
    val = True if dtype == torch.bool else -7
    for d in (0, 1, 2, -1):
        i = idx % x.shape[d] if d != 1 else torch.tensor([5, -6, 2])
        assert torch.equal(dev(x).index_fill(d, dev(i), val).cpu(), x.index_fill(d, i, val))
        y, yd = x.clone(), dev(x.clone())
        y.index_fill_(d, i, val); yd.index_fill_(d, dev(i), val)
        assert torch.equal(yd.cpu(), y)
        # permuted (non-contiguous) destination, in place
        z, zd = x.clone().permute(2, 0, 1), dev(x.clone()).permute(2, 0, 1)
        j = torch.tensor([1, 0])
        z.index_fill_(d, j, val); zd.index_fill_(d, dev(j), val)
        assert torch.equal(zd.cpu(), z)
    s, sd = x.clone(), dev(x.clone())
    s.index_fill_(0, torch.tensor(2), torch.tensor(3, dtype=dtype) if dtype != torch.bool else torch.tensor(True))
    sd.index_fill_(0, dev(torch.tensor(2)), dev(torch.tensor(3, dtype=dtype) if dtype != torch.bool else torch.tensor(True)))
    assert torch.equal(sd.cpu(), s)


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_nll_loss2d(reduction):
    torch.manual_seed(4)
    x = torch.randn(3, 7, 5, 6)
    t = torch.randint(0, 7, (3, 5, 6))
    t[0, 0, :3] = -100
    w = torch.rand(7) + 0.5
    for name, xl in layouts(x):
        for weight in (None, w):
            xr = F.log_softmax(xl, 1).detach().requires_grad_()
            xd = dev(xr.detach()).requires_grad_()
            lr_ = F.nll_loss(xr, t, weight, reduction=reduction)
            ld_ = F.nll_loss(xd, dev(t), None if weight is None else dev(weight), reduction=reduction)
            assert_tensors_equal(ld_, lr_, prec=1e-4, msg=name)
            g = torch.randn_like(lr_)
            lr_.backward(g); ld_.backward(dev(g))
            assert_tensors_equal(xd.grad, xr.grad, prec=1e-5, msg=name)
    # whole segmentation loss through cross_entropy
    xr = x.clone().requires_grad_(); xd = dev(x).requires_grad_()
    F.cross_entropy(xr, t).backward(); F.cross_entropy(xd, dev(t)).backward()
    assert_tensors_equal(xd.grad, xr.grad, prec=1e-5)


def test_linspace_equal_diag_cumsum():
    for dtype in (torch.float32, torch.float64, torch.bfloat16, torch.int64):
        for args in ((0, 1, 11), (-3, 7, 50), (5, 5, 1), (2, -2, 4), (0, 10, 0), (0, 100, 1001)):
            ref = torch.linspace(*args, dtype=dtype)
            got = torch.linspace(*args, dtype=dtype, device=DEV)
            assert_tensors_equal(got, ref, prec={torch.float32: 1e-5, torch.float64: 1e-9, torch.bfloat16: 0.5}.get(dtype, 0))
    out = torch.empty(9, device=DEV)
    torch.linspace(1, 2, 9, out=out)
    assert_tensors_equal(out, torch.linspace(1, 2, 9), prec=1e-6)
    a = torch.randn(5, 6)
    assert torch.equal(dev(a), dev(a.clone())) and not torch.equal(dev(a), dev(a + 1))
    assert not torch.equal(dev(a), dev(a[:4])) and torch.equal(dev(a).t(), dev(a.t().contiguous()))
    assert torch.equal(dev(torch.empty(0, 3)), dev(torch.empty(0, 3)))
    v = torch.randn(7)
    m = torch.randn(6, 8)
    for k in (0, 2, -1):
        assert torch.equal(torch.diag(dev(v), k).cpu(), torch.diag(v, k))
        assert torch.equal(torch.diag(dev(m), k).cpu(), torch.diag(m, k))
        assert torch.equal(torch.diag(dev(m).t(), k).cpu(), torch.diag(m.t(), k))
    i = torch.randint(0, 5, (100000,))
    assert torch.equal(torch.cumsum(dev(i), 0).cpu(), torch.cumsum(i, 0))
    assert torch.equal(torch.cumsum(dev(i > 2), 0).cpu(), torch.cumsum(i > 2, 0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.int64, torch.float64, torch.bfloat16, torch.int32])
def test_long_and_wide_sorts(dtype):
    torch.manual_seed(5)
    for shape, dim in (((3, 5000), 1), ((70000,), 0), ((4100, 3), 0), ((2, 3, 9000), -1)):
        if dtype.is_floating_point:
            x = torch.randn(shape).to(dtype)
        else:
            x = torch.randint(-2 ** 40 if dtype == torch.int64 else -2 ** 30, 2 ** 40 if dtype == torch.int64 else 2 ** 30, shape).to(dtype)
        for desc in (False, True):
            vr, ir = torch.sort(x, dim=dim, descending=desc, stable=True)
            vd, idd = torch.sort(dev(x), dim=dim, descending=desc, stable=True)
            assert torch.equal(vd.cpu(), vr)
            assert torch.equal(idd.cpu(), ir)          # stable: ties keep their order
            k = min(37, x.shape[dim])
            tv, ti = torch.topk(dev(x), k, dim=dim, largest=desc)
            tr, _ = torch.topk(x, k, dim=dim, largest=desc)
            assert torch.equal(tv.cpu(), tr)
            assert torch.equal(torch.gather(x, dim, ti.cpu()), tr)
    nan = torch.tensor([1.0, float("nan"), -2.0] * 2000)
    assert torch.equal(torch.sort(dev(nan)).values.cpu().isnan(), torch.sort(nan).values.isnan())
    # 64-bit integers that a float key could not tell apart
    close = torch.tensor([2 ** 53 + 1, 2 ** 53, 2 ** 53 + 2, -2 ** 62, 2 ** 62])
    assert torch.equal(torch.sort(dev(close)).values.cpu(), torch.sort(close).values)


CONV_CASES = [
    # (N, C, H, W, K, R, S, stride, padding, dilation)
    (2, 16, 20, 18, 32, 3, 3, (1, 1), (2, 2), (2, 2)),
    (2, 16, 20, 18, 32, 3, 3, (2, 2), (3, 3), (3, 3)),
    (2, 16, 21, 19, 24, 3, 3, (3, 3), (1, 1), (1, 1)),
    (2, 8, 22, 23, 16, 5, 3, (4, 3), (2, 1), (1, 1)),
    (2, 16, 17, 17, 16, 3, 3, (2, 1), (2, 2), (1, 2)),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", CONV_CASES)
def test_dilated_and_large_stride_convolutions(case, dtype):
    torch.manual_seed(6)
    N, C, H, W, K, R, S, stride, padding, dilation = case
    x = torch.randn(N, C, H, W)
    w = torch.randn(K, C, R, S) / (C * R * S) ** 0.5
    b = torch.randn(K)
    prec = 3e-3 if dtype == torch.float32 else 2e-2
    for name, xl in layouts(x):
        xr = xl.detach().clone().requires_grad_()
        wr = w.clone().requires_grad_()
        xd = dev(xl.to(dtype)).requires_grad_()
        wd = dev(w.to(dtype)).requires_grad_()
        yr = F.conv2d(xr, wr, b, stride, padding, dilation)
        yd = F.conv2d(xd, wd, dev(b.to(dtype)), stride, padding, dilation)
        assert_tensors_equal(yd.float(), yr, prec=prec, use_MSE=True, msg=name)
        g = torch.randn_like(yr)
        yr.backward(g); yd.backward(dev(g.to(dtype)))
        assert_tensors_equal(xd.grad.float(), xr.grad, prec=prec, use_MSE=True, msg=name + " dx")
        assert_tensors_equal(wd.grad.float(), wr.grad, prec=prec, use_MSE=True, msg=name + " dw")


def test_fp32_convolution_keeps_fp32_range_and_precision():
    """fp32 convolutions run as split-bf16 tensor-core passes: values far outside fp16's range must survive and
    the result must be much closer to the fp64 reference than a 10-bit-mantissa computation would be."""
    torch.manual_seed(7)
    x = torch.randn(2, 16, 12, 12)
    w = torch.randn(32, 16, 3, 3) / 12.0
    for xs, ws in ((1e6, 1.0), (1e-9, 1e-3), (3e4, 3e4), (1.0, 1.0)):
        xr, wr = (x * xs).double().requires_grad_(), (w * ws).double().requires_grad_()
        xd, wd = dev(x * xs).requires_grad_(), dev(w * ws).requires_grad_()
        yr = F.conv2d(xr, wr, None, 1, 1)
        yd = F.conv2d(xd, wd, None, 1, 1)
        assert torch.isfinite(yd).all()
        assert_tensors_equal(yd, yr, prec=2e-4, use_MSE=True, msg=f"scales {xs} {ws}")
        g = torch.randn_like(yr)
        yr.backward(g); yd.backward(dev(g.float()))
        assert_tensors_equal(xd.grad, xr.grad, prec=2e-4, use_MSE=True, msg="dx")
        assert_tensors_equal(wd.grad, wr.grad, prec=2e-4, use_MSE=True, msg="dw")
    # transposed convolution with dilation and a stride of 3
    xt = torch.randn(2, 16, 7, 6)
    wt = torch.randn(16, 8, 3, 3) / 12.0
    yr = F.conv_transpose2d(xt, wt, None, 3, 1, 1, 1, 2)
    yd = F.conv_transpose2d(dev(xt), dev(wt), None, 3, 1, 1, 1, 2)
    assert_tensors_equal(yd, yr, prec=2e-4, use_MSE=True)


def test_out_variants_and_dim_reductions():
    """out= overloads of the reference's list (gather.out, index_select.out, topk.values, max.dim_max,
    sum.IntList_out, mean.out, ...) and the reductions along one dimension that used to fall back (all / any / prod /
    norm with a dtype): device result against the CPU result, with out tensors that have to be resized."""
    torch.manual_seed(0)
    x = torch.randn(6, 10, 5)
    xd = dev(x)
    idx = torch.randint(0, 10, (6, 4, 5))
    cases = [
        ("gather", lambda t, o: torch.gather(t, 1, idx.to(t.device), out=o)),
        ("index_select", lambda t, o: torch.index_select(t, 1, torch.tensor([7, 0, 3]).to(t.device), out=o)),
        ("sum", lambda t, o: torch.sum(t, (0, 2), out=o)),
        ("mean", lambda t, o: torch.mean(t, 1, keepdim=True, out=o)),
        ("prod", lambda t, o: torch.prod(t, 2, out=o)),
        ("clamp_min", lambda t, o: torch.clamp_min(t, 0.25, out=o)),
        ("leaky_relu", lambda t, o: F.leaky_relu(t, 0.1) if o is None else torch._C._nn.leaky_relu(t, 0.1, out=o)),
        ("threshold", lambda t, o: torch.threshold(t, 0.1, -1.0) if o is None else torch.threshold(t, 0.1, -1.0, out=o)),
        ("masked_select", lambda t, o: torch.masked_select(t, t > 0.3, out=o)),
        ("nonzero", lambda t, o: torch.nonzero(t > 1.0, out=o)),
    ]
    for name, fn in cases:
        ref = fn(x, None)
        out = torch.empty(0, dtype=ref.dtype, device=DEV)
        got = fn(xd, out)
        assert got.data_ptr() == out.data_ptr(), name
        assert_tensors_equal(out.cpu().float(), ref.float(), prec=1e-5), name
    # two-result overloads
    v, i = torch.empty(0, device=DEV), torch.empty(0, dtype=torch.long, device=DEV)
    torch.max(xd, 1, out=(v, i))
    rv, ri = torch.max(x, 1)
    assert torch.equal(v.cpu(), rv) and torch.equal(i.cpu(), ri)
    torch.topk(xd, 3, dim=1, out=(v, i))
    rv, ri = torch.topk(x, 3, dim=1)
    assert torch.equal(v.cpu(), rv) and torch.equal(i.cpu(), ri)
    # reductions along one dimension
    b = x > 0.5
    assert torch.equal(dev(b).all(1).cpu(), b.all(1)) and torch.equal(dev(b).any(2, keepdim=True).cpu(), b.any(2, keepdim=True))
    o = torch.empty(0, dtype=torch.bool, device=DEV)
    torch.all(dev(b), 0, out=o)
    assert torch.equal(o.cpu(), b.all(0))
    assert_tensors_equal(xd[:, :3].prod().cpu(), x[:, :3].prod(), prec=1e-4, use_MSE=True)
    assert_tensors_equal(torch.norm(xd.half(), 2, [1], dtype=torch.float32).cpu(), torch.norm(x.half(), 2, [1], dtype=torch.float32),
                         prec=1e-3, use_MSE=True)
    y = xd.abs().clone()
    y.pow_(2.0)
    assert_tensors_equal(y.cpu(), x.abs().pow(2.0), prec=1e-5)
    # pooling / resampling / loss out= forms
    img = torch.randn(2, 8, 12, 12)
    o = torch.empty(0, device=DEV)
    torch._C._nn.adaptive_avg_pool2d(dev(img), (3, 3), out=o)
    assert_tensors_equal(o.cpu(), F.adaptive_avg_pool2d(img, (3, 3)), prec=1e-5)
    torch._C._nn.upsample_nearest2d(dev(img), (24, 24), out=o)
    assert_tensors_equal(o.cpu(), F.interpolate(img, size=(24, 24), mode="nearest"), prec=1e-6)
    torch._C._nn.upsample_bilinear2d(dev(img), (18, 18), False, out=o)
    assert_tensors_equal(o.cpu(), F.interpolate(img, size=(18, 18), mode="bilinear", align_corners=False), prec=1e-5)
    p, t = torch.rand(4, 7), torch.rand(4, 7)
    torch._C._nn.binary_cross_entropy(dev(p), dev(t), None, 1, out=o)
    assert_tensors_equal(o.cpu(), F.binary_cross_entropy(p, t), prec=1e-5)
    torch._C._nn.smooth_l1_loss(dev(p), dev(t), 1, 0.5, out=o)
    assert_tensors_equal(o.cpu(), F.smooth_l1_loss(p, t, beta=0.5), prec=1e-5)


def test_short_reductions_with_many_outputs():
    """Global average pooling over a channels-last tensor (mean over H, W: 49 elements per output, many outputs) and
    its relatives take the one-thread-per-output reduction kernel."""
    torch.manual_seed(0)
    x = torch.randn(64, 256, 7, 7)
    xc = x.contiguous(memory_format=torch.channels_last)
    for t in (x, xc):
        td = dev(t)
        assert_tensors_equal(td.mean((2, 3)).cpu(), t.mean((2, 3)), prec=1e-5)
        assert_tensors_equal(td.sum((2, 3), keepdim=True).cpu(), t.sum((2, 3), keepdim=True), prec=1e-4)
        assert_tensors_equal(td.amax((2, 3)).cpu(), t.amax((2, 3)), prec=0)
        v, i = td.flatten(2).max(2)
        rv, ri = t.flatten(2).max(2)
        assert torch.equal(v.cpu(), rv) and torch.equal(i.cpu(), ri)
    xb = xc.bfloat16()
    assert_tensors_equal(F.adaptive_avg_pool2d(dev(xb), 1).float().cpu(), F.adaptive_avg_pool2d(xb.float(), 1), prec=1e-2,
                         use_MSE=True)
    y = torch.randn(40000, 33)  # reduce the short inner dimension: outputs are not adjacent in memory -> other kernel
    assert_tensors_equal(dev(y).sum(1).cpu(), y.sum(1), prec=1e-4)
    assert_tensors_equal(dev(y.t().contiguous()).sum(0).cpu(), y.sum(1), prec=1e-4)


@pytest.mark.parametrize("cols", [1030, 4096, 30522])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_softmax_and_cross_entropy_with_rows_cached_in_shared_memory(cols, dtype):
    """Rows of 1024 columns and more are staged in shared memory (one read, 16-byte accesses); 1030 and 30522 columns
    give rows that do not start on 16-byte boundaries."""
    torch.manual_seed(0)
    rows = 37
    x = (torch.randn(rows, cols) * 3).to(dtype)
    t = torch.randint(0, cols, (rows,))
    t[3] = -100
    xd, td = dev(x), dev(t)
    prec = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert_tensors_equal(torch.softmax(xd, -1).float().cpu(), torch.softmax(x.float(), -1), prec=prec, use_MSE=True)
    assert_tensors_equal(torch.log_softmax(xd, -1).float().cpu(), torch.log_softmax(x.float(), -1), prec=prec, use_MSE=True)
    for smooth in (0.0, 0.1):
        xr = x.float().clone().requires_grad_()
        ref = F.cross_entropy(xr, t, label_smoothing=smooth)
        ref.backward()
        loss, grad = torch.ops.catch_b200.softmax_cross_entropy(xd, td, -100, smooth)  # (mean loss, d loss / d logits)
        assert abs(loss.item() - ref.item()) < 1e-3 * abs(ref.item()), (loss.item(), ref.item())
        assert_tensors_equal(grad.float().cpu(), xr.grad, prec=prec, use_MSE=True, msg=f"smooth {smooth}")
