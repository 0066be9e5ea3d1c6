"""The backend on a real B200: allocation, copies, element-wise kernels, mm."""
import pytest
import torch

from common import assert_tensors_equal

pytestmark = pytest.mark.gpu
DEV = "blackwell"


@pytest.fixture(scope="module", autouse=True)
def _backend():
    import catch_b200  # noqa: F401

    assert torch.b200.backend_name() == "cuda", "GPU tests must run on the CUDA backend, not the host simulation"
    yield


def test_roundtrip_and_stats():
    x = torch.randn(1000, 33)
    before = torch.b200.memory_allocated()
    y = x.to(DEV)
    assert torch.b200.memory_allocated() > before
    assert torch.equal(y.cpu(), x)
    z = y.t()[::2]
    assert torch.equal(z.cpu(), x.t()[::2])
    assert torch.equal(y.to(torch.float64).cpu(), x.double())
    assert torch.equal(y.to(torch.bfloat16).cpu(), x.bfloat16())
    props = torch.b200.get_device_properties(0)
    assert props.major == 10 and props.multi_processor_count > 100


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int64, torch.float64])
def test_binary_ops(dtype):
    torch.manual_seed(0)
    a = (torch.randn(64, 1, 37) * 4).to(dtype)
    b = (torch.randn(1, 5, 37) * 4).to(dtype)
    b = torch.where(b == 0, torch.ones_like(b), b)
    da, db = a.to(DEV), b.to(DEV)
    prec = 2e-2 if dtype in (torch.bfloat16, torch.float16) else 1e-5
    for fn in (torch.add, torch.sub, torch.mul, torch.maximum, torch.minimum):
        assert_tensors_equal(fn(da, db), fn(a, b), prec=prec, use_MSE=True, msg=fn.__name__)
    assert_tensors_equal(torch.add(da, db, alpha=2), torch.add(a, b, alpha=2), prec=prec, use_MSE=True)
    assert_tensors_equal(da / db, a / b, prec=prec, use_MSE=True)
    assert_tensors_equal(da * 3, a * 3, prec=prec, use_MSE=True)
    for fn in (torch.eq, torch.lt, torch.ge):
        assert torch.equal(fn(da, db).cpu(), fn(a, b))
    c = (da + torch.zeros_like(db)).clone()
    c += db
    assert_tensors_equal(c, a + b, prec=prec, use_MSE=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unary_and_activations(dtype):
    torch.manual_seed(1)
    x = torch.randn(3, 1000).to(dtype)
    d = x.to(DEV)
    prec = 2e-2 if dtype == torch.bfloat16 else 1e-5
    fns = [torch.relu, torch.sigmoid, torch.tanh, torch.exp, torch.neg, torch.abs,
           torch.nn.functional.gelu, torch.nn.functional.silu, lambda t: torch.clamp(t, -0.5, 0.5),
           lambda t: torch.nn.functional.leaky_relu(t, 0.1), lambda t: torch.nn.functional.softplus(t),
           lambda t: torch.nn.functional.hardtanh(t), lambda t: t.abs().sqrt(), lambda t: (t.abs() + 1).log()]
    for i, fn in enumerate(fns):
        assert_tensors_equal(fn(d), fn(x.float()).to(dtype), prec=prec, use_MSE=True, msg=f"fn{i}")
    # gradients of activations
    for fn in (torch.relu, torch.nn.functional.gelu, torch.tanh, torch.sigmoid):
        xr = x.float().clone().requires_grad_()
        dr = x.float().to(DEV).requires_grad_()
        fn(xr).sum().backward()
        fn(dr).sum().backward()
        assert_tensors_equal(dr.grad, xr.grad, prec=1e-4, use_MSE=True)


def test_fill_where_masked():
    x = torch.randn(17, 19)
    d = x.to(DEV)
    assert torch.equal(torch.zeros_like(d).cpu(), torch.zeros(17, 19))
    assert torch.equal(torch.full((5,), 3.5, device=DEV).cpu(), torch.full((5,), 3.5))
    assert torch.equal(torch.where(d > 0, d, -d).cpu(), x.abs())
    assert torch.equal(d.masked_fill(d < 0, 0.0).cpu(), x.clamp_min(0))
    assert_tensors_equal(torch.addcmul(d, d, d, value=2), torch.addcmul(x, x, x, value=2), prec=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_mm_addmm_bmm(dtype):
    torch.manual_seed(2)
    a, b = torch.randn(130, 72).to(dtype), torch.randn(72, 200).to(dtype)
    bias = torch.randn(200).to(dtype)
    da, db, dbias = a.to(DEV), b.to(DEV), bias.to(DEV)
    prec = 2e-2 if dtype == torch.bfloat16 else 3e-3
    assert_tensors_equal(da @ db, a.float() @ b.float(), prec=prec, use_MSE=True)
    assert_tensors_equal(torch.addmm(dbias, da, db), torch.addmm(bias.float(), a.float(), b.float()), prec=prec, use_MSE=True)
    assert_tensors_equal(da.t().contiguous().t() @ db, a.float() @ b.float(), prec=prec, use_MSE=True)
    assert_tensors_equal(db.t() @ da.t(), (a.float() @ b.float()).t(), prec=prec, use_MSE=True)
    x, y = torch.randn(6, 50, 64).to(dtype), torch.randn(6, 64, 40).to(dtype)
    assert_tensors_equal(torch.bmm(x.to(DEV), y.to(DEV)), torch.bmm(x.float(), y.float()), prec=prec, use_MSE=True)
    lin = torch.nn.Linear(72, 200).to(dtype)
    dl = torch.nn.Linear(72, 200).to(dtype)
    dl.load_state_dict(lin.state_dict())
    dl = dl.to(DEV)
    xr = a.clone().requires_grad_()
    xd = a.to(DEV).requires_grad_()
    lin(xr).float().pow(2).sum().backward()
    dl(xd).float().pow(2).sum().backward()
    assert_tensors_equal(xd.grad, xr.grad, prec=prec, use_MSE=True)
    assert_tensors_equal(dl.weight.grad, lin.weight.grad, prec=prec, use_MSE=True)


def test_queues_and_notifiers():
    q = torch.b200.current_queue()
    start, end = torch.b200.Notifier(), torch.b200.Notifier()
    start.place(q)
    x = torch.randn(1 << 20).to(DEV)
    for _ in range(10):
        x = x * 1.0001
    end.place(q)
    end.synchronize()
    assert start.elapsed_time(end) > 0
    with torch.b200.Queue() as side:
        assert torch.b200.current_queue() == side
        y = x + 1
    side.synchronize()
    assert_tensors_equal(y, x.cpu() + 1, prec=1e-6)


def test_profiler_lists_kernels_with_device_times(tmp_path):
    """The profiler preset records operators through the stock profiler and, next to them, every kernel launch with a
    positive device time; the Chrome trace gets a device row per queue."""
    import json

    from catch_b200 import profiler

    x = torch.randn(512, 512, device=DEV)
    w = torch.randn(512, 512, device=DEV)
    torch.b200.synchronize()
    with profiler.profile(record_shapes=True) as prof:
        with profiler.range("step"):
            y = torch.relu(x @ w)
            profiler.mark("after relu")
            z = y.sum()
    assert z.device.type == DEV
    assert {"aten::mm", "aten::relu"} <= {e.name for e in prof.function_events}
    mm = [e for e in prof.function_events if e.name == "aten::mm"]
    assert mm and mm[0].device_time > 0                      # operator-level device time from the stock profiler
    kt = prof.kernels
    names = [e.name for e in kt.kernels]
    assert "b200_gemm" in names and any(n.startswith("b200_elementwise") or "reduce" in n for n in names), names
    assert all(e.dur_us > 0 for e in kt.kernels)
    assert all(e.op for e in kt.kernels)                     # each launch knows the operator that issued it
    gemm = next(e for e in kt.kernels if e.name == "b200_gemm")
    assert gemm.op == "gemm" and gemm.start_us >= 0
    rng = [e for e in kt.events if e.kind == "range"]
    assert len(rng) == 1 and rng[0].name == "step" and rng[0].dur_us >= sum(e.dur_us for e in kt.kernels) * 0.5
    assert [e.name for e in kt.events if e.kind == "mark"] == ["after relu"]
    assert "b200_gemm" in kt.table() and kt.total_device_time_us() > 0
    path = str(tmp_path / "trace.json")
    prof.export_chrome_trace(path)
    events = json.load(open(path))["traceEvents"]
    assert any(e.get("pid") == "blackwell:0" and e.get("name") == "b200_gemm" and e.get("dur", 0) > 0 for e in events)
    # outside a trace nothing is recorded and launches cost nothing extra
    with profiler.kernel_trace() as kt2:
        pass
    assert kt2.events == []
