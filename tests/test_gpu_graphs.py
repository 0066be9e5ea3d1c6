"""Device graphs on a real B200: capture / replay of a queue, graphed callables, fusion groups replayed as graphs,
and the fused quantized convolution (int8 in, int8 out) against a floating-point reference."""
import pytest
import torch
import torch.nn.functional as F

import catch_b200  # noqa: F401
from catch_b200 import jit
from common import assert_tensors_equal

pytestmark = pytest.mark.gpu
DEV = "blackwell"


def test_capture_and_replay_a_queue():
    bw = torch.b200
    assert bw.graphs_supported()
    x = torch.randn(256, 256, device=DEV)
    w = torch.randn(256, 256, device=DEV)
    g = bw.Graph()
    with bw.graph(g):
        y = torch.relu(x @ w) + 1.0
    assert g.valid and g.num_nodes >= 2
    g.replay()
    bw.synchronize()
    ref = torch.relu(x.cpu() @ w.cpu()) + 1.0
    assert_tensors_equal(y.cpu(), ref, prec=2e-2, use_MSE=True)
    x.copy_(torch.randn(256, 256))
    g.replay()
    assert_tensors_equal(y.cpu(), torch.relu(x.cpu() @ w.cpu()) + 1.0, prec=2e-2, use_MSE=True)
    # memory of the graph stays out of the shared cache until the graph is reset
    ptr = y.data_ptr()
    other = [torch.empty_like(y) for _ in range(8)]
    assert all(o.data_ptr() != ptr for o in other)
    del other
    g.reset()
    assert not g.valid


def test_capture_that_waits_for_the_device_is_refused_and_leaves_the_device_usable():
    bw = torch.b200
    x = torch.ones(16, device=DEV)
    g = bw.Graph()
    with pytest.raises(RuntimeError):
        with bw.graph(g):
            y = x * 2
            y.sum().item()  # a host read: not recordable
    assert not g.valid
    assert (x * 3).sum().item() == 48.0  # ordinary work still runs


def test_graphed_callable_matches_eager():
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Conv2d(16, 32, 3, padding=1), torch.nn.ReLU(), torch.nn.Conv2d(32, 32, 1),
                            torch.nn.AdaptiveAvgPool2d(1), torch.nn.Flatten(), torch.nn.Linear(32, 10)).eval()
    m = m.half().to(DEV).to(memory_format=torch.channels_last)
    x = torch.randn(8, 16, 20, 20).half().to(DEV).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        ref = m(x).float().cpu()
        fast = torch.b200.make_graphed_callable(m, (x,))
        assert fast.graph.valid
        for _ in range(3):
            x2 = torch.randn(8, 16, 20, 20).half().to(DEV).contiguous(memory_format=torch.channels_last)
            assert_tensors_equal(fast(x2).float().cpu(), m(x2).float().cpu(), prec=1e-3, use_MSE=True)
        assert_tensors_equal(fast(x).float().cpu(), ref, prec=1e-3, use_MSE=True)
    with pytest.raises(ValueError):
        fast(x[:4])


class Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.c1 = torch.nn.Conv2d(32, 32, 3, padding=1, bias=False); self.b1 = torch.nn.BatchNorm2d(32)
        self.c2 = torch.nn.Conv2d(32, 32, 3, padding=1, bias=False); self.b2 = torch.nn.BatchNorm2d(32)
        self.fc = torch.nn.Linear(32, 10)

    def forward(self, x):
        y = torch.relu(self.b1(self.c1(x)))
        y = torch.relu(self.b2(self.c2(y)) + x)
        return self.fc(y.mean((2, 3)))


def test_fused_fp16_block_matches_eager_and_replays_as_a_graph():
    """Reference test strategy: fusion-mode output against eager (test/magicmind/op_test/*): here also through the
    device-graph path that fusion groups take from their third call."""
    torch.manual_seed(0)
    m = Block().eval()
    for bn in (m.b1, m.b2):
        bn.running_mean.normal_(); bn.running_var.uniform_(0.5, 2.0)
    x = torch.randn(16, 32, 28, 28)
    ref = m(x)
    md = m.half().to(DEV).to(memory_format=torch.channels_last)
    xd = x.half().to(DEV).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        opt = jit.optimize(torch.jit.trace(md, xd))
        before = jit.fusion_stats()
        outs = [opt(xd).float().cpu() for _ in range(5)]
        after = jit.fusion_stats()
    assert "catch_b200::FusionGroup" in str(opt.graph)
    for o in outs:
        assert_tensors_equal(o, ref, prec=2e-2, use_MSE=True)
    assert after["graph_captures"] >= before["graph_captures"] + 1
    assert after["graph_replays"] >= before["graph_replays"] + 2
    assert after["fallbacks"] == before["fallbacks"]
    with torch.no_grad():
        x2 = torch.randn(16, 32, 28, 28)
        assert_tensors_equal(opt(x2.half().to(DEV).contiguous(memory_format=torch.channels_last)).float().cpu(),
                             m.float().cpu()(x2), prec=2e-2, use_MSE=True)


@pytest.mark.parametrize("stride", [1, 2])
def test_fused_quantized_conv_int8_in_int8_out(stride):
    """catch_b200::qconv_act on the device: int8 input quantized by the producer, residual + ReLU in the epilogue,
    int8 output quantized for the consumer -- against the same arithmetic in fp32."""
    torch.manual_seed(1)
    N, C, K, H = 4, 64, 96, 14
    x = torch.randn(N, C, H, H)
    w = torch.randn(K, C, 3, 3) * 0.05
    b = torch.randn(K) * 0.1
    s_in = 127.0 / x.abs().max().item()
    xq = torch.clamp(torch.round(x * s_in), -127, 127)
    P = (H + 2 - 3) // stride + 1
    res = torch.randn(N, K, P, P)
    s_out = 20.0
    scale = torch.tensor([s_in, 1.0])
    mode = torch.tensor([3])  # per-channel weights
    # reference: fake-quantized operands, fp32 accumulation
    amax = w.reshape(K, -1).abs().amax(1).clamp_min(1e-30)
    sw = (127.0 / amax).view(K, 1, 1, 1)
    wq = torch.clamp(torch.round(w * sw), -127, 127) / sw
    y = F.conv2d(xq / s_in, wq, b, stride=stride, padding=1)
    y_relu = torch.relu(y + res.half().float())
    ref_q = torch.clamp(torch.round(y_relu * s_out), -127, 127)

    cl = torch.channels_last
    xd = xq.to(torch.int8).to(DEV).contiguous(memory_format=cl)
    args = (w.half().to(DEV), b.half().to(DEV), [1, 1], [stride, stride], [1, 1], 1, scale.to(DEV), mode.to(DEV))
    out_f = torch.ops.catch_b200.qconv_act(xd, *args, res.half().to(DEV).contiguous(memory_format=cl), 1, 0.0)
    assert out_f.dtype == torch.float16
    assert_tensors_equal(out_f.float().cpu(), y_relu, prec=5e-3, use_MSE=True)
    out_q = torch.ops.catch_b200.qconv_act(xd, *args, res.half().to(DEV).contiguous(memory_format=cl), 1, s_out)
    assert out_q.dtype == torch.int8 and out_q.shape == (N, K, P, P)
    diff = (out_q.cpu().float() - ref_q).abs()
    assert diff.max().item() <= 1.0 and (diff > 0).float().mean().item() < 0.05  # rounding ties only
    # floating-point input: quantized inside, same result as the pre-quantized path
    out_f2 = torch.ops.catch_b200.qconv_act((xq / s_in).half().to(DEV).contiguous(memory_format=cl), *args, None, 0, 0.0)
    assert_tensors_equal(out_f2.float().cpu(), y, prec=5e-3, use_MSE=True)
