"""Behaviours first met on the host-simulated device, checked on a real B200: batch norm's host path, LSTM / GRU
through the composed fused cells, arguments left on the host, int32 indices, an in-place activation behind a fused
batch norm.  The file sorts behind the kernel suites on purpose: they run first under ``pytest -x``."""
import copy

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


def test_batch_norm_with_a_channel_count_that_takes_the_host_path_updates_its_statistics():
    """Five channels have no device kernel (vectors of four / eight channels): the operator runs on the host, and the
    running statistics it updates there have to arrive in the module's buffers on the device."""
    torch.manual_seed(0)
    bn, ref = torch.nn.BatchNorm2d(5).to(DEV).train(), torch.nn.BatchNorm2d(5).train()
    for _ in range(3):
        x = torch.randn(8, 5, 6, 6) * 2 + 3
        a, b = bn(x.to(DEV)), ref(x)
        assert torch.allclose(a.cpu(), b, atol=1e-4)
    assert torch.allclose(bn.running_mean.cpu(), ref.running_mean, atol=1e-5)
    assert torch.allclose(bn.running_var.cpu(), ref.running_var, atol=1e-4)
    assert int(bn.num_batches_tracked) == 3


def test_lstm_and_gru_on_the_device():
    """nn.LSTM / nn.GRU: the fused-cell operators torch calls on non-CPU devices are composed from this backend's
    element-wise kernels (fp32 matrix products run as TF32, hence the tolerance)."""
    import copy

    torch.manual_seed(0)
    for ctor in (lambda: torch.nn.LSTM(16, 32, num_layers=2, batch_first=True, bidirectional=True), lambda: torch.nn.GRU(16, 32, batch_first=True)):
        ref = ctor()
        dev = copy.deepcopy(ref).to(DEV)
        x = torch.randn(4, 10, 16)
        xr, xd = x.clone().requires_grad_(), x.to(DEV).requires_grad_()
        o_ref, _ = ref(xr)
        o_dev, _ = dev(xd)
        assert_tensors_equal(o_dev, o_ref, prec=2e-2, use_MSE=True)
        o_ref.square().sum().backward()
        o_dev.square().sum().backward()
        assert_tensors_equal(xd.grad, xr.grad, prec=5e-2, use_MSE=True)
        for p, q in zip(ref.parameters(), dev.parameters()):
            assert_tensors_equal(q.grad, p.grad, prec=5e-2, use_MSE=True)


def test_an_argument_on_the_host_raises_instead_of_reaching_a_kernel():
    w = torch.randn(3, 4, device=DEV)
    for fn in (lambda: torch.randn(2, 3) @ w, lambda: torch.nn.functional.embedding(torch.tensor([1]), w),
               lambda: torch.nn.functional.nll_loss(w, torch.tensor([1, 2, 3])),
               lambda: torch.nn.functional.conv2d(torch.randn(1, 3, 8, 8, device=DEV), torch.randn(4, 3, 3, 3)),
               lambda: torch.nn.BatchNorm2d(4).to(DEV)(torch.randn(2, 4, 3, 3))):
        with pytest.raises(RuntimeError, match="same device"):
            fn()


def test_embedding_and_index_select_take_int32_indices():
    w = torch.randn(10, 6)
    idx = torch.tensor([[1, 9], [0, 3]], dtype=torch.int32)
    dw = w.to(DEV).requires_grad_()
    out = torch.nn.functional.embedding(idx.to(DEV), dw)
    assert torch.equal(out.detach().cpu(), torch.nn.functional.embedding(idx, w))
    out.sum().backward()
    ref = torch.zeros(10, 6).index_add_(0, idx.flatten().long(), torch.ones(4, 6))
    assert torch.equal(dw.grad.cpu(), ref)
    assert torch.equal(w.to(DEV).index_select(1, torch.tensor([5, 0], dtype=torch.int32, device=DEV)).cpu(), w[:, [5, 0]])


def test_inplace_activation_behind_a_fused_batch_norm():
    """BN followed by ReLU6(inplace=True) / SiLU(inplace=True) (MobileNet, EfficientNet): the fused batch norm does not
    keep its output for the backward, so the in-place activation behind it is legal."""
    from catch_b200.fusion import BatchNormAct2d, fuse_bn_act

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Conv2d(8, 64, 3, padding=1, bias=False), torch.nn.BatchNorm2d(64), torch.nn.ReLU6(inplace=True),
                              torch.nn.Conv2d(64, 64, 1, bias=False), torch.nn.BatchNorm2d(64), torch.nn.SiLU(inplace=True))
    x = torch.randn(16, 8, 20, 20)
    ref = copy.deepcopy(net)
    ref(x).square().mean().backward()
    fused = fuse_bn_act(copy.deepcopy(net)).to(DEV).to(memory_format=torch.channels_last)
    assert sum(isinstance(m, BatchNormAct2d) and m.act == 0 for m in fused.modules()) == 2
    with torch.autocast(DEV, dtype=torch.bfloat16):
        out = fused(x.to(DEV).contiguous(memory_format=torch.channels_last))
    out.float().square().mean().backward()
    for (n, p), q in zip(ref.named_parameters(), fused.parameters()):
        assert_tensors_equal(q.grad, p.grad, prec=1e-1, use_MSE=True, msg=n)   # bf16 activations against an fp32 run
