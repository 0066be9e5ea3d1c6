"""Comparison helpers shared by the test-suite.

Same four error metrics as the reference's ``TestCase.assertTensorsEqual``
(test/common_utils.py:479-541): NaN positions must agree, then either
max-abs error, relative RMS error (use_MSE), relative abs-sum error (use_RAE)
or relative mean error (use_RMA) must stay below ``prec``.
"""
import torch


def assert_tensors_equal(a, b, prec=3e-3, use_MSE=False, use_RAE=False, use_RMA=False, msg=""):
    a = a.detach().cpu().double() if isinstance(a, torch.Tensor) else torch.tensor(a, dtype=torch.double)
    b = b.detach().cpu().double() if isinstance(b, torch.Tensor) else torch.tensor(b, dtype=torch.double)
    assert a.shape == b.shape, f"{msg} shape mismatch {tuple(a.shape)} vs {tuple(b.shape)}"
    if a.numel() == 0:
        return
    nan_a, nan_b = torch.isnan(a), torch.isnan(b)
    assert torch.equal(nan_a, nan_b), f"{msg} NaN positions differ"
    a = torch.where(nan_a, torch.zeros_like(a), a)
    b = torch.where(nan_b, torch.zeros_like(b), b)
    inf_a, inf_b = torch.isinf(a), torch.isinf(b)
    assert torch.equal(inf_a, inf_b) and torch.equal(a[inf_a], b[inf_b]), f"{msg} infinities differ"
    a = torch.where(inf_a, torch.zeros_like(a), a)
    b = torch.where(inf_b, torch.zeros_like(b), b)
    eps = 1e-9
    if use_MSE:
        err = torch.sqrt(((a - b) ** 2).sum() / ((a ** 2).sum() + eps)).item()
    elif use_RAE:
        err = ((a - b).abs().sum() / (a.abs().sum() + eps)).item()
    elif use_RMA:
        err = ((a.abs().mean() - b.abs().mean()).abs() / (a.abs().mean() + eps)).item()
    else:
        err = (a - b).abs().max().item()
    assert err <= prec, f"{msg} error {err:.3e} exceeds {prec:.1e}"
