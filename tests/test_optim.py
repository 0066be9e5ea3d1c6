"""Fused optimizers against torch.optim on the host-simulated device."""
import copy

import torch

import catch_b200  # noqa: F401
from catch_b200.optim import FusedAdamW, FusedSGD
from common import assert_tensors_equal


def _run(make_fused, make_ref, steps=4):
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Linear(7, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
    dev = copy.deepcopy(ref).to("blackwell")
    o_ref, o_dev = make_ref(ref.parameters()), make_fused(dev.parameters())
    for _ in range(steps):
        x = torch.randn(6, 7)
        o_ref.zero_grad(); o_dev.zero_grad()
        ref(x).pow(2).sum().backward()
        dev(x.to("blackwell")).pow(2).sum().backward()
        o_ref.step(); o_dev.step()
    for a, b in zip(ref.parameters(), dev.parameters()):
        assert_tensors_equal(b, a, prec=1e-5)
    return o_ref, o_dev


def test_fused_sgd_matches_torch():
    o_ref, o_dev = _run(lambda p: FusedSGD(p, lr=0.05, momentum=0.9, weight_decay=1e-4),
                        lambda p: torch.optim.SGD(p, lr=0.05, momentum=0.9, weight_decay=1e-4))
    sd = o_dev.state_dict()
    assert "momentum_buffer" in next(iter(sd["state"].values()))


def test_fused_sgd_nesterov_no_momentum():
    _run(lambda p: FusedSGD(p, lr=0.05, momentum=0.9, nesterov=True), lambda p: torch.optim.SGD(p, lr=0.05, momentum=0.9, nesterov=True))
    _run(lambda p: FusedSGD(p, lr=0.05), lambda p: torch.optim.SGD(p, lr=0.05))


def test_fused_adamw_matches_torch():
    o_ref, o_dev = _run(lambda p: FusedAdamW(p, lr=1e-2, weight_decay=0.01), lambda p: torch.optim.AdamW(p, lr=1e-2, weight_decay=0.01))
    st = next(iter(o_dev.state_dict()["state"].values()))
    assert {"step", "exp_avg", "exp_avg_sq"} <= set(st)
