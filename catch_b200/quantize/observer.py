"""Observers that collect activation / weight ranges during calibration.

Parity: torch_mlu/core/quantized/observer.py:72-322 (abs-max with optional running
average and ``data_scale``, per-channel abs-max, a norm-based variant, the squared-range
observer for LRN inputs, a no-op).  The
scale convention is the reference's: ``scale = qmax / absmax`` with qmax 127 (int8) or
32767 (int16).
"""
from __future__ import annotations

import torch

QMAX = {"int8": 127.0, "int16": 32767.0}


class ObserverBase(torch.nn.Module):
    def __init__(self, dtype: str = "int8"):
        super().__init__()
        if dtype not in QMAX:
            raise ValueError(f"unknown quantization dtype {dtype!r}")
        self.qdtype = dtype
        self.qmax = QMAX[dtype]

    def scale(self) -> torch.Tensor:
        raise NotImplementedError


class MinMaxObserver(ObserverBase):
    """Per-tensor abs-max; ``use_avg`` averages the per-batch maxima over ``iteration`` batches."""

    def __init__(self, dtype: str = "int8", use_avg: bool = False, data_scale: float = 1.0, iteration: int = 1):
        super().__init__(dtype)
        self.use_avg, self.data_scale, self.iteration = use_avg, float(data_scale), max(int(iteration), 1)
        self.register_buffer("absmax", torch.zeros(()), persistent=False)
        self.register_buffer("seen", torch.zeros((), dtype=torch.long), persistent=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            m = torch.ops.catch_b200.absmax(x.detach()).to(self.absmax.device).reshape(())
            if self.use_avg:
                n = self.seen.item()
                self.absmax.copy_((self.absmax * n + m) / (n + 1))
            else:
                self.absmax.copy_(torch.maximum(self.absmax, m))
            self.seen += 1
        return x

    def scale(self) -> torch.Tensor:
        # data_scale multiplies the observed range, as in the reference (observer.py:154-155): a value
        # above one widens the range and lowers the scale
        amax = (self.absmax * self.data_scale).clamp_min(1e-12)
        return (self.qmax / amax).reshape(1)


class LrnObserver(MinMaxObserver):
    """Range observer for the input of a local-response normalisation: the layer squares its input, so the
    scale is taken from the squared extremes (reference: MLULrnObserver, observer.py:172-200)."""

    def scale(self) -> torch.Tensor:
        amax = ((self.absmax * self.data_scale) ** 2).clamp_min(1e-12)
        return (self.qmax / amax).reshape(1)


class PerChannelMinMaxObserver(ObserverBase):
    """Abs-max per output channel (dimension 0) of a weight tensor."""

    def __init__(self, dtype: str = "int8"):
        super().__init__(dtype)
        self.absmax = None

    def forward(self, w: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            m = w.detach().abs().reshape(w.shape[0], -1).max(1).values.float().cpu()
            self.absmax = m if self.absmax is None else torch.maximum(self.absmax, m)
        return w

    def scale(self) -> torch.Tensor:
        return self.qmax / self.absmax.clamp_min(1e-12)


class NormObserver(MinMaxObserver):
    """Range from mean + k * std of |x| (less sensitive to outliers than the plain maximum)."""

    def __init__(self, dtype: str = "int8", k: float = 6.0, **kw):
        super().__init__(dtype, **kw)
        self.k = k

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            a = x.detach().float().abs()
            m = torch.minimum(a.max(), a.mean() + self.k * a.std()).cpu().reshape(())
            self.absmax.copy_(torch.maximum(self.absmax, m))
            self.seen += 1
        return x


class NoopObserver(ObserverBase):
    def forward(self, x):
        return x

    def scale(self):
        return torch.ones(1)
