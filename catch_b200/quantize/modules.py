"""Quantized Conv1d / Conv2d / Conv3d / Linear modules.

Parity: torch_mlu/core/quantized/modules/{conv.py,linear.py,mlumodel.py}.  During
calibration (``gen_quant=True``) a module runs in floating point and its observers
record ranges; ``state_dict()`` then carries, next to ``weight`` / ``bias``:

    <prefix>scale                    [input_scale, weight_scale]   (scale = 127 / absmax)
    <prefix>quantized_mode           1 int8 per tensor, 2 int16, 3 int8 per channel, 4 int16 per channel
    <prefix>scale_weight_per_channel per-output-channel weight scales (per-channel modes)
    <prefix>quantized_by_channel     flag
    <prefix>input_mean / input_std   first convolution only: per-channel mean / std of the raw input, times 255

Loading such a state dict into a module built without ``gen_quant`` switches it to the
int8 tensor-core path: ``torch.ops.catch_b200.conv2d / linear`` with the reference's
argument order.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .observer import MinMaxObserver, NoopObserver, PerChannelMinMaxObserver

_FIRSTCONV_ERROR = ("You are using firstconv but forget setting mean or std, please set mean and std in qconfig!")

_MODE = {("int8", False): 1, ("int16", False): 2, ("int8", True): 3, ("int16", True): 4}


class QuantModule(torch.nn.Module):
    """Shared bookkeeping of quantized layers."""

    _EXTRA_KEYS = ("scale", "quantized_mode", "scale_weight_per_channel", "quantized_by_channel", "input_mean", "input_std")

    def _init_quant(self, qconfig: Optional[dict], gen_quant: bool):
        qconfig = qconfig or {}
        self.qdtype = qconfig.get("dtype", "int8")
        self.per_channel = bool(qconfig.get("per_channel", False))
        self.gen_quant = gen_quant
        self.register_buffer("scale", None)
        self.register_buffer("quantized_mode", None)
        self.register_buffer("scale_weight_per_channel", None)
        # first convolution (raw 0..255 pixels in, normalisation folded into the layer): see set_mean_std
        self.register_buffer("input_mean", None)
        self.register_buffer("input_std", None)
        if gen_quant:
            self.activation_observer = qconfig.get("activation_observer") or MinMaxObserver(
                self.qdtype, qconfig.get("use_avg", False), qconfig.get("data_scale", 1.0), qconfig.get("iteration", 1))
            self.weight_observer = (PerChannelMinMaxObserver(self.qdtype) if self.per_channel
                                    else MinMaxObserver(self.qdtype))
        else:
            self.activation_observer = NoopObserver(self.qdtype)
            self.weight_observer = NoopObserver(self.qdtype)

    # ---- quantization parameters -------------------------------------------------------
    def set_scale(self, scale: torch.Tensor) -> None:
        self.scale = scale.detach().clone().float()

    def set_quantized_mode(self, mode) -> None:
        self.quantized_mode = torch.as_tensor(mode, dtype=torch.int32).reshape(-1)[:1].clone()

    def set_mean_std(self, mean, std) -> None:
        """Per-channel mean / std that the layer applies to its (raw) input on the device:
        ``(x - mean) / std`` before the convolution (reference: MLUConv2d.forward, conv.py:171-180)."""
        mean, std = torch.as_tensor(mean, dtype=torch.float32), torch.as_tensor(std, dtype=torch.float32)
        if mean.dim() == 1:
            shape = (1, -1) + (1,) * (self.weight.dim() - 2)
            mean, std = mean.reshape(shape), std.reshape(shape)
        self.input_mean, self.input_std = mean.clone(), std.clone()

    def is_quantized(self) -> bool:
        return self.scale is not None and self.quantized_mode is not None and int(self.quantized_mode.reshape(-1)[0]) != 0

    def _collect(self):
        """Scales from the observers -> (scale, mode, per-channel scales or None)."""
        in_scale = self.activation_observer.scale().reshape(1).float().cpu()
        if self.per_channel:
            self.weight_observer(self.weight)
            wpc = self.weight_observer.scale().float().cpu()
            w_scale = wpc.min().reshape(1)
        else:
            wpc = None
            self.weight_observer(self.weight)
            w_scale = self.weight_observer.scale().reshape(1).float().cpu()
        mode = torch.tensor([_MODE[(self.qdtype, self.per_channel)]], dtype=torch.int32)
        return torch.cat([in_scale, w_scale]), mode, wpc

    # ---- state dict ------------------------------------------------------------------------
    def _save_to_state_dict(self, destination, prefix, keep_vars):
        for name, p in self._parameters.items():
            if p is not None:
                destination[prefix + name] = p if keep_vars else p.detach()
        if self.gen_quant:
            scale, mode, wpc = self._collect()
        else:
            scale, mode, wpc = self.scale, self.quantized_mode, self.scale_weight_per_channel
        if scale is not None:
            destination[prefix + "scale"] = scale
            destination[prefix + "quantized_mode"] = mode
            if wpc is not None:
                destination[prefix + "scale_weight_per_channel"] = wpc
                destination[prefix + "quantized_by_channel"] = torch.tensor([1], dtype=torch.int32)
        if self.input_std is not None:
            # calibration stores the [0, 1] values of the qconfig times 255; an inference module holds them as loaded
            k = 255.0 if self.gen_quant else 1.0
            destination[prefix + "input_mean"] = self.input_mean.detach() * k
            destination[prefix + "input_std"] = self.input_std.detach() * k

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        if prefix + "scale" in state_dict:
            self.set_scale(state_dict.pop(prefix + "scale"))
        if prefix + "quantized_mode" in state_dict:
            self.set_quantized_mode(state_dict.pop(prefix + "quantized_mode"))
        if prefix + "scale_weight_per_channel" in state_dict:
            self.scale_weight_per_channel = state_dict.pop(prefix + "scale_weight_per_channel").detach().clone().float()
        state_dict.pop(prefix + "quantized_by_channel", None)
        if prefix + "input_mean" in state_dict and prefix + "input_std" in state_dict:
            self.set_mean_std(state_dict.pop(prefix + "input_mean"), state_dict.pop(prefix + "input_std"))
        for k in ("input_mean", "input_std"):
            state_dict.pop(prefix + k, None)
        # buffers declared as None must not be reported missing
        super()._load_from_state_dict(state_dict, prefix, local_metadata, False, missing_keys, unexpected_keys, error_msgs)
        for k in list(missing_keys):
            if k.startswith(prefix) and k[len(prefix):] in self._EXTRA_KEYS:
                missing_keys.remove(k)


class _QuantConvNd(QuantModule):
    """Quantized convolution over ``ND`` spatial dimensions (subclasses set ``ND``, the float module type and the op)."""

    ND = 2
    FLOAT = torch.nn.Conv2d

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 qconfig: Optional[dict] = None, gen_quant: bool = False):
        super().__init__()
        tup = torch.nn.modules.utils._ntuple(self.ND)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.dilation = tup(kernel_size), tup(stride), tup(padding), tup(dilation)
        self.groups = groups
        self.weight = torch.nn.Parameter(torch.empty(out_channels, in_channels // groups, *self.kernel_size))
        self.bias = torch.nn.Parameter(torch.empty(out_channels)) if bias else None
        self._init_quant(qconfig, gen_quant)

    @classmethod
    def from_float(cls, mod, qconfig=None, gen_quant=False):
        if not isinstance(mod, cls.FLOAT):
            raise ValueError(f"{cls.__name__} only works for {cls.FLOAT.__name__} or its subclasses")
        if mod.padding_mode != "zeros" or isinstance(mod.padding, str):
            raise ValueError(f"{cls.__name__} supports numeric zero padding only")
        q = cls(mod.in_channels, mod.out_channels, mod.kernel_size, mod.stride, mod.padding, mod.dilation, mod.groups,
                mod.bias is not None, qconfig, gen_quant)
        q.weight = mod.weight
        q.bias = mod.bias
        return q

    def _float_conv(self, x):
        fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[self.ND]
        return fn(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)

    def _device_op(self):
        return {1: torch.ops.catch_b200.conv1d, 2: torch.ops.catch_b200.conv2d, 3: torch.ops.catch_b200.conv3d}[self.ND]

    def forward(self, x):
        if self.gen_quant:
            # calibration runs in floating point on inputs that are already normalised
            self.activation_observer(x)
            return self._float_conv(x)
        if self.input_std is not None:
            x = (x - self.input_mean.to(x.device, x.dtype)) / self.input_std.to(x.device, x.dtype)
        scale = self.scale if self.is_quantized() else None
        return self._device_op()(x, self.weight, self.bias, list(self.padding), list(self.stride), list(self.dilation),
                                 self.groups, scale, self.quantized_mode)

    def extra_repr(self):
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}, "
                f"padding={self.padding}, quantized={self.is_quantized()}, first_conv={self.input_std is not None}")


class QuantConv2d(_QuantConvNd):
    ND, FLOAT = 2, torch.nn.Conv2d


class QuantConv1d(_QuantConvNd):
    """Reference: MLUConv1d (torch_mlu/core/quantized/modules/conv.py:258-311)."""
    ND, FLOAT = 1, torch.nn.Conv1d


class QuantConv3d(_QuantConvNd):
    """Reference: MLUConv3d (torch_mlu/core/quantized/modules/conv.py:313-377)."""
    ND, FLOAT = 3, torch.nn.Conv3d


class QuantLinear(QuantModule):
    def __init__(self, in_features, out_features, bias=True, qconfig: Optional[dict] = None, gen_quant: bool = False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features))
        self.bias = torch.nn.Parameter(torch.empty(out_features)) if bias else None
        self._init_quant(qconfig, gen_quant)

    @classmethod
    def from_float(cls, mod: torch.nn.Linear, qconfig=None, gen_quant=False):
        q = cls(mod.in_features, mod.out_features, mod.bias is not None, qconfig, gen_quant)
        q.weight = mod.weight
        q.bias = mod.bias
        return q

    def forward(self, x):
        if self.gen_quant:
            self.activation_observer(x)
            return F.linear(x, self.weight, self.bias)
        scale = self.scale if self.is_quantized() else None
        return torch.ops.catch_b200.linear(x, self.weight, self.bias, scale, self.quantized_mode)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, quantized={self.is_quantized()}"
