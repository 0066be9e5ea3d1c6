"""``quantize_dynamic`` -- swap Conv2d / Linear for their quantized counterparts.

Same flow and signature as the reference's ``quantize_dynamic_mlu``
(torch_mlu/core/mlu_quantize.py:155-229): propagate a qconfig, add observers when
``gen_quant`` is set, replace modules through a mapping.

    # 1. calibrate (floating point, any device) and export the scales
    qm = quantize_dynamic(model, {"per_channel": True, "iteration": 8}, dtype="int8", gen_quant=True)
    for batch in calibration_batches: qm(batch)
    sd = qm.state_dict()
    # 2. build the inference model and load the scales
    infer = quantize_dynamic(model)
    infer.load_state_dict(sd)
    infer.to("blackwell")(x)          # int8 tcgen05 convolutions / linears

qconfig keys (the reference's, torch_mlu/core/quantized/qscheme.py:11-19): ``iteration``, ``use_avg``,
``data_scale``, ``per_channel``, ``method`` ("minmax", "norm" or "lrn"), ``firstconv`` with ``mean`` / ``std``
(per-channel values in [0, 1]; the first ``Conv2d`` then normalises raw 0..255 inputs itself at inference
time); ``mixed_layer`` maps module names to "float" to keep them unquantized.
"""
from __future__ import annotations

import copy
from typing import Dict, Optional

import torch
import torch.nn as nn

from .modules import _FIRSTCONV_ERROR, QuantConv1d, QuantConv2d, QuantConv3d, QuantLinear, QuantModule
from .observer import LrnObserver, MinMaxObserver, NormObserver

DEFAULT_MODULE_MAPPING = {nn.Conv1d: QuantConv1d, nn.Conv2d: QuantConv2d, nn.Conv3d: QuantConv3d, nn.Linear: QuantLinear}


def _layer_qconfig(qconfig_spec: Optional[dict], dtype: Optional[str]) -> dict:
    cfg = dict(qconfig_spec or {})
    cfg["dtype"] = dtype or cfg.get("dtype", "int8")
    if cfg["dtype"] not in ("int8", "int16"):
        raise ValueError("Unknown dtype for quantization")
    method = cfg.get("method", "minmax")
    if method == "norm":
        cfg["activation_observer_factory"] = lambda: NormObserver(cfg["dtype"])
    elif method == "lrn":
        cfg["activation_observer_factory"] = lambda: LrnObserver(cfg["dtype"], cfg.get("use_avg", False),
                                                                cfg.get("data_scale", 1.0), cfg.get("iteration", 1))
    elif method == "minmax":
        cfg["activation_observer_factory"] = lambda: MinMaxObserver(cfg["dtype"], cfg.get("use_avg", False),
                                                                   cfg.get("data_scale", 1.0), cfg.get("iteration", 1))
    else:
        raise ValueError(f"unknown calibration method {method!r}")
    return cfg


def _first_conv_setup(q: QuantModule, cfg: dict, state: dict) -> None:
    """The first Conv2d met during conversion takes the qconfig's mean / std (reference: conv.py:203-247)."""
    if not isinstance(q, QuantConv2d) or state.get("seen_first_conv"):
        return
    state["seen_first_conv"] = True
    if not cfg.get("firstconv"):
        return
    mean, std = cfg.get("mean"), cfg.get("std")
    if mean is None or std is None:
        raise AssertionError(_FIRSTCONV_ERROR)
    if q.in_channels not in (1, 3, 4):
        raise AssertionError("firstconv: the first Conv2d must take 1 (gray), 3 (RGB) or 4 (RGBA) input channels, "
                             f"not {q.in_channels}; set firstconv False for a generic convolution")
    if not (min(mean) >= 0 and max(mean) <= 1 and min(std) >= 0 and max(std) <= 1):
        raise AssertionError(f"firstconv: mean and std must lie in [0, 1] (they are multiplied by 255 for inference); "
                             f"mean is {mean}, std is {std}")
    q.set_mean_std(torch.tensor(mean, dtype=torch.float32), torch.tensor(std, dtype=torch.float32))


def _convert(module: nn.Module, mapping: Dict, cfg: dict, gen_quant: bool, mixed_layer: Optional[dict], prefix: str = "",
             state: Optional[dict] = None):
    state = {} if state is None else state
    for name, child in list(module.named_children()):
        full = prefix + name
        target = mapping.get(type(child))
        keep_float = mixed_layer is not None and str(mixed_layer.get(full, "")).strip() in ("float", "fp32", "fp16")
        if target is not None and not keep_float and not isinstance(child, QuantModule):
            try:
                layer_cfg = dict(cfg)
                layer_cfg["activation_observer"] = cfg["activation_observer_factory"]() if gen_quant else None
                q = target.from_float(child, layer_cfg, gen_quant)
            except ValueError:
                continue  # unsupported layer variant stays in floating point
            if gen_quant:
                _first_conv_setup(q, cfg, state)
            setattr(module, name, q)
        else:
            _convert(child, mapping, cfg, gen_quant, mixed_layer, full + ".", state)


def quantize_dynamic(model: nn.Module, qconfig_spec: Optional[dict] = None, dtype: Optional[str] = None,
                     mapping: Optional[Dict] = None, inplace: bool = False, gen_quant: bool = False,
                     mixed_layer: Optional[dict] = None) -> nn.Module:
    if mixed_layer is not None and not isinstance(mixed_layer, dict):
        raise ValueError(f"type(mixed_layer) must be dict, now is {type(mixed_layer)}")
    if qconfig_spec is not None and not isinstance(qconfig_spec, dict):
        raise ValueError("Unknown qconfig_spec")
    cfg = _layer_qconfig(qconfig_spec, dtype)
    if not inplace:
        try:
            model = copy.deepcopy(model)
        except Exception:
            print('Warning: Failed to deepcopy model, "inplace" is set to True by default.')
    model.eval()
    _convert(model, mapping or DEFAULT_MODULE_MAPPING, cfg, gen_quant, mixed_layer)
    return model


quantize_dynamic_blackwell = quantize_dynamic
