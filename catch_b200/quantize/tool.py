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

qconfig keys: ``iteration``, ``use_avg``, ``data_scale``, ``per_channel``, ``method``
("minmax" or "norm"); ``mixed_layer`` maps module names to "float" to keep them
unquantized (e.g. the 3-channel first convolution).
"""
from __future__ import annotations

import copy
from typing import Dict, Optional

import torch
import torch.nn as nn

from .modules import QuantConv2d, QuantLinear
from .observer import MinMaxObserver, NormObserver

DEFAULT_MODULE_MAPPING = {nn.Conv2d: QuantConv2d, nn.Linear: QuantLinear}


def _layer_qconfig(qconfig_spec: Optional[dict], dtype: Optional[str]) -> dict:
    cfg = dict(qconfig_spec or {})
    cfg["dtype"] = dtype or cfg.get("dtype", "int8")
    if cfg["dtype"] not in ("int8", "int16"):
        raise ValueError("Unknown dtype for quantization")
    method = cfg.get("method", "minmax")
    if method == "norm":
        cfg["activation_observer_factory"] = lambda: NormObserver(cfg["dtype"])
    elif method == "minmax":
        cfg["activation_observer_factory"] = lambda: MinMaxObserver(cfg["dtype"], cfg.get("use_avg", False),
                                                                   cfg.get("data_scale", 1.0), cfg.get("iteration", 1))
    else:
        raise ValueError(f"unknown calibration method {method!r}")
    return cfg


def _convert(module: nn.Module, mapping: Dict, cfg: dict, gen_quant: bool, mixed_layer: Optional[dict], prefix: str = ""):
    for name, child in list(module.named_children()):
        full = prefix + name
        target = mapping.get(type(child))
        keep_float = mixed_layer is not None and str(mixed_layer.get(full, "")).strip() in ("float", "fp32", "fp16")
        if target is not None and not keep_float and not isinstance(child, (QuantConv2d, QuantLinear)):
            try:
                layer_cfg = dict(cfg)
                layer_cfg["activation_observer"] = cfg["activation_observer_factory"]() if gen_quant else None
                q = target.from_float(child, layer_cfg, gen_quant)
            except ValueError:
                continue  # unsupported layer variant stays in floating point
            setattr(module, name, q)
        else:
            _convert(child, mapping, cfg, gen_quant, mixed_layer, full + ".")


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
