"""Post-training int8 quantization tool."""
from .observer import (LrnObserver, MinMaxObserver, NoopObserver, NormObserver, PerChannelMinMaxObserver)  # noqa: F401
from .modules import QuantConv1d, QuantConv2d, QuantConv3d, QuantLinear, QuantModule  # noqa: F401
from .tool import DEFAULT_MODULE_MAPPING, quantize_dynamic, quantize_dynamic_blackwell  # noqa: F401
