"""catch_b200 -- an out-of-tree PyTorch device backend ("b200") for NVIDIA B200.

Importing the package loads the native runtime, registers the ``blackwell`` device
with PyTorch through the PrivateUse1 extension point and exposes the device
module as ``torch.blackwell`` (alias ``torch.b200``) (the counterpart of ``torch.mlu`` in the reference:
torch_mlu/__init__.py:4-14).
"""
from __future__ import annotations

import os as _os

import torch as _torch

from . import _loader

_C = _loader.load_native()

# torch.device() accepts only letters and "_" in a device-type name, hence "blackwell".
DEVICE_TYPE = "blackwell"
_torch.utils.rename_privateuse1_backend(DEVICE_TYPE)

from . import device_module as _device_module  # noqa: E402

_torch._register_device_module(DEVICE_TYPE, _device_module)
_torch.b200 = _device_module  # short alias: torch.b200 is torch.blackwell
_torch.utils.generate_methods_for_privateuse1_backend(for_tensor=True, for_module=True, for_storage=False,
                                                      for_packed_sequence=True)



def _accept_queues_in_record_stream() -> None:
    """``tensor.record_stream(s)`` takes this backend's Queue objects (what ``torch.blackwell.current_stream()``
    returns) as well as ``torch.Stream``: scripts written for ``torch.cuda`` pass the former."""
    original = _torch.Tensor.record_stream

    def record_stream(self, stream):
        if isinstance(stream, _device_module.Queue):
            if self.device.type == DEVICE_TYPE:
                _device_module.record_queue(self, stream)
            return None
        return original(self, stream)

    record_stream.__doc__ = original.__doc__
    _torch.Tensor.record_stream = record_stream


_accept_queues_in_record_stream()

from .device_module import *  # noqa: F401,F403,E402
from . import distributed  # noqa: F401,E402  (registers the "bwccl" backend)

__version__ = "0.1.0"
