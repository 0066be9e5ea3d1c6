"""Profiling helpers.

The stock profiler understands the device through the PrivateUse1 profiler stubs this
backend registers: ``torch.autograd.profiler.profile(use_device="blackwell")`` gives
per-op device times (``device_time`` columns of ``.table()`` / ``key_averages()`` /
``export_chrome_trace()``), ``profile_memory=True`` reports the caching allocator's
allocations.  Reference: ``torch.autograd.profiler.profile(use_mlu=True)``
(torch_mlu/core/profile/profile_mlu.py:10-23, docs user guide section on profiling).
"""
from __future__ import annotations

import torch


def profile(record_shapes: bool = False, profile_memory: bool = False, with_stack: bool = False, enabled: bool = True):
    """``torch.autograd.profiler.profile`` preset for the blackwell device."""
    return torch.autograd.profiler.profile(enabled=enabled, use_device="blackwell", record_shapes=record_shapes,
                                           profile_memory=profile_memory, with_stack=with_stack, use_kineto=False)


class timed_region:
    """Device time of a code region measured with two notifiers (milliseconds in ``.ms``)."""

    def __enter__(self):
        self._a, self._b = torch.b200.Notifier(), torch.b200.Notifier()
        self._a.place()
        return self

    def __exit__(self, *exc):
        self._b.place()
        self._b.synchronize()
        self.ms = self._a.elapsed_time(self._b)
        self.us = self._a.hardware_time(self._b)
        return False
