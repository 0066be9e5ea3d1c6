"""Profiling helpers.

* ``profile(...)`` -- ``torch.autograd.profiler.profile`` preset for the device: the stock profiler
  understands the device through the PrivateUse1 profiler stubs this backend registers, so
  ``.table()`` / ``key_averages()`` / ``export_chrome_trace()`` carry per-operator device times and,
  with ``profile_memory=True``, the caching allocator's allocations.  With ``kernels=True`` (default)
  the returned object also records every kernel launch (``.kernels``) and its Chrome trace gets device
  rows with one slice per kernel.
* ``kernel_trace()`` -- only the kernel-level trace: launcher name, issuing operator, queue, device start
  time and duration of every launch, plus ``mark`` / ``range`` annotations.
* ``timed_region()`` -- device time of a code region from two notifiers.

Reference: ``torch.autograd.profiler.profile(use_mlu=True)`` and its device-event join
(torch_mlu/core/profile/profile_mlu.py:10-23, torch_mlu/csrc/aten/profile/profile_mlu.cpp:76-211).
"""
from __future__ import annotations

import collections
import contextlib
import json
from dataclasses import dataclass
from typing import List

import torch

from . import _C

_KINDS = {0: "kernel", 1: "range", 2: "mark"}


@dataclass
class KernelEvent:
    name: str
    op: str
    kind: str
    device: int
    queue: int
    cpu_ns: int
    start_us: float
    dur_us: float


class KernelTrace:
    """Every kernel launched between ``__enter__`` and ``__exit__`` (``.events`` afterwards)."""

    def __init__(self):
        self.events: List[KernelEvent] = []

    def __enter__(self):
        _C._kernel_trace_start()
        return self

    def __exit__(self, *exc):
        self.events = [KernelEvent(n, op, _KINDS.get(k, "kernel"), d, q, c, s, u) for n, op, k, d, q, c, s, u in _C._kernel_trace_stop()]
        return False

    # ---- summaries ------------------------------------------------------------------------------
    @property
    def kernels(self) -> List[KernelEvent]:
        return [e for e in self.events if e.kind == "kernel"]

    def total_device_time_us(self) -> float:
        return sum(e.dur_us for e in self.kernels)

    def key_averages(self):
        """[(name, launches, total us, mean us)] sorted by total device time."""
        tot, cnt = collections.Counter(), collections.Counter()
        for e in self.kernels:
            tot[e.name] += e.dur_us
            cnt[e.name] += 1
        return [(n, cnt[n], t, t / cnt[n]) for n, t in tot.most_common()]

    def table(self, row_limit: int = 30) -> str:
        rows = self.key_averages()[:row_limit]
        total = self.total_device_time_us() or 1.0
        width = max([len(r[0]) for r in rows] + [6])
        lines = [f"{'kernel':{width}s}  {'launches':>8s}  {'device us':>12s}  {'mean us':>10s}  {'share':>6s}",
                 "-" * (width + 46)]
        for n, c, t, m in rows:
            lines.append(f"{n:{width}s}  {c:8d}  {t:12.1f}  {m:10.2f}  {100 * t / total:5.1f}%")
        lines.append(f"{len(self.kernels)} launches, {total:.1f} us of device time")
        return "\n".join(lines)

    def chrome_events(self) -> list:
        """Trace-event dictionaries: one row (tid) per device queue, one slice per kernel / range, instants for marks."""
        out = []
        for e in self.events:
            base = {"name": e.name, "pid": f"blackwell:{e.device}", "tid": f"queue {e.queue & 0xffffffff}", "ts": e.start_us,
                    "cat": e.kind, "args": {"op": e.op, "launch_cpu_ns": e.cpu_ns}}
            if e.kind == "mark":
                out.append(dict(base, ph="i", s="t"))
            else:
                out.append(dict(base, ph="X", dur=max(e.dur_us, 0.001)))
        return out

    def export_chrome_trace(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"traceEvents": self.chrome_events()}, f)


def kernel_trace() -> KernelTrace:
    return KernelTrace()


def mark(name: str) -> None:
    """An instant annotation on the current queue (recorded while a kernel trace is active)."""
    _C._trace_mark(name)


@contextlib.contextmanager
def range(name: str):  # noqa: A001 - mirrors torch.cuda.nvtx.range
    """Bracket a region of the current queue's work with a named slice."""
    _C._trace_range_push(name)
    try:
        yield
    finally:
        _C._trace_range_pop()


class _Profile:
    """The stock autograd profiler plus the kernel-level trace of the same region."""

    def __init__(self, prof, kernels: bool):
        self._prof = prof
        self._kt = KernelTrace() if kernels else None

    def __enter__(self):
        if self._kt is not None:
            self._kt.__enter__()
        self._prof.__enter__()
        return self

    def __exit__(self, *exc):
        r = self._prof.__exit__(*exc)
        if self._kt is not None:
            self._kt.__exit__(*exc)
        return r

    def __getattr__(self, name):  # function_events, key_averages, table, total_average, ...
        return getattr(self._prof, name)

    @property
    def kernels(self) -> KernelTrace:
        return self._kt

    def export_chrome_trace(self, path: str) -> None:
        """The stock trace with the kernel rows of every device queue added."""
        self._prof.export_chrome_trace(path)
        if self._kt is None:
            return
        with open(path) as f:
            data = json.load(f)
        events = data["traceEvents"] if isinstance(data, dict) else data
        events.extend(self._kt.chrome_events())
        with open(path, "w") as f:
            json.dump({"traceEvents": events} if isinstance(data, dict) else events, f)


def profile(record_shapes: bool = False, profile_memory: bool = False, with_stack: bool = False, enabled: bool = True,
            kernels: bool = True):
    """``torch.autograd.profiler.profile`` preset for the blackwell device (see the module docstring)."""
    prof = torch.autograd.profiler.profile(enabled=enabled, use_device="blackwell", record_shapes=record_shapes,
                                           profile_memory=profile_memory, with_stack=with_stack, use_kineto=False)
    return _Profile(prof, kernels and enabled)


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
