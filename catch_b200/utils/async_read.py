"""Reading per-step scalars (loss, metrics) back to the host without stalling the compute queue.

``loss.item()`` makes the host wait for the whole step and only then start launching the next one, so the device
idles while the host catches up.  ``DelayedScalar.push(loss)`` starts a non-blocking copy into pinned memory on a side
queue and hands back the value pushed one call earlier, which by then has arrived: every step's value is still read,
one step late, and the host stays one step ahead of the device.
"""
from __future__ import annotations

from typing import Optional

import torch


class DelayedScalar:
    def __init__(self, device: Optional[int] = None):
        bw = torch.b200
        self._bw = bw
        self._device = bw.current_device() if device is None else device
        self._side = bw.queue_from_pool(self._device)
        self._slots = [bw.pin_memory(torch.zeros((), dtype=torch.float32)) for _ in range(2)]
        self._n = 0
        self._pending = None  # (notifier placed after the copy, slot)

    def push(self, value: torch.Tensor) -> Optional[float]:
        """Start reading ``value`` (a one-element device tensor); return the value of the previous push, if any."""
        bw = self._bw
        ready = bw.Notifier(enable_timing=False)
        ready.place(bw.current_queue(self._device))
        slot = self._slots[self._n % 2]
        self._n += 1
        prev = self._pending
        with bw.stream(self._side):
            ready.wait(self._side)
            bw.record_queue(value, self._side)  # the allocator must not reuse the block before the side queue is done
            src = value.detach().reshape(())
            if src.dtype != torch.float32:
                src = src.float()
            slot.copy_(src, non_blocking=True)
            done = bw.Notifier(enable_timing=False)
            done.place(self._side)
        self._pending = (done, slot)
        return self._take(prev)

    def flush(self) -> Optional[float]:
        """Value of the last push (waits for it)."""
        prev, self._pending = self._pending, None
        return self._take(prev)

    @staticmethod
    def _take(entry) -> Optional[float]:
        if entry is None:
            return None
        entry[0].synchronize()
        return float(entry[1])
