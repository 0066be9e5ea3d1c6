"""Host-to-device prefetching for ``torch.utils.data.DataLoader``.

The reference's ``_MLUMultiProcessingDataLoaderIter`` (torch_mlu/core/utils/
data_loader.py:51-227, switched on with ``USE_IO_QUEUE=ON``) copies the next batch to
the device on a dedicated IO queue while the current batch is being consumed and hands
it over with a notifier.  ``PrefetchLoader`` does the same around any iterable of
batches: batches are pinned, copied on a side queue taken from the pool, recorded on
that queue for the caching allocator, and the consumer's queue waits on the copy's
notifier before the batch is returned -- the host never blocks on the copy.
"""
from __future__ import annotations

import os
from typing import Any, Iterable, Iterator

import torch


def _map(obj: Any, fn):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, dict):
        return {k: _map(v, fn) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        seq = [_map(v, fn) for v in obj]
        return type(obj)(seq) if not hasattr(obj, "_fields") else type(obj)(*seq)
    return obj


class PrefetchLoader:
    """Wraps a loader; yields batches that already live on ``device``.

    ``use_io_queue`` (default: the ``USE_IO_QUEUE`` environment variable, ON unless set
    to OFF) selects the overlapped path; otherwise batches are copied synchronously.
    ``depth`` batches are kept in flight on the IO queue (two by default, so a copy that takes
    longer than one step does not stall the next one).  ``transform`` (optional) is applied to
    each device batch on the IO queue, e.g. a cast to the compute dtype and memory format, which
    takes that pass off the compute queue.
    """

    def __init__(self, loader: Iterable, device="blackwell", use_io_queue=None, pin: bool = True, depth: int = 2,
                 transform=None):
        self.loader = loader
        self.device = torch.device(device)
        if self.device.index is None:
            self.device = torch.device(self.device.type, torch.b200.current_device())
        if use_io_queue is None:
            use_io_queue = os.environ.get("USE_IO_QUEUE", "ON").upper() != "OFF"
        self.use_io_queue = use_io_queue
        self.pin = pin
        self.depth = max(1, int(depth))
        self.transform = transform

    def __len__(self):
        return len(self.loader)

    def _to_device(self, batch, queue):
        def move(t):
            if self.pin and not torch.b200.is_pinned(t):
                t = torch.b200.pin_memory(t)
            d = t.to(self.device, non_blocking=True)
            if queue is not None:
                torch.b200.record_queue(d, queue)
            return d
        return _map(batch, move)

    def __iter__(self) -> Iterator:
        if not self.use_io_queue:
            for batch in self.loader:
                moved = self._to_device(batch, None)
                yield self.transform(moved) if self.transform is not None else moved
            return
        io_queue = torch.b200.queue_from_pool(self.device)
        it = iter(self.loader)

        def prefetch():
            try:
                batch = next(it)
            except StopIteration:
                return None
            with torch.b200.stream(io_queue):
                moved = self._to_device(batch, io_queue)
                if self.transform is not None:
                    moved = self.transform(moved)
                    _map(moved, lambda t: torch.b200.record_queue(t, io_queue) or t)
                done = torch.b200.Notifier(enable_timing=False)
                done.place(io_queue)
            return moved, done

        import collections

        inflight = collections.deque()
        for _ in range(self.depth):
            item = prefetch()
            if item is None:
                break
            inflight.append(item)
        while inflight:
            cur, cur_ev = inflight.popleft()
            item = prefetch()                          # overlaps with the consumer's compute
            if item is not None:
                inflight.append(item)
            cur_ev.wait(torch.b200.current_queue(self.device))  # device-side hand-off
            _map(cur, lambda t: torch.b200.record_queue(t, torch.b200.current_queue(self.device)) or t)
            yield cur
