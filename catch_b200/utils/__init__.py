"""Utilities: prefetching data loader, delayed read-back of per-step scalars, NUMA placement of a rank's host side."""
from .async_read import DelayedScalar  # noqa: F401
from .data_loader import PrefetchLoader  # noqa: F401
from .numa import bind_to_device_node, gpu_numa_node  # noqa: F401
