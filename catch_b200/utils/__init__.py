"""Utilities: prefetching data loader, NUMA placement of a rank's host side."""
from .data_loader import PrefetchLoader  # noqa: F401
from .numa import bind_to_device_node, gpu_numa_node  # noqa: F401
