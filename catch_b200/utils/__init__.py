"""Utilities: prefetching data loader."""
from .data_loader import PrefetchLoader  # noqa: F401
