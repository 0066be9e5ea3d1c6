"""Fused optimizers of the blackwell backend."""
from .fused import FusedAdamW, FusedSGD  # noqa: F401
