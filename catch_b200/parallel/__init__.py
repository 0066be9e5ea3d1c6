"""Data-parallel training on the blackwell device."""
from .fused_ddp import FusedDataParallel  # noqa: F401
from .legacy import DistributedDataParallel, init_process_group  # noqa: F401
from . import hooks  # noqa: F401
