"""``torch.distributed`` backend ``"bwccl"`` for the blackwell device.

``init_process_group(backend="bwccl")`` gives a process group whose collectives
are this project's own kernels over peer-mapped GPU memory (or, under host
simulation, messages through the rendezvous Store).  Stock
``DistributedDataParallel`` works on top of it; the counterpart in the reference
is the ``"cncl"`` backend (torch_mlu/csrc/distributed/process_group_cncl.hpp:288-294).
"""
from __future__ import annotations

import datetime

import torch
import torch.distributed as dist

from . import _C

BACKEND_NAME = "bwccl"


def _create_backend(store, rank, size, timeout):
    if not isinstance(timeout, datetime.timedelta):
        timeout = datetime.timedelta(seconds=600)
    return _C.ProcessGroupB200(store, rank, size, timeout)


def register() -> None:
    if not hasattr(dist.Backend, BACKEND_NAME.upper()):
        dist.Backend.register_backend(BACKEND_NAME, _create_backend, devices=["blackwell"])


def get_backend(group=None) -> "_C.ProcessGroupB200":
    """The native ProcessGroupB200 object behind a torch.distributed group."""
    group = group or dist.group.WORLD
    return group._get_backend(torch.device("blackwell"))


register()

# Watchdog threads use the Store; they must be gone before the interpreter tears down the objects they use
# (a group can outlive destroy_process_group() when something else still references its backend).
import atexit  # noqa: E402

if hasattr(_C, "_stop_all_watchdogs"):  # absent only while an older native library is being rebuilt
    atexit.register(_C._stop_all_watchdogs)
