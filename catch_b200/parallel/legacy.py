"""Deprecated-style wrappers kept for scripts written against the reference's
``torch_mlu.distributed`` module (torch_mlu/distributed/mlu_ddp.py:44-199): thin
shims over ``torch.distributed`` that default to this backend and to one device
per process."""
from __future__ import annotations

import warnings

import torch
import torch.distributed as dist

from ..distributed import BACKEND_NAME


def init_process_group(backend: str = BACKEND_NAME, **kwargs):
    warnings.warn("catch_b200.parallel.init_process_group is a compatibility shim; call "
                  "torch.distributed.init_process_group(backend='bwccl') directly.", DeprecationWarning, stacklevel=2)
    if backend in ("cncl", "nccl"):
        backend = BACKEND_NAME
    return dist.init_process_group(backend=backend, **kwargs)


class DistributedDataParallel(torch.nn.parallel.DistributedDataParallel):
    """``DistributedDataParallel`` pinned to the current blackwell device."""

    def __init__(self, module, device_ids=None, output_device=None, **kwargs):
        warnings.warn("catch_b200.parallel.DistributedDataParallel is a compatibility shim over "
                      "torch.nn.parallel.DistributedDataParallel.", DeprecationWarning, stacklevel=2)
        if device_ids is None:
            device_ids = [torch.b200.current_device()]
        assert len(device_ids) == 1, "only one device per process is supported"
        super().__init__(module, device_ids=device_ids, output_device=output_device, **kwargs)
