"""Communication hooks for stock ``torch.nn.parallel.DistributedDataParallel`` on ``bwccl``.

    ddp = DistributedDataParallel(model.to("blackwell"))
    ddp.register_comm_hook(None, catch_b200.parallel.hooks.bf16_compress_hook)

Stock DDP already reduces its buckets through the process group of this backend; a hook
changes what goes over NVLink.  ``allreduce_hook`` is the plain average (the default
behaviour spelled out); ``bf16_compress_hook`` halves the bytes of fp32 gradient buckets
by reducing them in bfloat16.  The fused all-reduce + optimizer path is a different
wrapper (``FusedDataParallel``), because it also owns the parameter update.

The reference has no hooks (its DDP predates them: torch_mlu/distributed/mlu_ddp.py is a
thin alias of the stock wrapper).
"""
import torch
import torch.distributed as dist


def _done(value: torch.Tensor) -> torch.futures.Future[torch.Tensor]:
    fut = torch.futures.Future()
    fut.set_result(value)
    return fut


def allreduce_hook(process_group, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Average the bucket over the group (what DDP does without a hook)."""
    group = process_group if process_group is not None else dist.group.WORLD
    buf = bucket.buffer()
    buf.div_(dist.get_world_size(group))
    dist.all_reduce(buf, group=group)
    return _done(buf)


def bf16_compress_hook(process_group, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Average the bucket in bfloat16: half the bytes on the wire for fp32 gradients."""
    group = process_group if process_group is not None else dist.group.WORLD
    buf = bucket.buffer()
    if buf.dtype != torch.float32:
        return allreduce_hook(process_group, bucket)
    small = buf.div(dist.get_world_size(group)).to(torch.bfloat16)
    dist.all_reduce(small, group=group)
    buf.copy_(small)
    return _done(buf)
