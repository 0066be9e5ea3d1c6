"""Data parallelism whose gradient all-reduce is fused with the optimizer.

``FusedDataParallel`` replaces the three hot loops of a stock DDP step (the
Reducer's per-gradient copy-and-scale, the bucket all-reduce and the optimizer's
per-parameter kernels; see the reference's training call stack in
torch_mlu/csrc/distributed/process_group_cncl.cpp:334-356 and its user guide) by
ONE kernel per bucket that runs while the rest of backward is still computing:

* parameters and gradients live in symmetric (peer-mapped) memory, ``p.grad`` is a
  view of the bucket, so autograd accumulates straight into the communication buffer;
* when the last gradient of a bucket has been produced, the bucket's kernel is queued
  on the communication queue: every rank pulls its shard of the bucket from all peers
  over NVLink, reduces in fp32, scales by 1/world, applies SGD-momentum or AdamW to its
  shard of the fp32 master parameters (optimizer state is sharded: 1/world per rank)
  and pushes the updated parameters to every peer;
* ``step()`` only makes the compute queue wait for those kernels.

All ranks end every step with bit-identical parameters because each element is
updated by exactly one rank and then broadcast.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..distributed import get_backend


def _view_like(flat: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
    """A view of the flat slice with p's shape that keeps a channels-last layout."""
    if p.dim() == 4 and p.is_contiguous(memory_format=torch.channels_last) and not p.is_contiguous():
        n, c, h, w = p.shape
        return flat.view(n, h, w, c).permute(0, 3, 1, 2)
    return flat.view(p.shape)


class _Bucket:
    def __init__(self, params: List[torch.nn.Parameter]):
        self.params = params
        self.numel = sum(p.numel() for p in params)
        self.pending = 0
        self.grads = None      # symmetric flat gradient buffer
        self.flat = None       # symmetric flat fp32 parameter buffer
        self.state1 = None
        self.state2 = None
        self.first = True
        self.work = None


class FusedDataParallel(torch.nn.Module):
    """Wrap ``module`` for data-parallel training with a fused all-reduce + optimizer.

    Args:
        module: the model, already on the blackwell device.
        optimizer: ``"sgd"`` or ``"adamw"``.
        lr, momentum, dampening, weight_decay, nesterov, betas, eps: optimizer
            hyper-parameters (``param_groups``-style updates through ``set_lr``).
        bucket_mb: bucket size in MiB (gradients are bucketed in reverse
            registration order, the order backward produces them in).
        grad_dtype: dtype of the communication buffer (``torch.float32`` or
            ``torch.bfloat16`` to halve the NVLink traffic).
        process_group: a ``bwccl`` group (default: the world group).

    With a world size of one (or without an initialised process group) the same
    kernels run on local memory through the fused single-device optimizers.
    """

    def __init__(self, module: torch.nn.Module, optimizer: str = "sgd", lr: float = 0.1, momentum: float = 0.0,
                 dampening: float = 0.0, weight_decay: float = 0.0, nesterov: bool = False, betas=(0.9, 0.999),
                 eps: float = 1e-8, bucket_mb: float = 25.0, grad_dtype: torch.dtype = torch.float32,
                 process_group=None, broadcast_buffers: bool = True):
        super().__init__()
        self.module = module
        self.kind = {"sgd": 0, "adamw": 1}[optimizer.lower()]
        self.lr, self.momentum, self.dampening, self.weight_decay = lr, momentum, dampening, weight_decay
        self.nesterov, self.betas, self.eps = nesterov, betas, eps
        assert grad_dtype == torch.float32, "gradient buckets are fp32 (autograd accumulates into them in place)"
        self.grad_dtype = grad_dtype
        self.step_count = 0
        self.group = process_group or (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.pg = get_backend(self.group) if self.world > 1 else None
        self.broadcast_buffers = broadcast_buffers
        params = [p for p in module.parameters() if p.requires_grad]
        assert params, "FusedDataParallel needs at least one trainable parameter"
        assert all(p.dtype == torch.float32 for p in params), "master parameters must be fp32 (use autocast for bf16 compute)"
        self.device = params[0].device
        # bucket in reverse registration order
        cap = int(bucket_mb * 1024 * 1024 / 4)
        self.buckets: List[_Bucket] = []
        cur, cur_n = [], 0
        for p in reversed(params):
            cur.append(p)
            cur_n += p.numel()
            if cur_n >= cap:
                self.buckets.append(_Bucket(cur))
                cur, cur_n = [], 0
        if cur:
            self.buckets.append(_Bucket(cur))
        self._param_bucket = {}
        for b in self.buckets:
            self._setup_bucket(b)
        if self.world > 1:
            self._sync_initial_state()
        for b in self.buckets:
            for p in b.params:
                p.register_post_accumulate_grad_hook(self._make_hook(b))
        self._arm()

    # ------------------------------------------------------------------ setup
    def _alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        if self.pg is not None:
            return self.pg.symm_empty(numel, dtype)
        return torch.empty(numel, dtype=dtype, device=self.device)

    def _setup_bucket(self, b: _Bucket) -> None:
        # pad so every rank's shard is a whole number of 16-byte vectors
        b.flat = self._alloc(b.numel, torch.float32)
        b.grads = self._alloc(b.numel, self.grad_dtype)
        b.grads.zero_()
        off = 0
        b.grad_views = []
        for p in b.params:
            n = p.numel()
            view = _view_like(b.flat[off:off + n], p.data)
            view.copy_(p.data)
            b.grad_views.append(_view_like(b.grads[off:off + n], p.data))
            p.data = view
            self._param_bucket[p] = b
            off += n
        if self.pg is not None:
            shard = self.pg.shard_elems(b.numel, self.grad_dtype)
        else:
            shard = b.numel
        b.state1 = torch.zeros(shard, dtype=torch.float32, device=self.device)
        b.state2 = torch.zeros(shard if self.kind == 1 else 0, dtype=torch.float32, device=self.device)

    def _sync_initial_state(self) -> None:
        for b in self.buckets:
            dist.broadcast(b.flat, 0, group=self.group)
        if self.broadcast_buffers:
            for buf in self.module.buffers():
                dist.broadcast(buf, 0, group=self.group)
        torch.b200.synchronize()

    def _arm(self) -> None:
        for b in self.buckets:
            b.pending = len(b.params)
            b.work = None
            for p, g in zip(b.params, b.grad_views):
                p.grad = g

    # ---------------------------------------------------------------- backward
    def _make_hook(self, b: _Bucket):
        def hook(param):
            b.pending -= 1
            if b.pending == 0:
                self._launch(b)
        return hook

    def _launch(self, b: _Bucket) -> None:
        step = self.step_count + 1
        if self.pg is not None:
            b.work = self.pg.fused_allreduce_step(b.grads, b.flat, b.state1, b.state2, self.kind, self.lr, self.momentum,
                                                  self.dampening, self.weight_decay, self.betas[0], self.betas[1],
                                                  self.eps, step, self.nesterov, b.first, 1.0 / self.world)
        else:
            if self.kind == 0:
                torch.ops.catch_b200.fused_sgd_step([b.flat], [b.grads], [b.state1] if self.momentum != 0 else [], [],
                                                    self.lr, self.momentum, self.dampening, self.weight_decay,
                                                    self.nesterov, b.first, 1.0)
            else:
                torch.ops.catch_b200.fused_adamw_step([b.flat], [b.grads], [b.state1], [b.state2], [], self.lr,
                                                      self.betas[0], self.betas[1], self.eps, self.weight_decay, step,
                                                      1.0, False)
        b.first = False

    # -------------------------------------------------------------------- API
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def step(self) -> None:
        """Finish the optimizer step started during backward and re-arm the buckets."""
        for b in self.buckets:
            if b.pending != 0:
                # a parameter received no gradient this step: run the bucket now
                self._launch(b)
            if b.work is not None:
                b.work.wait()
        self.step_count += 1
        for b in self.buckets:
            b.grads.zero_()
        self._arm()

    def zero_grad(self, set_to_none: bool = False) -> None:  # gradients are zeroed by step()
        pass

    def set_lr(self, lr: float) -> None:
        self.lr = lr

    def state_dict_optimizer(self) -> dict:
        return {"step": self.step_count, "state1": [b.state1.cpu() for b in self.buckets],
                "state2": [b.state2.cpu() for b in self.buckets], "first": [b.first for b in self.buckets]}

    def load_state_dict_optimizer(self, sd: dict) -> None:
        self.step_count = sd["step"]
        for b, s1, s2, f in zip(self.buckets, sd["state1"], sd["state2"], sd["first"]):
            b.state1.copy_(s1)
            b.state2.copy_(s2)
            b.first = f
