"""Data parallelism whose gradient all-reduce is fused with the optimizer.

``FusedDataParallel`` replaces the three hot loops of a stock DDP step (the
Reducer's per-gradient copy-and-scale, the bucket all-reduce and the optimizer's
per-parameter kernels; see the reference's training call stack in
torch_mlu/csrc/distributed/process_group_cncl.cpp:334-356 and its user guide) by
ONE kernel per bucket that runs while the rest of backward is still computing:

* parameters and gradients live in symmetric (peer-mapped) memory, ``p.grad`` is a
  view of the bucket, so autograd accumulates straight into the communication buffer
  (convolutions of ``catch_b200.fusion`` add their weight gradient into it from inside
  the weight-gradient kernel);
* when the last gradient of a bucket has been produced, the bucket's kernel is queued
  on the communication queue: every rank pulls its shard of the bucket from all peers
  over NVLink, reduces in fp32, scales by 1/world, applies SGD-momentum or AdamW to its
  shard of the fp32 master parameters (optimizer state is sharded: 1/world per rank),
  pushes the updated parameters, and the 16-bit copy that autocast forward passes
  read, to every peer, and clears the gradients for the next step;
* ``step()`` only makes the compute queue wait for those kernels.

All ranks end every step with bit-identical parameters because each element is
updated by exactly one rank and then broadcast.  Buckets are always launched in bucket
order (a bucket waits for the ones before it), so every rank issues the same sequence
of kernels even when some parameters receive no gradient on some ranks.
"""
from __future__ import annotations

import contextlib
from typing import Dict, List, Optional

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
    def __init__(self, index: int, params: List[torch.nn.Parameter]):
        self.index = index
        self.params = params
        # every parameter starts on a 16-byte boundary of the flat fp32 buffers (kernels that add gradients into
        # the bucket address it with tensor maps); the few padding elements stay zero
        self.offsets: List[int] = []
        off = 0
        for p in params:
            off = (off + 3) // 4 * 4
            self.offsets.append(off)
            off += p.numel()
        self.numel = off
        self.pending = 0
        self.launched = False
        self.grads = None      # flat fp32 gradient buffer (p.grad are views of it)
        self.comm = None       # 16-bit exchange buffer (only with a 16-bit grad_dtype)
        self.flat = None       # symmetric flat fp32 parameter buffer
        self.lowp = None       # symmetric flat 16-bit parameter copy
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
            hyper-parameters (``set_lr`` changes the learning rate between steps).
        bucket_mb: bucket size in MiB (gradients are bucketed in reverse
            registration order, the order backward produces them in).
        grad_dtype: dtype in which gradients cross NVLink.  ``torch.float32`` exchanges
            the accumulation buffers in place; ``torch.bfloat16`` / ``torch.float16`` halve
            the traffic: the bucket kernel first converts this rank's fp32 gradients into a
            16-bit exchange buffer (the reduction itself stays fp32).
        lowp_dtype: keep a 16-bit copy of every parameter, refreshed by the bucket kernel,
            and publish it as ``param._b200_lowp`` (modules of ``catch_b200.fusion`` read
            it instead of casting the fp32 weight in every forward pass).  ``None`` = off.
        process_group: a ``bwccl`` group (default: the world group).

    Gradient accumulation: run the extra backward passes inside ``no_sync()``; the
    bucket kernels start during the first backward outside of it.  A second backward
    without ``step()`` or ``no_sync()`` raises.

    With a world size of one (or without an initialised process group) the same
    update runs on local memory through the fused single-device optimizers.
    """

    def __init__(self, module: torch.nn.Module, optimizer: str = "sgd", lr: float = 0.1, momentum: float = 0.0,
                 dampening: float = 0.0, weight_decay: float = 0.0, nesterov: bool = False, betas=(0.9, 0.999),
                 eps: float = 1e-8, bucket_mb: float = 25.0, grad_dtype: torch.dtype = torch.float32,
                 process_group=None, broadcast_buffers: bool = True,
                 lowp_dtype: Optional[torch.dtype] = torch.bfloat16):
        super().__init__()
        self.module = module
        self.kind = {"sgd": 0, "adamw": 1}[optimizer.lower()]
        self.lr, self.momentum, self.dampening, self.weight_decay = lr, momentum, dampening, weight_decay
        self.nesterov, self.betas, self.eps = nesterov, betas, eps
        if grad_dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise ValueError("grad_dtype must be float32, bfloat16 or float16")
        if lowp_dtype not in (None, torch.bfloat16, torch.float16):
            raise ValueError("lowp_dtype must be None, bfloat16 or float16")
        self.grad_dtype = grad_dtype
        self.lowp_dtype = lowp_dtype
        self.step_count = 0
        self.group = process_group or (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.pg = get_backend(self.group) if self.world > 1 else None
        self.broadcast_buffers = broadcast_buffers
        self._sync = True
        self._next = 0          # index of the next bucket to launch
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
                self.buckets.append(_Bucket(len(self.buckets), cur))
                cur, cur_n = [], 0
        if cur:
            self.buckets.append(_Bucket(len(self.buckets), cur))
        self._param_bucket: Dict[torch.nn.Parameter, _Bucket] = {}
        for b in self.buckets:
            self._setup_bucket(b)
        if self.world > 1:
            self._sync_initial_state()
        self.refresh_lowp()
        for b in self.buckets:
            for p in b.params:
                p.register_post_accumulate_grad_hook(self._grad_ready)
        module.register_load_state_dict_post_hook(lambda m, keys: self.refresh_lowp())
        self._arm()

    # ------------------------------------------------------------------ setup
    def _alloc(self, numel: int, dtype: torch.dtype, symmetric: bool = True) -> torch.Tensor:
        if self.pg is not None and symmetric:
            return self.pg.symm_empty(numel, dtype)
        return torch.empty(numel, dtype=dtype, device=self.device)

    def _padded(self, numel: int, dtype: torch.dtype) -> int:
        """Elements of a bucket buffer of `dtype`: every rank's shard is a whole number of 16-byte vectors."""
        if self.pg is not None:
            return self.pg.shard_elems(numel, dtype) * self.world
        return (numel + 7) // 8 * 8

    def _setup_bucket(self, b: _Bucket) -> None:
        comm16 = self.grad_dtype != torch.float32 and self.pg is not None
        n_pad = max(self._padded(b.numel, torch.float32), self._padded(b.numel, self.grad_dtype))
        b.flat = self._alloc(n_pad, torch.float32)[:b.numel]
        # fp32 accumulation buffer: exchanged in place (symmetric) or converted by the kernel (local)
        b.grads = self._alloc(n_pad, torch.float32, symmetric=not comm16)
        b.grads.zero_()
        b.comm = self._alloc(n_pad, self.grad_dtype) if comm16 else None
        if self.lowp_dtype is not None:
            b.lowp = self._alloc(n_pad, self.lowp_dtype)[:b.numel]
        b.flat.zero_()
        if b.lowp is not None:
            b.lowp.zero_()
        b.grad_views, b.flat_grads = [], []
        for p, off in zip(b.params, b.offsets):
            n = p.numel()
            view = _view_like(b.flat[off:off + n], p.data)
            view.copy_(p.data)
            b.grad_views.append(_view_like(b.grads[off:off + n], p.data))
            b.flat_grads.append(b.grads[off:off + n])
            p.data = view
            if b.lowp is not None:
                p._b200_lowp = _view_like(b.lowp[off:off + n], p.data)
            self._param_bucket[p] = b
        ex_dtype = self.grad_dtype if comm16 else torch.float32
        shard = self.pg.shard_elems(b.numel, ex_dtype) if self.pg is not None else b.numel
        b.state1 = torch.zeros(shard, dtype=torch.float32, device=self.device)
        b.state2 = torch.zeros(shard if self.kind == 1 else 0, dtype=torch.float32, device=self.device)

    def _sync_initial_state(self) -> None:
        for b in self.buckets:
            dist.broadcast(b.flat, 0, group=self.group)
        if self.broadcast_buffers:
            for buf in self.module.buffers():
                dist.broadcast(buf, 0, group=self.group)
        torch.b200.synchronize()

    def refresh_lowp(self) -> None:
        """Recompute the 16-bit parameter copies from the fp32 masters (after the parameters were changed
        by anything other than ``step()``: ``load_state_dict`` does this by itself)."""
        for b in self.buckets:
            if b.lowp is not None:
                b.lowp.copy_(b.flat)

    def _arm(self) -> None:
        self._next = 0
        for b in self.buckets:
            b.pending = len(b.params)
            b.launched = False
            b.work = None
            for p, g, fg in zip(b.params, b.grad_views, b.flat_grads):
                p.grad = g
                # modules that can add their gradient into the bucket themselves look for this
                p._b200_grad_acc = fg

    # ---------------------------------------------------------------- backward
    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside this context only accumulate gradients (no bucket kernels, no update)."""
        old, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = old

    def _grad_ready(self, param) -> None:
        if not self._sync:
            return
        b = self._param_bucket[param]
        if b.launched or b.pending <= 0:
            raise RuntimeError("FusedDataParallel: a parameter received a second gradient before step(); "
                               "wrap the extra backward passes in no_sync() to accumulate gradients")
        b.pending -= 1
        # strictly in bucket order: every rank launches the same kernels in the same order
        while self._next < len(self.buckets) and self.buckets[self._next].pending == 0:
            self._launch(self.buckets[self._next])
            self._next += 1

    def _launch(self, b: _Bucket) -> None:
        step = self.step_count + 1
        b.launched = True
        if self.pg is not None:
            grads = b.comm if b.comm is not None else b.grads
            b.work = self.pg.fused_allreduce_step(grads[:b.numel], b.flat, b.state1, b.state2, self.kind, self.lr,
                                                  self.momentum, self.dampening, self.weight_decay, self.betas[0],
                                                  self.betas[1], self.eps, step, self.nesterov, b.first,
                                                  1.0 / self.world, lowp=b.lowp,
                                                  cast_src=b.grads if b.comm is not None else None, zero_grads=True)
        else:
            lowp = [b.lowp] if b.lowp is not None else []
            g = b.grads[:b.numel]
            if self.kind == 0:
                torch.ops.catch_b200.fused_sgd_step([b.flat], [g], [b.state1] if self.momentum != 0 else [], lowp,
                                                    self.lr, self.momentum, self.dampening, self.weight_decay,
                                                    self.nesterov, b.first, 1.0)
            else:
                torch.ops.catch_b200.fused_adamw_step([b.flat], [g], [b.state1], [b.state2], lowp, self.lr,
                                                      self.betas[0], self.betas[1], self.eps, self.weight_decay, step,
                                                      1.0, False)
            b.grads.zero_()
        b.first = False

    # -------------------------------------------------------------------- API
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def step(self) -> None:
        """Finish the optimizer step started during backward and re-arm the buckets."""
        # buckets whose parameters did not all receive a gradient: launched here, still in bucket order
        while self._next < len(self.buckets):
            self._launch(self.buckets[self._next])
            self._next += 1
        for b in self.buckets:
            if b.work is not None:
                b.work.wait()
        self.step_count += 1
        self._arm()

    def zero_grad(self, set_to_none: bool = False) -> None:  # gradients are cleared by the bucket kernels
        pass

    def set_lr(self, lr: float) -> None:
        self.lr = lr

    # ------------------------------------------------------------- checkpoints
    def _gather_state(self, shard: torch.Tensor, b: _Bucket) -> torch.Tensor:
        """The full flat optimizer-state vector of a bucket (rank r holds elements [r * shard, (r + 1) * shard))."""
        if self.pg is None:
            return shard[:b.numel].clone()
        full = torch.empty(shard.numel() * self.world, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        return full[:b.numel]

    def optimizer_state_dict(self) -> dict:
        """Optimizer state in the layout of ``torch.optim.SGD`` / ``torch.optim.AdamW`` ``state_dict()``:
        per-parameter ``momentum_buffer`` or ``exp_avg`` / ``exp_avg_sq`` / ``step`` entries, indexed in
        ``module.parameters()`` order, plus one param group.  Every rank must call it (the shards are
        all-gathered); the result does not depend on the world size, so a checkpoint written at 8 ranks
        resumes at 4, at 1, or in the stock optimizer (``torch.optim.SGD.load_state_dict``)."""
        order = {p: i for i, p in enumerate(p for p in self.module.parameters() if p.requires_grad)}
        state: Dict[int, dict] = {}
        for b in self.buckets:
            s1 = self._gather_state(b.state1, b) if (self.kind == 1 or self.momentum != 0) else None
            s2 = self._gather_state(b.state2, b) if self.kind == 1 else None
            for p, off in zip(b.params, b.offsets):
                n = p.numel()
                if self.step_count == 0:
                    continue

                def piece(flat):
                    return _view_like(flat[off:off + n], p.data).detach().cpu().clone()

                if self.kind == 0:
                    if s1 is not None:
                        state[order[p]] = {"momentum_buffer": piece(s1)}
                else:
                    state[order[p]] = {"step": torch.tensor(float(self.step_count)), "exp_avg": piece(s1),
                                       "exp_avg_sq": piece(s2)}
        if self.kind == 0:
            group = {"lr": self.lr, "momentum": self.momentum, "dampening": self.dampening,
                     "weight_decay": self.weight_decay, "nesterov": self.nesterov, "maximize": False, "foreach": None,
                     "differentiable": False, "fused": None}
        else:
            group = {"lr": self.lr, "betas": tuple(self.betas), "eps": self.eps, "weight_decay": self.weight_decay,
                     "amsgrad": False, "maximize": False, "foreach": None, "capturable": False,
                     "differentiable": False, "fused": None, "decoupled_weight_decay": True}
        group["params"] = list(range(len(order)))
        return {"state": state, "param_groups": [group]}

    def load_optimizer_state_dict(self, sd: dict) -> None:
        """Load a state dict produced by ``optimizer_state_dict()`` at any world size or by the stock
        ``torch.optim.SGD`` / ``AdamW`` over the same parameters."""
        order = {p: i for i, p in enumerate(p for p in self.module.parameters() if p.requires_grad)}
        group = sd["param_groups"][0]
        self.lr = group.get("lr", self.lr)
        state = sd["state"]
        steps = [int(v["step"]) for v in state.values() if "step" in v]
        rank = dist.get_rank(self.group) if self.pg is not None else 0
        any_state = False
        for b in self.buckets:
            shard = b.state1.numel()
            full1 = torch.zeros(shard * self.world, dtype=torch.float32)
            full2 = torch.zeros(shard * self.world if self.kind == 1 else 0, dtype=torch.float32)
            for p, off in zip(b.params, b.offsets):
                st = state.get(order[p], state.get(str(order[p])))
                if not st:
                    continue
                any_state = True
                n = p.numel()

                def put(full, t):
                    _view_like(full[off:off + n], p.data).copy_(t.to(torch.float32))

                if self.kind == 0 and st.get("momentum_buffer") is not None:
                    put(full1, st["momentum_buffer"])
                elif self.kind == 1:
                    put(full1, st["exp_avg"])
                    put(full2, st["exp_avg_sq"])
            b.state1.copy_(full1[rank * shard:(rank + 1) * shard])
            if self.kind == 1:
                b.state2.copy_(full2[rank * shard:(rank + 1) * shard])
            b.first = not any_state
        if steps:
            self.step_count = max(steps)
        elif any_state:
            self.step_count = max(self.step_count, 1)

    # former names, kept for callers of the first version of this class
    state_dict_optimizer = optimizer_state_dict
    load_state_dict_optimizer = load_optimizer_state_dict
