"""Training-time module fusion: batch norm + (residual add) + ReLU in one kernel pair.

    model = catch_b200.fusion.fuse_bn_act(model)      # torch.fx rewrite, same state_dict

Every ``BatchNorm2d -> ReLU`` and ``BatchNorm2d -> add(residual) -> ReLU`` chain of an
fx-traceable model (torchvision ResNets are) is replaced by ``BatchNormAct2d``, a
``BatchNorm2d`` subclass (same parameters and buffers, same state-dict keys) whose
forward calls ``torch.ops.catch_b200.batch_norm_act``: the normalisation, the residual
add and the ReLU are applied in one pass over the activation, and the backward masks
the gradient inside the batch-norm reduction and apply kernels instead of running a
separate ReLU backward.  The reference has no counterpart (its fusion exists only in
inference mode); on B200 the batch-norm and activation passes are memory-bound and
dominate a ResNet step, which is why they are fused here.
"""
from __future__ import annotations

import operator
from typing import Optional

import os

import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F


class _GradSink:
    """Meeting point for the gradients that reach one activation tensor over several paths of a residual block.

    A tensor that feeds a fused convolution (and, as the skip connection, a fused batch norm + add) would receive one
    gradient per consumer and autograd would add them with an element-wise kernel per fork.  Instead every fused
    convolution that consumes the tensor registers here in the forward pass; in the backward pass a consumer that is
    not the last one to run parks its gradient here and returns none, and the last convolution hands the parked
    gradient to its data-gradient kernel, whose epilogue adds it.  The skip connection's batch norm runs before the
    convolutions of its block (it was created after them), so it always parks."""

    __slots__ = ("consumers", "remaining", "pending")

    def __init__(self):
        self.consumers = 0
        self.remaining = 0
        self.pending = None

    def park(self, grad):
        self.pending = grad if self.pending is None else self.pending + grad
        # every parked gradient has to be picked up before the backward pass ends: check when it does
        if not _open_sinks:
            torch.autograd.Variable._execution_engine.queue_callback(_check_sinks)
        _open_sinks.append(self)

    def take(self):
        grad, self.pending = self.pending, None
        return grad


_SINKS_ENABLED = os.environ.get("CATCH_B200_GRAD_SINKS", "1") != "0"
_open_sinks = []


def _check_sinks() -> None:
    """Runs when a backward pass ends: a gradient that is still parked was never added to anything (a registered
    consumer's backward did not run, e.g. because its output does not reach the loss)."""
    lost = [s for s in _open_sinks if s.pending is not None]
    for s in _open_sinks:
        s.pending = None
        s.remaining = s.consumers
    _open_sinks.clear()
    if lost:
        raise RuntimeError("catch_b200.fusion: a gradient parked at a residual fork was not consumed in this backward pass "
                           "(a fused convolution that reads the same tensor took no part in it); call "
                           "catch_b200.fusion.set_gradient_sinks(False) for this model")


def set_gradient_sinks(enabled: bool) -> None:
    """Fold the gradient additions at residual forks into the data-gradient kernels (default on)."""
    global _SINKS_ENABLED
    _SINKS_ENABLED = bool(enabled)


def _sink_for(x: torch.Tensor, create: bool) -> Optional["_GradSink"]:
    if not (_SINKS_ENABLED and torch.is_grad_enabled() and x.requires_grad):
        return None
    sink = getattr(x, "_b200_grad_sink", None)
    if sink is None and create:
        sink = _GradSink()
        x._b200_grad_sink = sink
    return sink


class _BNActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, residual, training, momentum, eps, act, sums=None,
                num_batches_tracked=None, res_sink=None):
        out, mean, invstd, mask = torch.ops.catch_b200.batch_norm_act_mask(x, weight, bias, running_mean, running_var,
                                                                           residual, training, momentum, eps, act, sums,
                                                                           num_batches_tracked)
        # with a ReLU the backward only needs to know which outputs were positive: one bit each; without one it does
        # not need the output at all (and must not hold it: an in-place activation such as ReLU6(inplace=True) or
        # SiLU(inplace=True) right behind the batch norm would invalidate a saved output)
        ctx.save_for_backward((mask if mask.numel() else out) if act == 1 else None, x, weight, running_mean, mean, invstd)
        ctx.cfg = (training, act, residual is not None)
        ctx.res_sink = res_sink
        return out

    @staticmethod
    def backward(ctx, grad_out):
        out, x, weight, running_mean, mean, invstd = ctx.saved_tensors
        training, act, has_res = ctx.cfg
        if out is None:  # no activation: the operator ignores this argument, any tensor of the right shape will do
            out = grad_out
        dx, dgamma, dbeta, dres = torch.ops.catch_b200.batch_norm_act_backward(
            grad_out, out, x, weight, running_mean, mean, invstd, training, act, has_res)
        sink = ctx.res_sink
        if has_res and sink is not None and sink.remaining > 0:
            sink.park(dres)  # a convolution that also consumes the skip tensor adds it in its data-gradient epilogue
            dres = None
        return (dx, dgamma if weight is not None else None, dbeta if weight is not None else None, None, None,
                dres if has_res else None, None, None, None, None, None, None, None)


class _ConvStatsFn(torch.autograd.Function):
    """Convolution whose epilogue also accumulates per-channel sum / sum of squares of the output.

    ``weight`` is the (fp32) parameter itself.  Its 16-bit compute copy is ``weight._b200_lowp`` when a data-parallel
    wrapper maintains one (refreshed by the optimizer kernel), else a cast made here.  The backward returns the
    weight gradient in fp32 straight from the weight-gradient kernel's accumulation buffer (no rounding to 16 bits,
    no cast kernels); when the parameter's gradient lives in a flat bucket (``weight._b200_grad_acc``, the flat
    fp32 slice behind ``weight.grad``) the kernel adds into that bucket directly."""

    @staticmethod
    def forward(ctx, x, weight, stride, padding, compute_dtype, sink=None):
        ctx.sink = sink
        lowp = getattr(weight, "_b200_lowp", None)
        if weight.dtype == compute_dtype:
            w = weight
        elif lowp is not None and lowp.dtype == compute_dtype and lowp.shape == weight.shape:
            w = lowp
        else:
            w = weight.to(compute_dtype)
        y, sums = torch.ops.catch_b200.conv2d_stats(x, w, stride, padding)
        ctx.save_for_backward(x, w)
        ctx.cfg = (stride, padding, weight.dtype)
        ctx.param = weight
        ctx.mark_non_differentiable(sums)
        return y, sums

    @staticmethod
    def backward(ctx, grad_y, _grad_sums):
        x, w = ctx.saved_tensors
        stride, padding, wdtype = ctx.cfg
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        sink = ctx.sink if need_dx else None
        parked = None
        if sink is not None:
            parked = sink.take()
            sink.remaining -= 1

        def finish(dx):
            """Park the input gradient for a later consumer of the same tensor, or hand the total to autograd."""
            if sink is None:
                return dx
            if sink.remaining > 0:
                sink.park(dx)
                return None
            sink.remaining = sink.consumers  # ready for another backward pass over the same graph
            return dx

        if wdtype == torch.float32:
            acc = getattr(ctx.param, "_b200_grad_acc", None) if need_dw else None
            p = ctx.param
            # the bucket slice must hold the gradient as [K][R][S][C]: channels-last parameters and 1x1 filters do
            if (acc is not None and p.grad is not None and p.grad.dtype == torch.float32 and p.dim() == 4
                    and (p.shape[2] * p.shape[3] == 1 or p.is_contiguous(memory_format=torch.channels_last))):
                # The parameter's post-accumulate-grad hook still fires for the undefined gradient returned
                # here, after this function has queued the kernel: that is what tells the bucket's owner.
                dx, _ = torch.ops.catch_b200.conv2d_backward_fp32w(grad_y, x, w, stride, padding, need_dx, True, acc, parked)
                return finish(dx), None, None, None, None, None
            dx, dw = torch.ops.catch_b200.conv2d_backward_fp32w(grad_y, x, w, stride, padding, need_dx, need_dw, None, parked)
        else:
            dx, dw, _ = torch.ops.aten.convolution_backward(grad_y, x, w, None, stride, padding, [1, 1], False, [0, 0], 1,
                                                            [need_dx, need_dw, False])
            if parked is not None and dx is not None:
                dx = dx + parked
        return finish(dx), dw, None, None, None, None


class StatsConv2d(nn.Conv2d):
    """``Conv2d`` feeding a batch norm: in training it hands the batch norm the channel sums of its
    output (computed in the convolution epilogue), which saves the batch norm's statistics pass over
    the activation.  The sums travel as an attribute of the returned tensor object."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if (self.training and _device_kernels_available(x) and x.dim() == 4 and self.bias is None and self.groups == 1
                and self.padding_mode == "zeros" and self.dilation == (1, 1) and not isinstance(self.padding, str)
                and all(s in (1, 2) for s in self.stride) and self.in_channels % 8 == 0 and self.out_channels % 64 == 0
                and x.numel() > 0):
            autocast = torch.is_autocast_enabled("blackwell")
            if autocast:
                x = x.to(torch.get_autocast_dtype("blackwell"))
            if x.dtype in (torch.bfloat16, torch.float16) and (self.weight.dtype == x.dtype or
                                                              (autocast and self.weight.dtype == torch.float32)):
                sink = _sink_for(x, create=True)
                if sink is not None:
                    sink.consumers += 1
                    sink.remaining += 1
                y, sums = _ConvStatsFn.apply(x, self.weight, list(self.stride), list(self.padding), x.dtype, sink)
                y._b200_channel_sums = sums
                return y
        return super().forward(x)


_FUSED_ON_HOST = os.environ.get("CATCH_B200_FUSION_ON_HOSTSIM", "0") == "1"


def fused_ops_on_host(enabled: bool) -> None:
    """Under host simulation the fused modules normally fall back to the stock layers.  With this switch (or
    ``CATCH_B200_FUSION_ON_HOSTSIM=1``) they take the same autograd functions as on the device, whose operators then
    run their host paths: for testing the bookkeeping around them (gradient sinks, direct accumulation into gradient
    buckets, 16-bit weight copies, the transformer fusions) without a GPU."""
    global _FUSED_ON_HOST
    _FUSED_ON_HOST = bool(enabled)


def _device_kernels_available(x: torch.Tensor) -> bool:
    return x.device.type == "blackwell" and (_FUSED_ON_HOST or not torch.b200.is_hostsim())


class BatchNormAct2d(nn.BatchNorm2d):
    """``BatchNorm2d`` followed by an optional residual add and ReLU, fused on the device."""

    act: int = 1

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        training = self.training or (self.running_mean is None and self.running_var is None)
        momentum = 0.0 if self.momentum is None else self.momentum
        count_batch = self.training and self.track_running_stats and self.num_batches_tracked is not None
        if count_batch and self.momentum is None:
            # cumulative moving average: the count is needed on the host
            self.num_batches_tracked.add_(1)
            momentum = 1.0 / float(self.num_batches_tracked)
            count_batch = False
        rm = self.running_mean if (not self.training or self.track_running_stats) else None
        rv = self.running_var if (not self.training or self.track_running_stats) else None
        c_vec = 4 if x.dtype == torch.float32 else 8
        if (_device_kernels_available(x) and x.dim() == 4 and x.shape[1] % c_vec == 0
                and x.dtype in (torch.float32, torch.bfloat16, torch.float16) and x.numel() > 0
                and (residual is None or (residual.shape == x.shape and residual.dtype == x.dtype))):
            sums = getattr(x, "_b200_channel_sums", None) if training else None
            # the fused kernel also increments num_batches_tracked (no separate tiny launch per batch norm)
            res_sink = _sink_for(residual, create=False) if residual is not None else None
            return _BNActFn.apply(x, self.weight, self.bias, rm, rv, residual, training, momentum, self.eps, self.act,
                                  sums, self.num_batches_tracked if count_batch else None, res_sink)
        if count_batch:
            self.num_batches_tracked.add_(1)
        y = F.batch_norm(x, rm, rv, self.weight, self.bias, training, momentum, self.eps)
        if residual is not None:
            y = y + residual
        return F.relu(y) if self.act == 1 else y


class _LinearFn(torch.autograd.Function):
    """``x @ weight^T + bias`` in a 16-bit compute dtype with fp32 master parameters.

    Forward reads the parameter's 16-bit copy (``weight._b200_lowp``, kept current by the data-parallel wrapper's
    optimizer kernel) instead of casting the weight; backward computes the weight gradient in fp32 with the K
    dimension (all tokens) split over the whole GPU and adds it, like the bias gradient, straight into the
    parameter's gradient bucket when there is one (``param._b200_grad_acc``)."""

    @staticmethod
    def forward(ctx, x, weight, bias, compute_dtype):
        lowp = getattr(weight, "_b200_lowp", None)
        if weight.dtype == compute_dtype:
            w = weight
        elif lowp is not None and lowp.dtype == compute_dtype and lowp.shape == weight.shape:
            w = lowp
        else:
            w = weight.to(compute_dtype)
        y = torch.ops.catch_b200.linear_act(x, w, bias, 0)
        ctx.save_for_backward(x, w)
        ctx.params = (weight, bias)
        return y

    @staticmethod
    def backward(ctx, grad):
        x, w = ctx.saved_tensors
        weight, bias = ctx.params
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_db = bias is not None and ctx.needs_input_grad[2]

        def bucket(p, need):
            acc = getattr(p, "_b200_grad_acc", None) if (need and p is not None) else None
            return acc if (acc is not None and p.grad is not None and p.grad.dtype == torch.float32 and p.dtype == torch.float32) else None

        acc_w, acc_b = bucket(weight, need_dw), bucket(bias, need_db)
        dx, dw, db = torch.ops.catch_b200.linear_backward_fp32w(grad, x, w, need_dx, need_dw, need_db, acc_w, acc_b)
        if dw is not None and weight.dtype != torch.float32:
            dw = dw.to(weight.dtype)
        if db is not None and bias.dtype != torch.float32:
            db = db.to(bias.dtype)
        # gradients that went into a bucket come back undefined; the parameters' post-accumulate hooks still fire
        return dx, dw, db, None


class FusedLinear(nn.Linear):
    """``nn.Linear`` whose autocast path runs through ``_LinearFn`` (same parameters, same state dict)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if _device_kernels_available(x) and x.numel() > 0 and self.in_features % 8 == 0 and self.out_features % 8 == 0:
            autocast = torch.is_autocast_enabled("blackwell")
            cd = torch.get_autocast_dtype("blackwell") if autocast else x.dtype
            if cd in (torch.bfloat16, torch.float16) and (autocast or self.weight.dtype == x.dtype):
                if x.dtype != cd:
                    x = x.to(cd)
                with torch.autocast("blackwell", enabled=False):
                    return _LinearFn.apply(x, self.weight, self.bias, cd)
        return super().forward(x)


def fuse_linear(model: nn.Module) -> nn.Module:
    """Switch every plain ``nn.Linear`` of ``model`` to ``FusedLinear`` in place (returns the model)."""
    for m in model.modules():
        if type(m) is nn.Linear:
            m.__class__ = FusedLinear
    return model


def _empty_with_layout_of(t: torch.Tensor) -> torch.Tensor:
    """An uninitialised tensor with t's shape and, when t is a dense permutation of its memory, t's strides."""
    extent = 1 + sum((n - 1) * st for n, st in zip(t.shape, t.stride()))
    if t.numel() > 0 and all(st > 0 for st in t.stride()) and extent == t.numel():
        return torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=t.device)
    return torch.empty_like(t, memory_format=torch.contiguous_format)


class _MatmulNdFn(torch.autograd.Function):
    """``alpha * a @ b`` over 4-D operands with arbitrary batch strides (``torch.ops.catch_b200.gemm_nd``).

    Head-split views ``[batch, heads, seq, dim]`` of ``[batch, seq, heads * dim]`` activations are multiplied as they
    are; gradients are produced in the memory layout of the operand they belong to, so the view / permute nodes
    around the call never have to copy either."""

    @staticmethod
    def forward(ctx, a, b, alpha, out_strides):
        ctx.save_for_backward(a, b)
        ctx.alpha = alpha
        out = None
        if out_strides is not None:
            out = torch.empty_strided(a.shape[:3] + b.shape[3:], out_strides, dtype=a.dtype, device=a.device)
        return torch.ops.catch_b200.gemm_nd(a, b, out, alpha)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        da = db = None
        if ctx.needs_input_grad[0]:
            da = _empty_with_layout_of(a)
            torch.ops.catch_b200.gemm_nd(g, b.transpose(-1, -2), da, ctx.alpha)
        if ctx.needs_input_grad[1]:
            db = _empty_with_layout_of(b)
            if db.stride(-1) != 1:   # the kernel writes rows: produce the transposed product into the transposed view
                torch.ops.catch_b200.gemm_nd(g.transpose(-1, -2), a, db.transpose(-1, -2), ctx.alpha)
            else:
                torch.ops.catch_b200.gemm_nd(a.transpose(-1, -2), g, db, ctx.alpha)
        return da, db, None, None


def matmul_nd(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, out_strides=None) -> torch.Tensor:
    """Batched ``alpha * a @ b`` for 4-D 16-bit tensors on the device without copying strided operands.
    ``out_strides`` (optional, innermost 1) chooses the memory layout of the result, e.g. that of a
    ``[batch, seq, heads, dim]`` buffer seen as ``[batch, heads, seq, dim]``."""
    return _MatmulNdFn.apply(a, b, alpha, out_strides)


class _DropoutAddLayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, residual, weight, bias, p, training, eps):
        y, s, mask, mean, rstd = torch.ops.catch_b200.dropout_add_layer_norm(h, residual, weight, bias, p, training, eps)
        ctx.save_for_backward(s, mask, weight, mean, rstd)
        ctx.p = p if training else 0.0
        ctx.params = (weight, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        s, mask, weight, mean, rstd = ctx.saved_tensors
        ds, dh, dgamma, dbeta = torch.ops.catch_b200.dropout_add_layer_norm_backward(dy, s, mask, weight, mean, rstd, ctx.p)
        w, b = ctx.params
        return (dh, ds, dgamma.to(w.dtype) if w is not None else None, dbeta.to(b.dtype) if b is not None else None,
                None, None, None)


def dropout_add_layer_norm(h: torch.Tensor, residual: torch.Tensor, norm: nn.LayerNorm, p: float, training: bool) -> torch.Tensor:
    """``norm(residual + dropout(h))`` as one kernel (forward) and one kernel (backward) on the device."""
    ok = (_device_kernels_available(h) and h.dtype in (torch.bfloat16, torch.float16, torch.float32) and h.dtype == residual.dtype
          and h.shape == residual.shape and len(norm.normalized_shape) == 1 and h.shape[-1] % 4 == 0 and h.shape[-1] <= 1536
          and h.numel() > 0)
    if not ok:
        return norm(residual + F.dropout(h, p, training))
    with torch.autocast("blackwell", enabled=False):
        return _DropoutAddLayerNormFn.apply(h, residual, norm.weight, norm.bias, float(p), bool(training), float(norm.eps))


def _feeds_only(node: fx.Node, consumer: fx.Node) -> bool:
    return len(node.users) == 1 and next(iter(node.users)) is consumer


def _is_relu(node: fx.Node, modules) -> bool:
    if node.op == "call_module":
        return isinstance(modules[node.target], nn.ReLU)
    if node.op == "call_function":
        return node.target in (F.relu, torch.relu, torch.relu_)
    if node.op == "call_method":
        return node.target in ("relu", "relu_")
    return False


def _is_add(node: fx.Node) -> bool:
    if node.op == "call_function" and node.target in (operator.add, operator.iadd, torch.add):
        return len(node.args) == 2 and all(isinstance(a, fx.Node) for a in node.args) and not node.kwargs
    if node.op == "call_method" and node.target in ("add", "add_"):
        return len(node.args) == 2 and all(isinstance(a, fx.Node) for a in node.args) and not node.kwargs
    return False


class _FusionTracer(fx.Tracer):
    """Traces only as deep as the rewrite needs: a sub-module without a convolution or batch norm inside stays one
    call (torchvision's StochasticDepth, custom activations, attention blocks ...).  Tracing into such a module would
    freeze its Python-level decisions, ``self.training`` above all, at their value on the day of the trace."""

    def is_leaf_module(self, m: nn.Module, module_qualified_name: str) -> bool:
        if super().is_leaf_module(m, module_qualified_name):
            return True
        return not any(isinstance(c, (nn.Conv2d, nn.BatchNorm2d)) for c in m.modules())


def fuse_bn_act(model: nn.Module) -> fx.GraphModule:
    """Return an fx GraphModule of ``model`` with BN(+add)+ReLU chains fused (see module docstring).

    A ``Conv2d`` whose only consumer is a batch norm becomes a ``StatsConv2d`` and that batch norm a
    ``BatchNormAct2d`` (with ``act = 0`` when no ReLU follows), so the convolution's epilogue supplies
    the batch statistics."""
    gm = fx.GraphModule(model, _FusionTracer().trace(model))
    modules = dict(gm.named_modules())
    fused = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_module" or type(modules[node.target]) is not nn.BatchNorm2d:
            continue
        bn = modules[node.target]
        src = node.args[0] if node.args else None
        if (isinstance(src, fx.Node) and src.op == "call_module" and type(modules[src.target]) is nn.Conv2d
                and _feeds_only(src, node)):
            modules[src.target].__class__ = StatsConv2d
            bn.__class__ = BatchNormAct2d  # consumes the statistics; stays activation-free unless a chain is fused below
            bn.act = 0
        user = next(iter(node.users)) if len(node.users) == 1 else None
        residual, relu_node, add_node = None, None, None
        if user is not None and _is_relu(user, modules):
            relu_node = user
        elif (user is not None and _is_add(user) and len(user.users) == 1 and _is_relu(next(iter(user.users)), modules)):
            add_node, relu_node = user, next(iter(user.users))
            residual = user.args[1] if user.args[0] is node else user.args[0]
            if residual is node:
                continue
        else:
            continue
        bn.__class__ = BatchNormAct2d
        bn.act = 1
        # the residual must be computed before the fused node: place the fused call where the ReLU was
        with gm.graph.inserting_before(relu_node):
            args = (node.args[0],) if residual is None else (node.args[0], residual)
            new = gm.graph.call_module(node.target, args)
        relu_node.replace_all_uses_with(new)
        gm.graph.erase_node(relu_node)
        if add_node is not None:
            gm.graph.erase_node(add_node)
        gm.graph.erase_node(node)
        fused += 1
    gm.graph.lint()
    gm.recompile()
    gm.fused_bn_act_count = fused
    return gm
