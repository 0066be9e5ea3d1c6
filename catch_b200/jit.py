"""TorchScript fusion mode.

* ``set_fusion_enabled(bool)`` / ``fusion_enabled()`` -- the global toggle (the
  reference's ``_jit_override_can_fuse_on_mlu`` / ``_jit_can_fuse_on_mlu``,
  torch_mlu/csrc/jit/interface.cpp:36-45).
* ``optimize(module, example_inputs=None)`` -- freeze an eval-mode scripted / traced
  module (folds batch norm into the preceding convolution), lower the graph, rewrite
  conv(+BN)+ReLU(+residual) and linear+bias(+activation) chains into the backend's fused
  tcgen05 ops and group supported nodes into ``catch_b200::FusionGroup`` nodes.
* The same passes are registered as graph-executor pre-passes, so a scripted module
  that was not explicitly optimised still gets fusion groups on its first run.

* A fusion group whose inputs are all device tensors is captured as a device graph on its third call with the same
  shapes; later calls copy the inputs into the graph's buffers and replay it with one submission
  (``CATCH_B200_JIT_GRAPHS=0`` keeps the interpreter).

Environment: ``CATCH_B200_FORCED_FALLBACK_OPS=a,b`` keeps the listed ops out of fusion
groups; ``CATCH_B200_FUSED_KERNEL_DEBUG=cpu`` also runs every group on the CPU and
writes both results to ``fused_kernel_<n>_{device,cpu}.pt``.
"""
from __future__ import annotations

import torch

from . import _C

_C._jit_register_passes()


def fusion_enabled() -> bool:
    return _C._jit_can_fuse_on_b200()


def set_fusion_enabled(enable: bool) -> None:
    _C._jit_override_can_fuse_on_b200(bool(enable))


def lower_graph(graph) -> None:
    _C._jit_pass_lower_graph(graph)


def fuse_kernels(graph) -> None:
    _C._jit_pass_fuse_kernels(graph)


def segment_graph(graph) -> None:
    _C._jit_pass_segment_graph(graph)


def unfuse_graph(graph) -> None:
    _C._jit_pass_unfuse_graph(graph)


def save(module: torch.jit.ScriptModule, f, _extra_files=None) -> None:
    """``torch.jit.save`` for a module that went through ``optimize``: fusion groups are dissolved first (a group's
    subgraph cannot be written to a file); the fused operators themselves (``catch_b200::conv_bn_act`` ...) are
    ordinary registered operators and are saved as they are.  The groups of ``module`` are rebuilt after the file
    is written.  Load with ``catch_b200.jit.load`` (or ``torch.jit.load`` after importing this package)."""
    graph = module.forward.graph if hasattr(module, "forward") else None
    if graph is not None:
        unfuse_graph(graph)
    try:
        torch.jit.save(module, f, _extra_files=_extra_files)
    finally:
        if graph is not None and fusion_enabled():
            segment_graph(graph)


def load(f, map_location=None, _extra_files=None) -> torch.jit.ScriptModule:
    """``torch.jit.load`` followed by the segmentation pass (parameters and constants go to ``map_location``, e.g.
    ``"blackwell"``)."""
    m = torch.jit.load(f, map_location=map_location, _extra_files=_extra_files)
    if fusion_enabled() and hasattr(m, "forward"):
        segment_graph(m.forward.graph)
    return m


def fusion_stats() -> dict:
    return {"runners": _C._jit_fusion_cache_size(), "compiles": _C._jit_fusion_compile_count(),
            "fallbacks": _C._jit_fusion_fallback_count(), "graph_captures": _C._jit_fusion_graph_capture_count(),
            "graph_replays": _C._jit_fusion_graph_replay_count()}


def optimize(module: torch.jit.ScriptModule, preserved_attrs=None) -> torch.jit.ScriptModule:
    """Freeze ``module`` (must be in eval mode) and run the fusion passes on its forward graph."""
    if module.training:
        raise ValueError("catch_b200.jit.optimize expects a module in eval() mode")
    frozen = torch.jit.freeze(module, preserved_attrs=preserved_attrs or [])
    graph = frozen.graph
    torch._C._jit_pass_fold_frozen_conv_bn(graph)
    torch._C._jit_pass_fold_frozen_conv_add_or_sub(graph)
    torch._C._jit_pass_fold_frozen_conv_mul_or_div(graph)
    if fusion_enabled():
        lower_graph(graph)
        fuse_kernels(graph)
        segment_graph(graph)
    return frozen
