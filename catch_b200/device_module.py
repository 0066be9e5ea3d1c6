"""The ``torch.b200`` device module.

API parity with ``torch.mlu`` of the reference (torch_mlu/core/mlu_model.py:48-544,
torch_mlu/core/device/{queue,notifier,device}.py): device management, queues and
notifiers, memory statistics, legacy tensor constructors, ``torch.load`` with a
``map_location`` naming the device, seeds, optimizer ``to``, memory debugging,
pinning, and the fusion toggle.  Names that PyTorch's generic accelerator code
looks up on a device module (``current_stream``, ``Stream``, ``Event``,
``get_amp_supported_dtype`` ...) are provided as well.
"""
from __future__ import annotations

import contextlib
import warnings
from typing import Any, Optional, Union

import torch

from . import _C  # type: ignore[attr-defined]

DEVICE_TYPE = "blackwell"
_device_t = Union[torch.device, str, int, None]
_initialized = False


# --------------------------------------------------------------------------- device
def init() -> None:
    """Initialise the device runtime (lazy; calling it is optional)."""
    global _initialized
    if not _initialized:
        _C._device_count()
        _initialized = True


def _lazy_init() -> None:
    init()


def is_initialized() -> bool:
    return _initialized


def is_available() -> bool:
    return _C._device_count() > 0


def is_hostsim() -> bool:
    """True when the device is simulated in host memory (no GPU visible)."""
    return _C._is_hostsim()


def backend_name() -> str:
    return _C._backend_name()


def device_count() -> int:
    return _C._device_count()


def _get_device_index(device: Any, optional: bool = False) -> int:
    if device is None:
        if optional:
            return current_device()
        raise ValueError("Expected a b200 device, but got None")
    if isinstance(device, int):
        return device if device >= 0 else current_device()
    if isinstance(device, str):
        device = torch.device(device)
    if isinstance(device, torch.device):
        if device.type == "cuda":  # scripts written for GPUs keep working
            device = torch.device(DEVICE_TYPE, device.index)
        if device.type != DEVICE_TYPE:
            raise ValueError(f"Expected a b200 device, but got: {device}")
        return device.index if device.index is not None else current_device()
    if isinstance(device, (Queue,)):
        return device.device_index
    raise ValueError(f"Cannot interpret {device!r} as a b200 device")


def set_device(device: _device_t) -> None:
    idx = _get_device_index(device)
    if idx >= 0:
        _C._set_device(idx)


def current_device() -> int:
    return _C._current_device()


def get_device() -> int:
    return current_device()


def b200_device() -> torch.device:
    """``torch.device`` of the current b200 device."""
    return torch.device(DEVICE_TYPE, current_device())


class device:
    """Context manager that changes the selected device."""

    def __init__(self, device: _device_t):
        self.idx = _get_device_index(device, optional=True)
        self.prev_idx = -1

    def __enter__(self):
        self.prev_idx = current_device()
        if self.idx != -1 and self.idx != self.prev_idx:
            set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev_idx != -1 and self.prev_idx != current_device():
            set_device(self.prev_idx)
        return False


Device = device


class device_of(device):
    """Context manager that selects the device of the given tensor (no-op for CPU tensors)."""

    def __init__(self, obj: torch.Tensor):
        idx = obj.device.index if is_b200_tensor(obj) else -1
        super().__init__(idx)


def get_device_properties(device: _device_t = None):
    return _C._get_device_properties(_get_device_index(device, optional=True))


def get_device_name(device: _device_t = None) -> str:
    return get_device_properties(device).name


def get_device_capability(device: _device_t = None):
    p = get_device_properties(device)
    return p.major, p.minor


def synchronize(device: _device_t = None) -> None:
    _C._synchronize(_get_device_index(device, optional=True))


def is_b200_tensor(t: Any) -> bool:
    return isinstance(t, torch.Tensor) and t.device.type == DEVICE_TYPE


def get_version() -> str:
    return _C._get_version()


# ------------------------------------------------------------------ queues / notifiers
class Queue:
    """An ordered queue of device work (a CUDA stream).

    ``Queue()`` names the current queue of the device; used as a context manager
    it takes a queue from the per-device pool, makes it current (switching the
    device if needed) and restores the previous one on exit
    (reference: torch_mlu/core/device/queue.py:35-61).
    """

    def __init__(self, device_index: int = -1, _native=None, device=None, priority: int = 0):
        # `device` / `priority`: the keywords of torch.cuda.Stream (queues of the pool have one priority)
        if device is not None:
            device_index = _get_device_index(device, optional=True)
        self._native = _native if _native is not None else _C._getCurrentQueue(device_index)
        self._prev = None
        self._prev_device = None

    @property
    def device_index(self) -> int:
        return self._native.device_index

    @property
    def device(self) -> torch.device:
        return torch.device(DEVICE_TYPE, self._native.device_index)

    @property
    def queue_id(self) -> int:
        return self._native.id

    @property
    def native_handle(self) -> int:
        return self._native.handle

    # torch.Stream-like spelling
    cuda_stream = native_handle

    def query(self) -> bool:
        return self._native.query()

    def synchronize(self) -> None:
        self._native.synchronize()

    def record_event(self, event: Optional["Notifier"] = None) -> "Notifier":
        event = event or Notifier()
        event.place(self)
        return event

    def wait_event(self, event: "Notifier") -> None:
        event.wait(self)

    def wait_stream(self, other: "Queue") -> None:
        self.wait_event(other.record_event(Notifier(enable_timing=False)))

    def __eq__(self, other) -> bool:
        return isinstance(other, Queue) and self._native == other._native

    def __hash__(self) -> int:
        return hash(self._native)

    def __repr__(self) -> str:
        return f"<torch.b200.Queue device=blackwell:{self.device_index} id={self.queue_id}>"

    def __enter__(self):
        self._prev_device = current_device()
        pooled = _C._getQueueFromPool(self.device_index)
        self._prev = _C._getCurrentQueue(self.device_index)
        if self.device_index != self._prev_device:
            set_device(self.device_index)
        self._native = pooled
        _C._setCurrentQueue(pooled)
        return self

    def __exit__(self, *exc):
        _C._setCurrentQueue(self._prev)
        if self._prev_device != current_device():
            set_device(self._prev_device)
        return False


Stream = Queue


class Notifier:
    """A marker placed in a queue (a CUDA event); reference: torch_mlu/core/device/notifier.py:36-77."""

    def __init__(self, enable_timing: bool = True, blocking: bool = False, interprocess: bool = False):
        self._native = _C._Notifier(enable_timing)

    def place(self, queue: Optional[Queue] = None) -> None:
        if queue is None:
            self._native.place()
        else:
            self._native.place(queue._native)

    record = place

    def wait(self, queue: Optional[Queue] = None) -> None:
        q = queue._native if queue is not None else _C._getCurrentQueue(-1)
        self._native.wait(q)

    def query(self) -> bool:
        return self._native.query()

    def synchronize(self) -> None:
        self._native.synchronize()

    def elapsed_time(self, end: "Notifier") -> float:
        """Milliseconds between this notifier and ``end``."""
        return self._native.elapsed_time(end._native)

    def hardware_time(self, end: "Notifier") -> float:
        """Microseconds of device time between this notifier and ``end``."""
        return self._native.hardware_time(end._native)


Event = Notifier


def current_queue(device: _device_t = None) -> Queue:
    return Queue(_native=_C._getCurrentQueue(_get_device_index(device, optional=True)))


def default_queue(device: _device_t = None) -> Queue:
    return Queue(_native=_C._getDefaultQueue(_get_device_index(device, optional=True)))


def queue_from_pool(device: _device_t = None) -> Queue:
    return Queue(_native=_C._getQueueFromPool(_get_device_index(device, optional=True)))


current_stream = current_queue
default_stream = default_queue


def set_stream(queue: Queue) -> None:
    _C._setCurrentQueue(queue._native)


class StreamContext:
    def __init__(self, queue: Optional[Queue]):
        self.queue = queue
        self._prev = None
        self._prev_dev = None

    def __enter__(self):
        if self.queue is None:
            return
        self._prev_dev = current_device()
        self._prev = _C._getCurrentQueue(self.queue.device_index)
        if self.queue.device_index != self._prev_dev:
            set_device(self.queue.device_index)
        _C._setCurrentQueue(self.queue._native)

    def __exit__(self, *exc):
        if self.queue is None:
            return False
        _C._setCurrentQueue(self._prev)
        if self._prev_dev != current_device():
            set_device(self._prev_dev)
        return False


def stream(queue: Optional[Queue]) -> StreamContext:
    """Context manager making ``queue`` current (``torch.cuda.stream`` spelling)."""
    return StreamContext(queue)


# --------------------------------------------------------------------------- memory
def empty_cache() -> None:
    _C._empty_cache()


empty_cached_memory = empty_cache


def memory_allocated(device: _device_t = None) -> int:
    return _C._memory_allocated(_get_device_index(device, optional=True))


def max_memory_allocated(device: _device_t = None) -> int:
    return _C._max_memory_allocated(_get_device_index(device, optional=True))


def memory_reserved(device: _device_t = None) -> int:
    return _C._memory_reserved(_get_device_index(device, optional=True))


def max_memory_reserved(device: _device_t = None) -> int:
    return _C._max_memory_reserved(_get_device_index(device, optional=True))


def memory_cached(device: _device_t = None) -> int:
    return memory_reserved(device)


def max_memory_cached(device: _device_t = None) -> int:
    return max_memory_reserved(device)


def reset_peak_memory_stats(device: _device_t = None) -> None:
    _C._reset_peak_memory_stats(_get_device_index(device, optional=True))


reset_max_memory_allocated = reset_peak_memory_stats
reset_max_memory_cached = reset_peak_memory_stats


def memory_stats(device: _device_t = None) -> dict:
    return dict(_C._memory_stats(_get_device_index(device, optional=True)))


def memory_summary(device: _device_t = None) -> str:
    return _C._memory_summary(_get_device_index(device, optional=True))


def set_memory_strategy(native_memory_strategy: bool) -> None:
    """True: ask the driver for exactly the requested size; False: cache-friendly segment sizes."""
    _C._set_memory_strategy(bool(native_memory_strategy))


def set_per_process_memory_fraction(fraction: float, device: _device_t = None) -> None:
    """Cap the device memory this process's caching allocator may hold at ``fraction`` of the device's capacity
    (``torch.cuda.set_per_process_memory_fraction``).  A request that would pass the cap fails with an out-of-memory
    error after cached blocks were given back; 0 lifts the cap."""
    _C._set_memory_fraction(float(fraction), _get_device_index(device, optional=True))


def caching_allocator_alloc(size: int, device: _device_t = None, stream=None) -> int:
    """A raw block of ``size`` bytes from the caching allocator, bound to ``stream`` (default: the current queue);
    returns its address (``torch.cuda.caching_allocator_alloc``).  Free it with ``caching_allocator_delete``."""
    d = _get_device_index(device, optional=True)
    q = getattr(stream, "_native", stream)
    return _C._raw_alloc(int(size), d, q)


def caching_allocator_delete(mem_ptr: int) -> None:
    _C._raw_free(int(mem_ptr))


def can_device_access_peer(device: _device_t, peer_device: _device_t) -> bool:
    """Every pair of distinct B200s of one NVSwitch domain maps each other's memory."""
    a, b = _get_device_index(device, optional=True), _get_device_index(peer_device, optional=True)
    n = device_count()
    if not (0 <= a < n and 0 <= b < n):
        raise ValueError("invalid device ordinal")
    return a != b


def get_arch_list():
    """The architectures the device library was compiled for."""
    return ["sm_100a"]


def ipc_collect() -> None:
    """Kept for scripts written for ``torch.cuda``: peer mappings of this backend live as long as their process group."""
    return None


def utilization(device: _device_t = None) -> int:
    """Percent of the last sampling period during which kernels ran on the device (read through NVML)."""
    import pynvml

    pynvml.nvmlInit()
    try:
        handle = pynvml.nvmlDeviceGetHandleByIndex(_get_device_index(device, optional=True))
        return int(pynvml.nvmlDeviceGetUtilizationRates(handle).gpu)
    finally:
        pynvml.nvmlShutdown()


class _Nvtx:
    """``torch.cuda.nvtx``-shaped annotations; they land in this backend's kernel trace
    (``catch_b200.profiler.kernel_trace``) and in profiler output."""

    @staticmethod
    def range_push(msg: str) -> None:
        _C._trace_range_push(str(msg))

    @staticmethod
    def range_pop() -> None:
        _C._trace_range_pop()

    @staticmethod
    def mark(msg: str) -> None:
        _C._trace_mark(str(msg))

    @staticmethod
    @contextlib.contextmanager
    def range(msg: str, *args, **kwargs):
        _C._trace_range_push(str(msg).format(*args, **kwargs))
        try:
            yield
        finally:
            _C._trace_range_pop()


nvtx = _Nvtx()


class _Amp:
    """``torch.cuda.amp``-shaped entry points for scripts written for GPUs."""

    @staticmethod
    def autocast(enabled: bool = True, dtype: torch.dtype = torch.bfloat16, cache_enabled: bool = True):
        return torch.autocast("blackwell", enabled=enabled, dtype=dtype, cache_enabled=cache_enabled)

    @staticmethod
    def GradScaler(*args, **kwargs):  # noqa: N802 - the name scripts use
        return torch.amp.GradScaler("blackwell", *args, **kwargs)


amp = _Amp()


def make_graphed_callables(callables, sample_args, num_warmup_iters: int = 3, **_ignored):
    """``torch.cuda.make_graphed_callables`` shape: one callable with its sample arguments, or a tuple of callables
    with a tuple of argument tuples.  Inference only (see :func:`make_graphed_callable`)."""
    if isinstance(callables, (tuple, list)):
        return tuple(make_graphed_callable(c, a, num_warmup_iters) for c, a in zip(callables, sample_args))
    return make_graphed_callable(callables, sample_args, num_warmup_iters)


def is_tf32_supported() -> bool:
    return True


def _nvml_query(device, fn):
    import pynvml

    pynvml.nvmlInit()
    try:
        return fn(pynvml, pynvml.nvmlDeviceGetHandleByIndex(_get_device_index(device, optional=True)))
    finally:
        pynvml.nvmlShutdown()


def temperature(device: _device_t = None) -> int:
    """Degrees Celsius (read through NVML)."""
    return int(_nvml_query(device, lambda n, h: n.nvmlDeviceGetTemperature(h, n.NVML_TEMPERATURE_GPU)))


def power_draw(device: _device_t = None) -> int:
    """Milliwatts (read through NVML)."""
    return int(_nvml_query(device, lambda n, h: n.nvmlDeviceGetPowerUsage(h)))


def clock_rate(device: _device_t = None) -> int:
    """SM clock in MHz (read through NVML)."""
    return int(_nvml_query(device, lambda n, h: n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)))


def device_memory_used(device: _device_t = None) -> int:
    """Bytes in use on the device by all processes (read through NVML)."""
    return int(_nvml_query(device, lambda n, h: n.nvmlDeviceGetMemoryInfo(h).used))


OutOfMemoryError = torch.OutOfMemoryError


def set_memory_debug(enable: bool) -> None:
    """Switch the guard-word debug allocator on or off.  Tensors allocated while it is on carry guard regions (and an
    allocation record) until they are freed; tensors allocated while it is off are not checked."""
    _C._set_memory_debug(bool(enable))


def memory_debug(tensor: Optional[torch.Tensor] = None):
    """Verify the guard regions of one tensor's block (or of every live block).

    Returns ``(blocks_checked, corrupted, detail)``; raises if corruption was found.
    """
    checked, corrupted, detail = _C._memory_debug(tensor)
    if corrupted:
        raise RuntimeError(f"b200 memory debug: {corrupted} block(s) with out-of-bounds writes:\n{detail}")
    return checked, corrupted, detail


def memory_debug_origin(tensor: torch.Tensor) -> str:
    """Where the block behind ``tensor`` was allocated (Python frames, then native frames); ``""`` unless the
    debug allocator was on when it was allocated.  The same text is part of every corruption report."""
    return _C._memory_debug_origin(tensor)


class Graph:
    """A sequence of device launches captured once and replayed with a single submission.

    ::

        g = torch.b200.Graph()
        static_x = torch.empty_like(x)            # inputs live outside the graph
        with torch.b200.graph(g):                 # runs the body once on a side queue while recording it
            static_y = model(static_x)
        static_x.copy_(x); g.replay()             # static_y now holds model(x)

    Memory allocated inside the ``with`` block belongs to the graph (a private pool of the caching allocator);
    tensors created there and still alive afterwards are overwritten by every replay.  The body must not wait for
    the device (``.item()``, ``.cpu()``, ``synchronize()``) and must make the same launches for the same shapes.
    """

    def __init__(self):
        self._native = _C._Graph()

    def capture_begin(self) -> None:
        self._native.capture_begin()

    def capture_end(self) -> bool:
        return self._native.capture_end()

    def replay(self) -> None:
        self._native.replay()

    def reset(self) -> None:
        self._native.reset()

    @property
    def valid(self) -> bool:
        return self._native.valid

    @property
    def num_nodes(self) -> int:
        return self._native.num_nodes


class graph:
    """Context manager that captures its body into ``g`` on a queue from the pool (the default queue cannot be
    captured).  Work already submitted to the previous current queue is waited for on the device first; after the
    block the previous queue waits for the side queue.  Raises if the body could not be captured."""

    def __init__(self, g: Graph, queue: Optional["Queue"] = None):
        self.g = g
        self._side = queue._native if queue is not None else _C._getQueueFromPool(-1)
        self._prev = None

    def __enter__(self):
        import gc

        gc.collect()  # tensors that die during capture would return their blocks to the wrong place in time
        self._prev = _C._getCurrentQueue(-1)
        n = _C._Notifier(False)
        n.place(self._prev)
        n.wait(self._side)
        _C._setCurrentQueue(self._side)
        try:
            self.g.capture_begin()
        except Exception:
            _C._setCurrentQueue(self._prev)
            raise
        global _capture_depth
        _capture_depth += 1
        return self.g

    def __exit__(self, exc_type, exc, tb):
        global _capture_depth
        _capture_depth -= 1
        try:
            if exc_type is not None:
                self.g._native.capture_abort()
                return False
            ok = self.g.capture_end()
        finally:
            _C._setCurrentQueue(self._prev)
        n = _C._Notifier(False)
        n.place(self._side)
        n.wait(self._prev)
        if not ok:
            raise RuntimeError("b200 graph capture failed: the captured region waited for the device or used a call "
                               "that cannot be recorded")
        return False


CUDAGraph = Graph  # the name scripts converted from torch.cuda use
_capture_depth = 0


def is_current_stream_capturing() -> bool:
    """True inside a ``with torch.b200.graph(g):`` block of this thread's interpreter."""
    return _capture_depth > 0


def graph_pool_handle() -> int:
    """An id of a private allocator pool (``torch.cuda.graph_pool_handle``); every :class:`Graph` of this backend
    owns its pool, so the handle is only kept for scripts that pass one around."""
    return int(_C._new_private_pool())


def graphs_supported() -> bool:
    """False under host simulation (work runs when it is submitted: there is nothing to record)."""
    return _C._graphs_supported()


def make_graphed_callable(fn, sample_args, warmup: int = 2):
    """Inference-only analogue of ``torch.cuda.make_graphed_callables``: runs ``fn(*sample_args)`` ``warmup`` times,
    captures one more run into a :class:`Graph` and returns a callable that copies its tensor arguments into the
    captured inputs, replays, and returns the captured outputs (overwritten by the next call: clone what has to
    live longer).  Arguments must keep the sample's shapes and dtypes.  Without graph support (host simulation)
    ``fn`` itself is returned."""
    if not graphs_supported():
        return fn
    sample_args = tuple(sample_args)
    with torch.no_grad():
        for _ in range(max(warmup, 1)):
            fn(*sample_args)
        static_in = tuple(a.clone() if isinstance(a, torch.Tensor) else a for a in sample_args)
        g = Graph()
        with graph(g):
            static_out = fn(*static_in)

    def run(*args):
        if len(args) != len(static_in):
            raise TypeError(f"graphed callable takes {len(static_in)} arguments")
        for dst, src in zip(static_in, args):
            if isinstance(dst, torch.Tensor):
                if src.shape != dst.shape or src.dtype != dst.dtype:
                    raise ValueError(f"graphed callable captured {tuple(dst.shape)} {dst.dtype}, got {tuple(src.shape)} {src.dtype}")
                if src.data_ptr() != dst.data_ptr():
                    dst.copy_(src, non_blocking=True)
        g.replay()
        return static_out

    run.graph = g
    run.static_inputs = static_in
    return run


def pin_memory(tensor: torch.Tensor) -> torch.Tensor:
    return _C._pin_memory(tensor)


def is_pinned(tensor: torch.Tensor) -> bool:
    return _C._is_pinned(tensor)


def record_queue(tensor: torch.Tensor, queue: Queue) -> None:
    """Tell the allocator that ``tensor`` is in use on ``queue`` (deferred reuse)."""
    _C._record_queue(tensor, queue._native)


def mem_get_info(device: _device_t = None):
    p = get_device_properties(device)
    return p.total_memory - memory_reserved(device), p.total_memory


# ------------------------------------------------------------------------------ RNG
def manual_seed(seed: int) -> None:
    _C._manual_seed(current_device(), int(seed) & 0xFFFFFFFFFFFFFFFF)


def manual_seed_all(seed: int) -> None:
    _C._manual_seed_all(int(seed) & 0xFFFFFFFFFFFFFFFF)


def seed() -> None:
    manual_seed(torch.seed())


def seed_all() -> None:
    manual_seed_all(torch.seed())


def initial_seed() -> int:
    return _C._default_generator(current_device()).initial_seed()


def get_rng_state(device: _device_t = None) -> torch.Tensor:
    return _C._default_generator(_get_device_index(device, optional=True)).get_state()


def set_rng_state(new_state: torch.Tensor, device: _device_t = None) -> None:
    _C._default_generator(_get_device_index(device, optional=True)).set_state(new_state)


def get_rng_state_all():
    return [get_rng_state(i) for i in range(device_count())]


def set_rng_state_all(states) -> None:
    for i, s in enumerate(states):
        set_rng_state(s, i)


def _is_in_bad_fork() -> bool:
    return False


# ---------------------------------------------------------------------- autocast / amp
def get_amp_supported_dtype():
    return [torch.bfloat16, torch.float16]


def is_bf16_supported(including_emulation: bool = True) -> bool:
    return True


# ----------------------------------------------------------------------- running mode
_floating_point_calculation = True


def enable_floating_point_calculation(enable: bool) -> None:
    """Kept for script compatibility; B200 always computes in floating point."""
    global _floating_point_calculation
    _floating_point_calculation = bool(enable)


def is_using_floating_device() -> bool:
    return True


def get_running_mode() -> str:
    return "eager"


def _jit_override_can_fuse_on_b200(enable: bool) -> None:
    from . import jit as _jit

    _jit.set_fusion_enabled(enable)


def _jit_can_fuse_on_b200() -> bool:
    from . import jit as _jit

    return _jit.fusion_enabled()


# ------------------------------------------------------------------ tensors and modules
def to(optimizer: torch.optim.Optimizer, device: _device_t) -> torch.optim.Optimizer:
    """Move every tensor of an optimizer's state to ``device`` (reference: mlu_model.py:503-508)."""
    dev = torch.device(device) if not isinstance(device, torch.device) else device
    for state in optimizer.state.values():
        for k, v in state.items():
            if isinstance(v, torch.Tensor):
                state[k] = v.to(dev)
    return optimizer


def _legacy_ctor(dtype: torch.dtype):
    def make(*args, **kwargs) -> torch.Tensor:
        dev = kwargs.pop("device", None) or b200_device()
        if len(args) == 1 and isinstance(args[0], (list, tuple, torch.Tensor)) or (
            len(args) == 1 and hasattr(args[0], "__array__")
        ):
            return torch.as_tensor(args[0], dtype=dtype).to(dev)
        if len(args) == 0:
            return torch.empty(0, dtype=dtype, device=dev)
        return torch.empty(*args, dtype=dtype, device=dev)

    return make


FloatTensor = _legacy_ctor(torch.float32)
HalfTensor = _legacy_ctor(torch.float16)
BFloat16Tensor = _legacy_ctor(torch.bfloat16)
DoubleTensor = _legacy_ctor(torch.float64)
ByteTensor = _legacy_ctor(torch.uint8)
CharTensor = _legacy_ctor(torch.int8)
ShortTensor = _legacy_ctor(torch.int16)
IntTensor = _legacy_ctor(torch.int32)
LongTensor = _legacy_ctor(torch.int64)
BoolTensor = _legacy_ctor(torch.bool)


_orig_torch_load = torch.load


def _map_to_b200(obj, dev):
    if isinstance(obj, torch.Tensor):
        return obj.to(dev)
    if isinstance(obj, dict):
        return type(obj)((k, _map_to_b200(v, dev)) for k, v in obj.items())
    if isinstance(obj, (list, tuple)):
        seq = [_map_to_b200(v, dev) for v in obj]
        return type(obj)(seq) if not hasattr(obj, "_fields") else type(obj)(*seq)
    if isinstance(obj, torch.nn.Module):
        return obj.to(dev)
    return obj


def load(f, map_location=None, *args, **kwargs):
    """``torch.load`` that understands ``map_location='blackwell[:i]'``.

    Objects are materialised on the CPU and then moved, exactly like the
    reference's wrapper (torch_mlu/core/mlu_model.py:351-382).
    """
    target = None
    if isinstance(map_location, (str, torch.device)):
        d = torch.device(map_location)
        if d.type == DEVICE_TYPE:
            target = d
    if target is None:
        return _orig_torch_load(f, map_location, *args, **kwargs)
    obj = _orig_torch_load(f, "cpu", *args, **kwargs)
    return _map_to_b200(obj, target)


torch.load = load


# ----------------------------------------------------------------------------- logging
def set_log_level(level: int) -> None:
    _C._set_min_log_level(int(level))


def get_log_level() -> int:
    return _C._get_min_log_level()


def show_config() -> str:
    """A text block for bug reports: versions, backend, devices, run-time switches and every ``CATCH_B200_*``
    environment variable that is set (the counterpart of ``torch.__config__.show()``)."""
    import os

    lines = [get_version(), f"torch {torch.__version__}", f"backend: {backend_name()}", f"devices: {device_count()}"]
    for d in range(device_count()):
        p = get_device_properties(d)
        lines.append(f"  blackwell:{d}: {p.name}, sm_{p.major}{p.minor}, {p.total_memory // (1 << 20)} MiB, "
                     f"{p.multi_processor_count} SMs")
    lines.append("device code: sm_100a")
    flags = ("async_disable", "op_trycatch", "test_cpu_dispatch", "fallback_to_cpu", "blocking_wait")
    lines.append("switches: " + ", ".join(f"{f}={int(get_flag(f))}" for f in flags) +
                 f", memory_debug={int(_C._memory_debug_enabled()) if hasattr(_C, '_memory_debug_enabled') else '?'}"
                 f", native_memory_strategy={int(_C._get_memory_strategy())}"
                 f", fusion={int(_C._jit_can_fuse_on_b200())}")
    env = sorted((k, v) for k, v in os.environ.items() if k.startswith("CATCH_B200_") or k == "USE_IO_QUEUE")
    lines.append("environment: " + (", ".join(f"{k}={v}" for k, v in env) if env else "(no CATCH_B200_* variable set)"))
    return "\n".join(lines)


def set_flag(name: str, value: bool) -> None:
    """Flip a runtime switch: async_disable, op_trycatch, test_cpu_dispatch, fallback_to_cpu, blocking_wait."""
    _C._set_flag(name, bool(value))


def get_flag(name: str) -> bool:
    return _C._get_flag(name)


__all__ = [n for n in dir() if not n.startswith("_") and n not in (
    "annotations", "contextlib", "warnings", "Any", "Optional", "Union", "torch")]
