"""Runtime API on the host-simulated device: devices, queues, notifiers, caching
allocator statistics, debug allocator, pinned memory, tensor movement, legacy
constructors, torch.load with a device map_location, RNG reproducibility.
Mirrors the reference's runtime tests (test/test_device.py, test_queue.py,
test_notifier.py, test_caching_allocator.py, test_mlu.py)."""
import io
import threading

import pytest
import torch

import catch_b200  # noqa: F401

DEV = "blackwell"
bw = torch.b200


def test_device_management():
    assert bw.is_available() and bw.device_count() >= 2
    assert torch.blackwell is torch.b200
    prev = bw.current_device()
    bw.set_device(1)
    assert bw.current_device() == 1
    with bw.device(0):
        assert bw.current_device() == 0
        assert torch.empty(1, device=DEV).device.index == 0
    assert bw.current_device() == 1
    x = torch.zeros(1, device="blackwell:0")
    with bw.device_of(x):
        assert bw.current_device() == 0
    bw.set_device(prev)
    p = bw.get_device_properties(0)
    assert p.major == 10 and p.total_memory > 0 and isinstance(p.name, str)
    assert bw.get_device_capability() == (10, 0)
    assert bw.get_device_name(0) == p.name
    with pytest.raises(Exception):
        bw.set_device(99)
    bw.synchronize()
    assert "catch_b200" in bw.get_version()


def test_tensor_to_and_device_strings():
    x = torch.arange(12.0).reshape(3, 4)
    for spec in (DEV, "blackwell:1", torch.device(DEV, 0)):
        y = x.to(spec)
        assert y.device.type == DEV and torch.equal(y.cpu(), x)
    assert x.blackwell().is_blackwell
    m = torch.nn.Linear(4, 2).blackwell()
    assert next(m.parameters()).device.type == DEV
    y = x.to(DEV)
    assert torch.equal(y.t().contiguous().cpu(), x.t())
    assert torch.equal(y[1:, ::2].cpu(), x[1:, ::2])
    assert y.double().dtype == torch.float64 and torch.equal(y.long().cpu(), x.long())
    z = torch.empty_strided((2, 3), (1, 2), device=DEV)
    assert z.stride() == (1, 2)
    assert y.sum().item() == x.sum().item()
    y2 = y.clone()
    y2.resize_(5, 4)
    assert y2.shape == (5, 4)
    assert bw.FloatTensor(2, 3).shape == (2, 3) and bw.LongTensor([1, 2]).dtype == torch.int64
    with pytest.raises(Exception):
        _ = y + torch.ones(3, 4, device="blackwell:1")  # tensors on different devices


def test_queues():
    d = bw.current_device()
    dq = bw.default_queue()
    assert bw.current_queue() == dq and dq.device_index == d
    with bw.Queue() as q:
        assert bw.current_queue() == q and q != dq
        assert q.query()
        q.synchronize()
    assert bw.current_queue() == dq
    seen = {bw.queue_from_pool().queue_id for _ in range(40)}
    assert len(seen) == 32  # the pool wraps around after 32 queues
    other = {}

    def worker():
        other["q"] = bw.current_queue()

    with bw.Queue():
        t = threading.Thread(target=worker)
        t.start(); t.join()
    assert other["q"] == dq  # the current queue is thread-local
    with bw.Queue(1) as q1:
        assert bw.current_device() == 1 and q1.device_index == 1
    assert bw.current_device() == d
    s = torch.Stream(device=DEV)  # generic torch.Stream goes through the device guard
    with s:
        assert torch.empty(1, device=DEV).device.type == DEV


def test_notifiers():
    a, b = bw.Notifier(), bw.Notifier()
    assert a.query()
    a.place()
    x = torch.ones(1000, device=DEV)
    for _ in range(10):
        x = x * 2
    b.place(bw.current_queue())
    b.synchronize()
    assert b.query()
    assert a.elapsed_time(b) >= 0.0
    assert a.hardware_time(b) == pytest.approx(a.elapsed_time(b) * 1000, rel=0.5, abs=1e3)
    b.wait(bw.current_queue())
    with pytest.raises(Exception):
        bw.Notifier().elapsed_time(b)
    e1, e2 = torch.Event(device=DEV, enable_timing=True), torch.Event(device=DEV, enable_timing=True)
    e1.record(); e2.record(); e2.synchronize()
    assert e1.elapsed_time(e2) >= 0.0


def test_caching_allocator_stats():
    bw.empty_cache()
    d = bw.current_device()
    base_a, base_r = bw.memory_allocated(d), bw.memory_reserved(d)
    x = torch.empty(1000, device=DEV)  # 4000 B -> rounded to 4096, from a 2 MiB segment
    assert bw.memory_allocated(d) == base_a + 4096
    # a new 2 MiB segment, unless a segment kept alive by tensors of earlier tests still had room
    assert bw.memory_reserved(d) >= max(base_r, 2 << 20)
    small_growth = bw.memory_reserved(d) - base_r
    assert small_growth in (0, 2 << 20)
    y = torch.empty(3 << 20, dtype=torch.uint8, device=DEV)  # large pool: a 20 MiB segment
    # (or room in a large segment that tensors of earlier tests still keep alive)
    large_growth = bw.memory_reserved(d) - base_r - small_growth
    assert large_growth in (0, 20 << 20)
    peak = bw.max_memory_allocated(d)
    assert peak >= bw.memory_allocated(d)
    del x, y
    assert bw.memory_allocated(d) == base_a
    assert bw.memory_reserved(d) == base_r + small_growth + large_growth  # cached, not returned
    grown = bw.memory_reserved(d)
    z = torch.empty(1000, device=DEV)
    assert bw.memory_reserved(d) == grown  # reuse, no growth
    del z
    bw.empty_cache()
    assert bw.memory_reserved(d) == base_r
    assert bw.max_memory_allocated(d) == peak
    bw.reset_peak_memory_stats(d)
    assert bw.max_memory_allocated(d) == bw.memory_allocated(d)
    assert bw.memory_cached(d) == bw.memory_reserved(d)
    st = bw.memory_stats(d)
    assert st["num_alloc"] >= 3 and "allocated_bytes.current" in st
    assert "allocated" in bw.memory_summary(d)


def test_record_queue_defers_reuse():
    with bw.Queue() as side:
        pass
    x = torch.empty(1 << 16, device=DEV)
    ptr = x.data_ptr()
    bw.record_queue(x, side)
    del x
    y = torch.empty(1 << 16, device=DEV)  # after the side queue's notifier has fired the block may come back
    assert y.data_ptr() is not None and ptr is not None


def test_native_memory_strategy_and_oom():
    bw.empty_cache()
    d = bw.current_device()
    bw.set_memory_strategy(True)
    try:
        r0 = bw.memory_reserved(d)
        t = torch.empty(3 << 20, dtype=torch.uint8, device=DEV)
        assert bw.memory_reserved(d) - r0 == 3 << 20  # exactly what was asked for
        del t
    finally:
        bw.set_memory_strategy(False)
        bw.empty_cache()
    catch_b200._C._hostsim_set_memory_limit(64 << 20)
    try:
        keep = torch.empty(40 << 20, dtype=torch.uint8, device=DEV)
        del keep  # cached: the next big request must free the cache and retry
        big = torch.empty(50 << 20, dtype=torch.uint8, device=DEV)
        assert bw.memory_stats(d)["num_alloc_retries"] >= 1
        with pytest.raises(torch.OutOfMemoryError, match="out of memory"):
            torch.empty(100 << 20, dtype=torch.uint8, device=DEV)
        del big
    finally:
        catch_b200._C._hostsim_set_memory_limit(8 << 30)
        bw.empty_cache()


def test_debug_allocator_detects_overrun():
    import ctypes

    keep = torch.ones(10, device=DEV)  # allocated outside debug mode: stays valid, is not checked
    bw.set_memory_debug(True)
    try:
        x = torch.zeros(100, device=DEV)
        checked, corrupted, _ = bw.memory_debug(x)
        assert checked == 1 and corrupted == 0
        # host simulation: device memory is host memory, so an overrun can be staged from here
        ctypes.memset(x.data_ptr() + 512, 0, 8)  # first bytes after the rounded block
        with pytest.raises(RuntimeError, match="out-of-bounds") as err:
            bw.memory_debug(x)
        # the report says where the damaged block came from: this test function, then native frames
        msg = str(err.value)
        del err  # its traceback keeps the frame that holds the tensor alive
        assert "allocated at:" in msg and "test_debug_allocator_detects_overrun" in msg
        origin = bw.memory_debug_origin(x)
        assert "test_runtime.py" in origin and "catch_b200" in origin
        ctypes.memset(x.data_ptr() + 512, 0xA5, 8)
        bw.memory_debug()
        assert bw.memory_debug(keep)[0] == 0 and keep.sum().item() == 10.0
        del x
    finally:
        bw.empty_cache()
        bw.set_memory_debug(False)


def test_private_pools_keep_graph_memory_apart():
    """Blocks allocated while a thread has a private pool set (graph capture) are reused only inside that pool until
    the pool is retired; then they serve everybody again."""
    C = catch_b200._C
    bw.empty_cache()
    assert not bw.graphs_supported()  # host simulation: nothing to capture
    f = lambda x: x + 1
    assert bw.make_graphed_callable(f, (torch.zeros(2, device=DEV),)) is f
    pool = C._new_private_pool()
    assert C._set_thread_private_pool(pool) == 0
    try:
        a = torch.empty(3 << 20, dtype=torch.uint8, device=DEV)
        pa = a.data_ptr()
        del a
        b = torch.empty(3 << 20, dtype=torch.uint8, device=DEV)  # reuse inside the pool
        assert b.data_ptr() == pa
        del b
    finally:
        assert C._set_thread_private_pool(0) == pool
    reserved = bw.memory_reserved()
    c = torch.empty(3 << 20, dtype=torch.uint8, device=DEV)  # the shared cache may not hand out the pool's block
    assert c.data_ptr() != pa
    del c
    bw.empty_cache()
    assert bw.memory_reserved() >= 20 << 20 and bw.memory_reserved() <= reserved + (20 << 20)  # pool segment survives
    C._retire_private_pool(pool)
    d = torch.empty(3 << 20, dtype=torch.uint8, device=DEV)
    assert d.data_ptr() == pa  # back in the shared cache
    del d
    bw.empty_cache()
    assert bw.memory_reserved() == 0 or bw.memory_reserved() < 20 << 20


def test_pinned_memory():
    x = torch.randn(1000)
    assert not bw.is_pinned(x)
    p = bw.pin_memory(x)
    assert bw.is_pinned(p) and torch.equal(p, x)
    y = p.to(DEV, non_blocking=True)
    bw.synchronize()
    assert torch.equal(y.cpu(), x)
    del p
    assert catch_b200._C._pinned_cached_bytes() >= 4000
    catch_b200._C._pinned_empty_cache()
    assert catch_b200._C._pinned_cached_bytes() == 0


def test_save_load_and_map_location():
    m = torch.nn.Linear(3, 2).to(DEV)
    buf = io.BytesIO()
    torch.save(m.state_dict(), buf)
    buf.seek(0)
    sd = torch.load(buf, map_location="cpu")
    assert all(v.device.type == "cpu" for v in sd.values())
    buf.seek(0)
    sd = torch.load(buf, map_location="blackwell:1")
    assert all(v.device == torch.device(DEV, 1) for v in sd.values())
    m2 = torch.nn.Linear(3, 2)
    m2.load_state_dict({k: v.cpu() for k, v in sd.items()})
    assert torch.equal(m2.weight, m.weight.cpu())
    opt = torch.optim.SGD(m2.parameters(), lr=0.1, momentum=0.9)
    m2(torch.randn(2, 3)).sum().backward(); opt.step()
    bw.to(opt, DEV)
    assert all(v.device.type == DEV for s in opt.state.values() for v in s.values() if isinstance(v, torch.Tensor))


def test_rng_reproducible():
    bw.manual_seed(7)
    a = torch.randn(100, device=DEV)
    bw.manual_seed(7)
    b = torch.randn(100, device=DEV)
    assert torch.equal(a.cpu(), b.cpu())
    st = bw.get_rng_state()
    c = torch.rand(10, device=DEV)
    bw.set_rng_state(st)
    assert torch.equal(torch.rand(10, device=DEV).cpu(), c.cpu())
    torch.manual_seed(3)  # seeds every device generator too
    d1 = torch.randn(5, device=DEV)
    torch.manual_seed(3)
    assert torch.equal(torch.randn(5, device=DEV).cpu(), d1.cpu())


def test_flags_and_logging(capfd):
    assert bw.get_flag("fallback_to_cpu") is True
    bw.set_log_level(-1)
    try:
        _ = torch.ones(2, device=DEV) + 1
        err = capfd.readouterr().err
        assert "[DEBUG]" in err and "runs on the CPU path" in err
    finally:
        bw.set_log_level(1)


def test_cuda_style_conveniences(monkeypatch):
    """Entry points that scripts converted from torch.cuda call: per-process memory cap, raw allocator blocks, nvtx and
    amp namespaces, peer access, architecture list."""
    import pytest

    bw = torch.b200
    dev = bw.current_device()
    bw.empty_cache()
    base = bw.memory_reserved()
    total = bw.get_device_properties(dev).total_memory
    # a cap a little above what is reserved now: a small tensor fits, a large one does not
    frac = (base + (8 << 20)) / total
    bw.set_per_process_memory_fraction(frac)
    try:
        ok = torch.empty(1 << 20, dtype=torch.uint8, device="blackwell")
        with pytest.raises(torch.OutOfMemoryError, match="per-process limit"):
            torch.empty(64 << 20, dtype=torch.uint8, device="blackwell")
        assert bw.memory_stats()["num_ooms"] >= 1
        del ok
    finally:
        bw.set_per_process_memory_fraction(0.0)
    big = torch.empty(64 << 20, dtype=torch.uint8, device="blackwell")     # the cap is lifted again
    del big
    bw.empty_cache()
    with pytest.raises(RuntimeError, match="fraction"):
        bw.set_per_process_memory_fraction(1.5)
    before = bw.memory_allocated()
    ptr = bw.caching_allocator_alloc(4096)
    assert ptr != 0 and bw.memory_allocated() >= before + 4096
    ptr2 = bw.caching_allocator_alloc(4096, stream=bw.current_queue())
    assert ptr2 not in (0, ptr)
    bw.caching_allocator_delete(ptr); bw.caching_allocator_delete(ptr2)
    assert bw.memory_allocated() == before
    with bw.nvtx.range("step {}", 3):
        bw.nvtx.mark("inside")
    bw.nvtx.range_push("a"); bw.nvtx.range_pop()
    with bw.amp.autocast(dtype=torch.bfloat16):
        assert torch.is_autocast_enabled("blackwell") and torch.get_autocast_dtype("blackwell") == torch.bfloat16
    assert type(bw.amp.GradScaler(enabled=False)).__name__ == "GradScaler"
    assert bw.get_arch_list() == ["sm_100a"]
    if bw.device_count() > 1:
        assert bw.can_device_access_peer(0, 1) and not bw.can_device_access_peer(0, 0)
    with pytest.raises(ValueError):
        bw.can_device_access_peer(0, 99)
    assert bw.ipc_collect() is None
    cfg = bw.show_config()
    assert "backend: hostsim" in cfg and "blackwell:0" in cfg and "op_trycatch=1" in cfg and "sm_100a" in cfg
    s = bw.Stream(priority=-1)
    assert bw.Stream(device=dev).device_index == dev and s.query() in (True, False)
    assert bw.CUDAGraph is bw.Graph and not bw.is_current_stream_capturing() and bw.graph_pool_handle() > 0
    assert bw.is_tf32_supported() and bw.OutOfMemoryError is torch.OutOfMemoryError
    double = bw.make_graphed_callables(lambda t: t * 2, (torch.ones(2, device="blackwell"),))
    assert torch.equal(double(torch.ones(2, device="blackwell")).cpu(), torch.full((2,), 2.0))
