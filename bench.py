"""Headline benchmark: ResNet-50 training throughput (images/sec) on N B200s.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

Config (the reference's DDP benchmark harness model, test/cnnl/test_ddp_benchmark.py:132-172,
at the B200 batch size): torchvision ResNet-50, random-init weights, bf16 autocast,
per-GPU batch 256 of 3x224x224 N(0,1) images with uniform labels from a per-rank
seed, SGD momentum 0.9 / lr 0.1 / wd 1e-4, 25 MB gradient buckets.

Arms (``--impl``):
  ours       this repository on the ``blackwell`` device: fused peer-memory all-reduce + optimizer
             kernel per bucket, everything through the public API.  Unless ``--no-stock`` is given
             the stock arm runs first in the same invocation and its numbers are reported inside the
             line (``stock``), so the ratio is taken on one box, back to back.
  stock      stock PyTorch on ``torch.cuda``: cuDNN / cuBLAS kernels, ``torch.optim.SGD``,
             ``DistributedDataParallel`` over NCCL -- the same-hardware comparison point, because the
             reference itself cannot run without Cambricon hardware.
  reference  prints why the reference cannot run here.

Two timed regions per arm, both K steps after W warm-up steps, bracketed by a barrier and a device
synchronize, timed with device events, max over ranks:
  * ``value``   : inputs already resident on the device;
  * ``e2e``     : each step copies its batch from pinned host memory and reads the loss back to the host.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

# Stock PyTorch (CUDA + cuDNN + NCCL DDP) on this pool's B200s, images/sec at 1 / 2 / 4 / 8 GPUs, measured
# with ``bench.py --impl stock``.  The reference publishes no throughput number, so
# ``vs_baseline`` is taken against these; a stock run made in the same invocation is reported next to it.
STOCK_IMAGES_PER_SEC = {1: 4826.0, 2: 9358.5, 4: 18660.2, 8: 37211.9}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "stock", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="per-GPU batch size")
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--grad-dtype", default="fp32", choices=["fp32", "bf16"],
                    help="dtype in which gradients cross NVLink (the reduction is fp32 either way)")
    ap.add_argument("--no-stock", action="store_true", help="ours: do not run the stock arm first")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def summary(self, t0: float = 0.0, t1: float = float("inf")) -> dict:
        """Summarise the samples taken between host times t0 and t1 (a timed region)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm, mx, reasons = [], [], set()
        for ts, ln in list(self.lines):
            if ts < t0 or ts > t1:
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()  # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass


def host_batch(B, rank, pin):
    import torch

    g = torch.Generator().manual_seed(1234 + rank)
    x = pin(torch.randn(B, 3, 224, 224, generator=g))
    y = pin(torch.randint(0, 1000, (B,), generator=g))
    return x, y


def checksum_words(tensors):
    """SHA-1 of the parameters' bytes as five int64 words (compared across ranks after the run)."""
    import torch

    h = hashlib.sha1()
    for t in tensors:
        h.update(t.detach().to("cpu").reshape(-1).contiguous().view(torch.uint8).numpy().tobytes())
    d = h.digest()
    return [int.from_bytes(d[i:i + 4], "little") for i in range(0, 20, 4)]


# ---------------------------------------------------------------------------------------- stock arm
def run_stock(args, rank, local_rank, world, store, sampler):
    """torchvision ResNet-50 on torch.cuda: channels_last, bf16 autocast, cuDNN benchmark mode, fused
    torch.optim.SGD, DistributedDataParallel over NCCL with 25 MB buckets, same batch / steps / warm-up and
    the same two timed regions as the main arm."""
    import torch
    import torch.distributed as dist
    import torchvision

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    torch.backends.cudnn.benchmark = True
    pg = None
    if world > 1:
        dist.init_process_group("nccl", store=dist.PrefixStore("stock", store), rank=rank, world_size=world,
                                device_id=dev)
        pg = dist.group.WORLD
    torch.manual_seed(0)
    model = getattr(torchvision.models, args.model)(weights=None).to(dev).to(memory_format=torch.channels_last)
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], bucket_cap_mb=25,
                                                          gradient_as_bucket_view=True)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4, fused=True)
    criterion = torch.nn.CrossEntropyLoss()
    B = args.batch
    host_x, host_y = host_batch(B, rank, lambda t: t.pin_memory())
    dev_x = host_x.to(dev, non_blocking=True).contiguous(memory_format=torch.channels_last)
    dev_y = host_y.to(dev, non_blocking=True)

    def step(x, y):
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
            loss = criterion(model(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss

    io = torch.cuda.Stream(dev)

    def e2e_steps(n):
        # two batches in flight on a copy stream; the compute stream waits on each copy's event
        def fetch():
            with torch.cuda.stream(io):
                x = host_x.to(dev, non_blocking=True).to(memory_format=torch.channels_last)
                y = host_y.to(dev, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(io)
            return x, y, ev
        q = [fetch() for _ in range(min(2, n))]
        issued = len(q)
        last = None
        # every step's loss is read back, one step late, through pinned memory on a side stream (the host stays one
        # step ahead of the device); the last one is read before the timed region ends
        side = torch.cuda.Stream(dev)
        slots = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(2)]
        pending = None
        for i in range(n):
            x, y, ev = q.pop(0)
            if issued < n:
                q.append(fetch()); issued += 1
            cur = torch.cuda.current_stream(dev)
            cur.wait_event(ev)
            x.record_stream(cur); y.record_stream(cur)
            loss = step(x, y)
            ready = torch.cuda.Event(); ready.record(cur)
            with torch.cuda.stream(side):
                side.wait_event(ready)
                loss.record_stream(side)
                slots[i % 2].copy_(loss.detach().float(), non_blocking=True)
                done = torch.cuda.Event(); done.record(side)
            if pending is not None:
                pending[0].synchronize(); last = float(pending[1])
            pending = (done, slots[i % 2])
        if pending is not None:
            pending[0].synchronize(); last = float(pending[1])
        return last

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps, whole_loop=False):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = fn(steps) if whole_loop else [fn() for _ in range(steps)][-1]
        end.record()
        end.synchronize()
        barrier()
        ms = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms, out

    for _ in range(max(args.warmup, 3)):
        step(dev_x, dev_y)
    t0 = time.time()
    ms, loss = timed(lambda: step(dev_x, dev_y), args.steps)
    t1 = time.time()
    e2e_steps(2)
    ms_e2e, _ = timed(e2e_steps, args.steps, whole_loop=True)
    identical = None
    if world > 1:
        words = torch.tensor(checksum_words(model.parameters()), dtype=torch.int64, device=dev)
        allw = [torch.empty_like(words) for _ in range(world)]
        dist.all_gather(allw, words)
        identical = all(bool((w == allw[0]).all()) for w in allw)
    res = {"value": round(world * B * args.steps / (ms / 1e3), 1), "ms_per_step": round(ms / args.steps, 3),
           "e2e_value": round(world * B * args.steps / (ms_e2e / 1e3), 1), "e2e_ms_per_step": round(ms_e2e / args.steps, 3),
           "final_loss": float(loss.detach()), "params_identical_across_ranks": identical,
           "clocks": sampler.summary(t0, t1) if sampler is not None else {},
           "stack": f"torch {torch.__version__}, cuDNN {torch.backends.cudnn.version()}, NCCL "
                    f"{'.'.join(map(str, torch.cuda.nccl.version()))}, SGD(fused=True), channels_last, cudnn.benchmark"}
    del model, opt, dev_x, dev_y
    if world > 1:
        dist.destroy_process_group()
    torch.cuda.synchronize(dev)
    torch.cuda.empty_cache()
    return res


# ----------------------------------------------------------------------------------------- our arm
def run_ours(args, rank, local_rank, world, store, sampler):
    import torch
    import torch.distributed as dist
    import torchvision

    import catch_b200  # noqa: F401
    from catch_b200.fusion import fuse_bn_act
    from catch_b200.parallel import FusedDataParallel
    from catch_b200.utils import DelayedScalar, PrefetchLoader

    # CATCH_B200_BENCH_DRY_RUN=1: walk the whole script on the host-simulated device (tests of the script itself;
    # the numbers it prints then mean nothing)
    assert torch.b200.backend_name() == "cuda" or os.environ.get("CATCH_B200_BENCH_DRY_RUN") == "1", \
        "bench.py needs a GPU (the host-simulated device is for tests)"
    torch.b200.set_device(local_rank)
    dev = torch.device("blackwell", local_rank)
    if world > 1:
        dist.init_process_group("bwccl", store=dist.PrefixStore("ours", store), rank=rank, world_size=world)

    torch.manual_seed(0)
    model = getattr(torchvision.models, args.model)(weights=None)
    model = fuse_bn_act(model)  # same parameters / state dict; BN(+add)+ReLU chains run as fused kernels
    model = model.to(dev).to(memory_format=torch.channels_last)
    grad_dtype = torch.bfloat16 if args.grad_dtype == "bf16" else torch.float32
    fdp = FusedDataParallel(model, "sgd", lr=0.1, momentum=0.9, weight_decay=1e-4, bucket_mb=25.0, grad_dtype=grad_dtype)
    criterion = torch.nn.CrossEntropyLoss()

    B = args.batch
    host_x, host_y = host_batch(B, rank, torch.b200.pin_memory)
    dev_x = host_x.to(dev, non_blocking=True).contiguous(memory_format=torch.channels_last)
    dev_y = host_y.to(dev, non_blocking=True)
    h2d_bytes = host_x.numel() * host_x.element_size() + host_y.numel() * host_y.element_size()

    def step(x, y):
        with torch.autocast(device_type="blackwell", dtype=torch.bfloat16):
            loss = criterion(fdp(x), y)
        loss.backward()
        fdp.step()
        return loss

    def to_compute_layout(batch):
        # runs on the IO queue: the cast to the compute dtype that autocast would otherwise do on the
        # compute queue at the start of every step
        x, y = batch
        return x.to(torch.bfloat16), y

    def e2e_steps(n):
        # Every step's batch is copied from pinned host memory inside the timed region; two batches are in
        # flight on an IO queue.
        last = None
        loader = PrefetchLoader(((host_x, host_y) for _ in range(n)), dev, use_io_queue=True, pin=False, depth=2,
                                transform=to_compute_layout)
        # every step's loss is read back, one step late, through pinned memory on a side queue (the host stays one
        # step ahead of the device); the last one is read before the timed region ends
        reader = DelayedScalar()
        for x, y in loader:
            v = reader.push(step(x, y))  # device -> host read of the result
            last = v if v is not None else last
        v = reader.flush()
        return v if v is not None else last

    def barrier():
        if world > 1:
            dist.barrier()
        torch.b200.synchronize()

    def timed(fn, steps, whole_loop=False):
        barrier()
        q = torch.b200.current_queue()
        start, end = torch.b200.Notifier(), torch.b200.Notifier()
        start.place(q)
        if whole_loop:
            out = fn(steps)
        else:
            for _ in range(steps):
                out = fn()
        end.place(q)
        end.synchronize()
        barrier()
        ms = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms, out

    for _ in range(max(args.warmup, 3)):
        step(dev_x, dev_y)
    barrier()
    catch_b200._C._reset_kernel_launch_count()
    t_begin = time.time()
    ms, loss = timed(lambda: step(dev_x, dev_y), args.steps)
    t_end = time.time()
    launches = catch_b200._C._kernel_launch_count()
    e2e_steps(2)
    ms_e2e, _ = timed(e2e_steps, args.steps, whole_loop=True)
    identical = None
    if world > 1:
        words = torch.tensor(checksum_words(b.flat for b in fdp.buckets), dtype=torch.int64).to(dev)
        allw = [torch.empty_like(words) for _ in range(world)]
        dist.all_gather(allw, words)
        identical = all(bool((w.cpu() == allw[0].cpu()).all()) for w in allw)
    from catch_b200.ops import capi

    res = {"ms": ms, "ms_e2e": ms_e2e, "loss": float(loss.item()), "launches": int(launches), "h2d_bytes": int(h2d_bytes),
           "identical": identical, "clocks": sampler.summary(t_begin, t_end) if sampler is not None else {},
           "kernel_error_flag": capi.read_error_flag()}
    if world > 1:
        dist.destroy_process_group()
    return res


def make_store(rank, world):
    """One TCP store for both arms (each initialises its process group on a prefix of it).  Under torchrun's
    static rendezvous the agent already serves a store on MASTER_PORT and the workers connect as clients."""
    import datetime

    import torch.distributed as dist

    addr = os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ["MASTER_PORT"])
    try:
        from torch.distributed.rendezvous import _create_c10d_store

        return _create_c10d_store(addr, port, rank, world, datetime.timedelta(seconds=600))
    except ImportError:
        agent = os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "False") == "True"
        return dist.TCPStore(addr, port, world, (rank == 0) and not agent, wait_for_workers=not agent)


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "Cambricon CATCH needs the Neuware SDK and MLU370 hardware; offline pip install stops at "
                          "'NEUWARE_HOME Environment Variable has not been set'"}))
        return 0

    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    # Host threads and the pinned staging buffers stay on the GPU's NUMA node.  The helper is loaded from its
    # file: importing the catch_b200 package registers the blackwell device with PyTorch, after which autograd
    # on torch.cuda tensors no longer works in this process, and the stock arm has to run before that.
    import importlib.util

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    spec = importlib.util.spec_from_file_location("_bench_numa", os.path.join(here, "catch_b200", "utils", "numa.py"))
    numa = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(numa)
    numa_node = numa.bind_to_device_node(local_rank)
    store = None
    if world > 1:
        store = make_store(rank, world)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler is not None:
        sampler.start()  # started before the warm-up: nvidia-smi needs a moment before its first sample

    B = args.batch
    config = {"model": args.model, "global_batch": world * B, "per_gpu_batch": B, "image": "3x224x224", "seq_len": None,
              "optimizer": "SGD(momentum 0.9, lr 0.1, wd 1e-4)", "bucket_mb": 25, "parallelism": f"dp{world}",
              "memory_format": "channels_last", "numa_node": numa_node,
              "l2_note": "per-step inputs (154 MB) and activations exceed the 126 MB L2"}
    common = {"metric": "ResNet-50 train images/sec", "unit": "images/sec", "n_gpus": world, "steps": args.steps,
              "warmup": max(args.warmup, 3), "higher_is_better": True, "scaling": "weak", "dtype": "bf16",
              "data": "synthetic N(0,1) images, uniform labels, random-init weights"}

    stock = None
    if args.impl == "stock" or not args.no_stock:
        try:
            stock = run_stock(args, rank, local_rank, world, store, sampler)
        except Exception as e:  # the stock arm must never take the main arm down with it
            if args.impl == "stock":
                raise
            import traceback

            traceback.print_exc(file=sys.stderr)
            stock = {"error": f"{type(e).__name__}: {e}"[:300]}
            if dist.is_initialized():
                dist.destroy_process_group()
    if args.impl == "stock":
        if rank == 0:
            line = dict(common, impl="stock", value=stock["value"], ms_per_step=stock["ms_per_step"],
                        vs_baseline=(stock["value"] / STOCK_IMAGES_PER_SEC[world]) if world in STOCK_IMAGES_PER_SEC else None,
                        config=dict(config, stack=stock["stack"]), clocks=stock["clocks"], gpu_launches=0,
                        e2e={"value": stock["e2e_value"], "unit": "images/sec", "ms_per_step": stock["e2e_ms_per_step"],
                             "h2d_bytes_per_step": B * 3 * 224 * 224 * 4 + B * 8, "d2h_bytes_per_step": 4},
                        final_loss=stock["final_loss"], params_identical_across_ranks=stock["params_identical_across_ranks"])
            print(json.dumps(line))
        if sampler is not None:
            sampler.stop()
        return 0

    ours = run_ours(args, rank, local_rank, world, store, sampler)
    if sampler is not None:
        sampler.stop()
    if rank == 0:
        ips = world * B * args.steps / (ours["ms"] / 1e3)
        ips_e2e = world * B * args.steps / (ours["ms_e2e"] / 1e3)
        base = STOCK_IMAGES_PER_SEC.get(world)
        line = dict(common, impl="ours", value=round(ips, 1), ms_per_step=round(ours["ms"] / args.steps, 3),
                    vs_baseline=round(ips / base, 4) if base else None,
                    baseline={"value": base, "what": "stock PyTorch CUDA + cuDNN + NCCL DDP, same config, same pool "
                                                     "(bench.py --impl stock)"},
                    config=dict(config, module_fusion="catch_b200.fusion.fuse_bn_act", grad_allreduce_dtype=args.grad_dtype),
                    clocks=ours["clocks"], gpu_launches=ours["launches"],
                    e2e={"value": round(ips_e2e, 1), "unit": "images/sec", "ms_per_step": round(ours["ms_e2e"] / args.steps, 3),
                         "h2d_bytes_per_step": ours["h2d_bytes"], "d2h_bytes_per_step": 4},
                    final_loss=ours["loss"], params_identical_across_ranks=ours["identical"],
                    kernel_error_flag=ours["kernel_error_flag"])
        if stock is not None:
            line["stock"] = stock
            if "value" in stock:
                line["vs_stock_same_run"] = round(ips / stock["value"], 4)
                line["e2e_vs_stock_same_run"] = round(ips_e2e / stock["e2e_value"], 4)
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
