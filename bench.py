"""Headline benchmark: ResNet-50 training throughput (images/sec) on N B200s.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

Config (the reference's DDP benchmark harness model, test/cnnl/test_ddp_benchmark.py,
at the B200 batch size): torchvision ResNet-50, random-init weights, bf16 autocast,
per-GPU batch 256 of 3x224x224 N(0,1) images with uniform labels from a per-rank
seed, SGD momentum 0.9 / lr 0.1 / wd 1e-4, 25 MB gradient buckets reduced by the
fused peer-memory all-reduce + optimizer kernel.  Everything runs through this
repository's public API on the ``blackwell`` device.

Two timed regions, both K steps after W warm-up steps, bracketed by a barrier and a
device synchronize, timed with device events, max over ranks:
  * ``value``   : inputs already resident on the device;
  * ``e2e``     : each step copies its batch from pinned host memory and reads the loss
                  back to the host.
``--impl reference`` reports that the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

BASELINE_IMAGES_PER_SEC = None  # the reference publishes no throughput number


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="per-GPU batch size")
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--grad-dtype", default="fp32", choices=["fp32", "bf16"])
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

    def stop(self, t0: float = 0.0, t1: float = float("inf")) -> dict:
        """Summarise the samples taken between host times t0 and t1 (the timed region)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for ts, ln in self.lines:
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


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "Cambricon CATCH needs the Neuware SDK and MLU370 hardware; offline pip install stops at "
                          "'NEUWARE_HOME Environment Variable has not been set'"}))
        return 0

    import torch
    import torch.distributed as dist
    import torchvision

    import catch_b200  # noqa: F401
    from catch_b200.fusion import fuse_bn_act
    from catch_b200.parallel import FusedDataParallel

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    assert torch.b200.backend_name() == "cuda", "bench.py needs a GPU (the host-simulated device is for tests)"
    torch.b200.set_device(local_rank)
    dev = torch.device("blackwell", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("bwccl", rank=rank, world_size=world)

    torch.manual_seed(0)
    model = getattr(torchvision.models, args.model)(weights=None)
    model = fuse_bn_act(model)  # same parameters / state dict; BN(+add)+ReLU chains run as fused kernels
    model = model.to(dev).to(memory_format=torch.channels_last)
    grad_dtype = torch.bfloat16 if args.grad_dtype == "bf16" else torch.float32
    fdp = FusedDataParallel(model, "sgd", lr=0.1, momentum=0.9, weight_decay=1e-4, bucket_mb=25.0, grad_dtype=grad_dtype)
    criterion = torch.nn.CrossEntropyLoss()

    B = args.batch
    g = torch.Generator().manual_seed(1234 + rank)
    host_x = torch.b200.pin_memory(torch.randn(B, 3, 224, 224, generator=g))
    host_y = torch.b200.pin_memory(torch.randint(0, 1000, (B,), generator=g))
    dev_x = host_x.to(dev, non_blocking=True).contiguous(memory_format=torch.channels_last)
    dev_y = host_y.to(dev, non_blocking=True)
    h2d_bytes = host_x.numel() * host_x.element_size() + host_y.numel() * host_y.element_size()

    def step(x, y):
        with torch.autocast(device_type="blackwell", dtype=torch.bfloat16):
            loss = criterion(fdp(x), y)
        loss.backward()
        fdp.step()
        return loss

    def resident_step():
        return step(dev_x, dev_y)

    def e2e_steps(n):
        # Every step's batch is copied from pinned host memory inside the timed region; the copy of
        # step i+1 is queued on an IO queue before the host blocks on step i's loss.
        from catch_b200.utils import PrefetchLoader

        last = None
        for x, y in PrefetchLoader(((host_x, host_y) for _ in range(n)), dev, use_io_queue=True, pin=False):
            last = step(x, y).item()  # device -> host read of the result
        return last

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

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # started before the warm-up: nvidia-smi needs a moment before its first sample
    for _ in range(max(args.warmup, 3)):
        resident_step()
    barrier()
    catch_b200._C._reset_kernel_launch_count()
    t_begin = time.time()
    ms, loss = timed(resident_step, args.steps)
    t_end = time.time()
    launches = catch_b200._C._kernel_launch_count()
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else {}
    e2e_steps(2)
    ms_e2e, _ = timed(e2e_steps, args.steps, whole_loop=True)

    if rank == 0:
        ips = world * B * args.steps / (ms / 1e3)
        ips_e2e = world * B * args.steps / (ms_e2e / 1e3)
        print(json.dumps({
            "metric": "ResNet-50 train images/sec", "value": round(ips, 1), "unit": "images/sec", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 3),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (ips / BASELINE_IMAGES_PER_SEC) if BASELINE_IMAGES_PER_SEC else None,
            "dtype": "bf16", "data": "synthetic N(0,1) images, uniform labels, random-init weights",
            "config": {"model": args.model, "global_batch": world * B, "per_gpu_batch": B, "image": "3x224x224",
                       "optimizer": "SGD(momentum 0.9, lr 0.1, wd 1e-4)", "bucket_mb": 25,
                       "parallelism": f"dp{world}", "memory_format": "channels_last", "module_fusion": "catch_b200.fusion.fuse_bn_act", "grad_allreduce_dtype": args.grad_dtype,
                       "l2_note": "per-step inputs (154 MB) and activations exceed the 126 MB L2"},
            "clocks": clocks, "gpu_launches": int(launches),
            "e2e": {"value": round(ips_e2e, 1), "unit": "images/sec", "ms_per_step": round(ms_e2e / args.steps, 3),
                    "h2d_bytes_per_step": int(h2d_bytes), "d2h_bytes_per_step": 4},
            "final_loss": float(loss.item() if hasattr(loss, "item") else loss),
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
