"""Data-parallel ResNet-50 training, one process per GPU (counterpart of the
reference's examples/training/multi_card_demo.py).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/multi_card_train.py [--fused]

Default: stock ``DistributedDataParallel`` over the ``bwccl`` backend.  ``--fused``
uses ``FusedDataParallel`` (all-reduce fused with the optimizer step).
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist
import torchvision

import catch_b200  # noqa: F401
from catch_b200.optim import FusedSGD
from catch_b200.parallel import FusedDataParallel


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--fused", action="store_true")
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--image", type=int, default=224)
    args = ap.parse_args()
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.b200.set_device(local)
    dist.init_process_group("bwccl")
    dev = torch.device("blackwell", local)
    model = getattr(torchvision.models, args.model)().to(dev).to(memory_format=torch.channels_last)
    if args.fused:
        ddp = FusedDataParallel(model, "sgd", lr=0.1, momentum=0.9, weight_decay=1e-4)
        opt = None
    else:
        ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local])
        opt = FusedSGD(ddp.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    g = torch.Generator().manual_seed(rank)
    for i in range(args.iters):
        x = torch.randn(args.batch, 3, args.image, args.image, generator=g).to(dev)
        y = torch.randint(0, 1000, (args.batch,), generator=g).to(dev)
        with torch.autocast(device_type="blackwell", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(ddp(x), y)
        if opt is not None:
            opt.zero_grad(set_to_none=True)
        loss.backward()
        ddp.step() if opt is None else opt.step()
        if rank == 0:
            print(f"iter {i}: loss {loss.item():.4f}")
    # collectives demo: all-reduce / broadcast / all-gather
    t = torch.full((4,), float(rank), device=dev)
    dist.all_reduce(t)
    outs = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(outs, t)
    dist.broadcast(t, 0)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
