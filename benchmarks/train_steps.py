"""Run a few ResNet training steps on one GPU (used for launch lists and ncu captures).

    python benchmarks/train_steps.py --model resnet50 --batch 256 --steps 4 [--stock]

``--stock`` runs the same model / optimizer / autocast configuration on stock PyTorch
CUDA (cuDNN / cuBLAS) for comparison and prints images/sec measured with CUDA events.
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torchvision


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--image", type=int, default=224)
    ap.add_argument("--stock", action="store_true")
    ap.add_argument("--no-fuse", action="store_true", help="do not fuse BN+ReLU chains with catch_b200.fusion.fuse_bn_act")
    args = ap.parse_args()
    torch.manual_seed(0)
    model = getattr(torchvision.models, args.model)(weights=None)
    x = torch.randn(args.batch, 3, args.image, args.image)
    y = torch.randint(0, 1000, (args.batch,))
    if args.stock:
        dev = torch.device("cuda", 0)
        torch.backends.cudnn.benchmark = True
        model = model.to(dev).to(memory_format=torch.channels_last)
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
        x, y = x.to(dev).contiguous(memory_format=torch.channels_last), y.to(dev)
        dtype_dev = "cuda"

        def step():
            opt.zero_grad(set_to_none=True)
            with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
                loss = torch.nn.functional.cross_entropy(model(x), y)
            loss.backward()
            opt.step()
            return loss
        sync = torch.cuda.synchronize
        ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
        rec = lambda e: e.record()  # noqa: E731
    else:
        import catch_b200  # noqa: F401
        from catch_b200.parallel import FusedDataParallel

        from catch_b200.fusion import fuse_bn_act

        dev = torch.device("blackwell", 0)
        if not args.no_fuse:
            model = fuse_bn_act(model)
        model = model.to(dev).to(memory_format=torch.channels_last)
        fdp = FusedDataParallel(model, "sgd", lr=0.1, momentum=0.9, weight_decay=1e-4)
        x, y = x.to(dev).contiguous(memory_format=torch.channels_last), y.to(dev)

        def step():
            with torch.autocast(device_type="blackwell", dtype=torch.bfloat16):
                loss = torch.nn.functional.cross_entropy(fdp(x), y)
            loss.backward()
            fdp.step()
            return loss
        sync = torch.b200.synchronize
        ev = lambda: torch.b200.Notifier()  # noqa: E731
        rec = lambda e: e.place()  # noqa: E731
    for _ in range(args.warmup):
        step()
    sync()
    a, b = ev(), ev()
    rec(a)
    for _ in range(args.steps):
        loss = step()
    rec(b)
    sync()
    ms = a.elapsed_time(b)
    print(f"{'stock' if args.stock else 'catch_b200'} {args.model} batch {args.batch}: "
          f"{ms / args.steps:.2f} ms/step, {args.batch * args.steps / ms * 1e3:.1f} images/sec, loss {loss.item():.4f}")


if __name__ == "__main__":
    main()
