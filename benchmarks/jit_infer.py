"""ResNet-50 fusion-mode (TorchScript) inference, fp16, batch 64, one GPU.

    python benchmarks/jit_infer.py [--stock] [--batch 64] [--iters 30]

Ours: trace on the blackwell device, ``catch_b200.jit.optimize`` (BN folded into the
convolutions, conv+ReLU(+residual) / linear chains lowered to fused tcgen05 ops inside
fusion groups).  ``--stock``: ``torch.jit.trace`` + ``torch.jit.freeze`` +
``optimize_for_inference`` on torch.cuda (cuDNN).  Prints images/sec (device events)
and the relative RMS error of the fused output against eager fp32 on the CPU.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torchvision


def rel_rms(a, b):
    a, b = a.double(), b.double()
    return ((a - b).pow(2).sum() / b.pow(2).sum()).sqrt().item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--stock", action="store_true")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--iters", type=int, default=30)
    args = ap.parse_args()
    torch.manual_seed(0)
    model = torchvision.models.resnet50().eval()
    for m in model.modules():
        if isinstance(m, torch.nn.BatchNorm2d):
            m.running_mean.normal_(0, 0.1); m.running_var.uniform_(0.5, 1.5)
    x = torch.randn(args.batch, 3, 224, 224)
    with torch.no_grad():
        ref = model(x[:8])
    if args.stock:
        dev = torch.device("cuda", 0)
        torch.backends.cudnn.benchmark = True
        sync, mk, rec = torch.cuda.synchronize, (lambda: torch.cuda.Event(enable_timing=True)), (lambda e: e.record())
    else:
        import catch_b200  # noqa: F401
        from catch_b200 import jit

        dev = torch.device("blackwell", 0)
        sync, mk, rec = torch.b200.synchronize, (lambda: torch.b200.Notifier()), (lambda e: e.place())
    m = model.half().to(dev).to(memory_format=torch.channels_last)
    xd = x.half().to(dev).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        traced = torch.jit.trace(m, xd)
        if args.stock:
            fused = torch.jit.optimize_for_inference(torch.jit.freeze(traced))
        else:
            fused = jit.optimize(traced)
        for _ in range(5):
            out = fused(xd)
        err = rel_rms(fused(xd[:8]).float().cpu(), ref)
        sync()
        a, b = mk(), mk()
        rec(a)
        for _ in range(args.iters):
            out = fused(xd)
        rec(b)
        sync()
    ms = a.elapsed_time(b) / args.iters
    extra = "" if args.stock else f", fusion groups {str(fused.graph).count('FusionGroup')}, stats {jit.fusion_stats()}"
    print(f"{'stock' if args.stock else 'catch_b200'} resnet50 fp16 fusion inference batch {args.batch}: {ms:.3f} ms, "
          f"{args.batch / ms * 1e3:.1f} images/sec, rel-RMS vs eager fp32 {err:.2e}{extra}")
    assert out.shape == (args.batch, 1000)


if __name__ == "__main__":
    main()
