"""ResNet-50 post-training int8 inference, batch 128, one GPU.

    python benchmarks/int8_infer.py [--batch 128] [--iters 20]

Per-channel symmetric int8 weights, per-tensor activation scales calibrated on 8
batches of 32 N(0,1) inputs (seed 1); evaluation on fresh N(0,1) inputs.  Reports
images/sec of the int8 and fp16 models on this backend, eager and traced + fused
(catch_b200.jit.optimize: conv + add + ReLU in one kernel; quantized layers hand int8
to each other), and the top-1 agreement with fp16 eager.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torchvision

import catch_b200  # noqa: F401
from catch_b200.quantize import quantize_dynamic


def bench(fn, iters):
    for _ in range(3):
        out = fn()
    torch.b200.synchronize()
    a, b = torch.b200.Notifier(), torch.b200.Notifier()
    a.place()
    for _ in range(iters):
        out = fn()
    b.place()
    torch.b200.synchronize()
    return a.elapsed_time(b) / iters, out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    dev = torch.device("blackwell", 0)
    torch.manual_seed(0)
    # batch norms are folded into the convolutions first (both arms), as any deployment flow does
    from torch.fx.experimental.optimization import fuse as fold_conv_bn
    model = torchvision.models.resnet50().eval()
    for m in model.modules():
        if isinstance(m, torch.nn.BatchNorm2d):
            m.running_mean.normal_(0, 0.1); m.running_var.uniform_(0.5, 1.5)
    model = fold_conv_bn(model)
    mixed = {"conv1": "float"}  # the 3-channel first layer stays in floating point
    calib = quantize_dynamic(model, {"per_channel": True, "iteration": 8}, dtype="int8", gen_quant=True, mixed_layer=mixed)
    calib = calib.half().to(dev).to(memory_format=torch.channels_last)
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for _ in range(8):
            calib(torch.randn(32, 3, 224, 224, generator=g).half().to(dev))
    sd = {k: v.cpu() for k, v in calib.state_dict().items()}
    qmodel = quantize_dynamic(model, mixed_layer=mixed)
    qmodel.load_state_dict(sd, strict=False)
    qmodel = qmodel.half().to(dev).to(memory_format=torch.channels_last)
    import copy
    fmodel = copy.deepcopy(model)
    fmodel = fmodel.half().to(dev).to(memory_format=torch.channels_last)
    x = torch.randn(args.batch, 3, 224, 224, generator=torch.Generator().manual_seed(2)).half().to(dev)
    x = x.contiguous(memory_format=torch.channels_last)
    from catch_b200 import jit

    with torch.no_grad():
        ms_q, out_q = bench(lambda: qmodel(x), args.iters)
        ms_f, out_f = bench(lambda: fmodel(x), args.iters)
        qjit = jit.optimize(torch.jit.trace(qmodel, x))
        fjit = jit.optimize(torch.jit.trace(fmodel, x))
        ms_qj, out_qj = bench(lambda: qjit(x), args.iters)
        ms_fj, out_fj = bench(lambda: fjit(x), args.iters)

    def cmp(o):
        return ((o.argmax(1) == out_f.argmax(1)).float().mean().item(),
                ((o.float() - out_f.float()).norm() / out_f.float().norm()).item())

    nq = sum(1 for m in qmodel.modules() if getattr(m, "is_quantized", lambda: False)())
    print(f"ResNet-50 inference, batch {args.batch}, {nq} quantized layers; images/sec (ms per batch); "
          f"top-1 agreement with / relative RMS to fp16 eager")
    for name, ms, o in (("fp16 eager", ms_f, out_f), ("fp16 fused", ms_fj, out_fj), ("int8 eager", ms_q, out_q),
                        ("int8 fused", ms_qj, out_qj)):
        a, r = cmp(o)
        print(f"{name}: {args.batch / ms * 1e3:9.1f} ({ms:.3f} ms); {a:.3f} / {r:.3e}")


if __name__ == "__main__":
    main()
