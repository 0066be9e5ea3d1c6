"""Achieved memory bandwidth of the fused batch-norm kernels on the ResNet-50 activation shapes
(batch 256, bf16, channels-last): forward (statistics from given sums + normalise + ReLU + mask),
backward reduction, backward apply.  Bytes counted are the algorithmic ones (each tensor once).

    python benchmarks/bn_kernels.py [--batch 256] [--iters 10]
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

import catch_b200  # noqa: F401

# (channels, spatial, residual, count in ResNet-50)
SHAPES = [(64, 112, False, 1), (64, 56, False, 6), (256, 56, True, 3), (256, 56, False, 1), (128, 56, False, 1),
          (128, 28, False, 7), (512, 28, True, 4), (512, 28, False, 1), (256, 28, False, 1), (256, 14, False, 11),
          (1024, 14, True, 6), (1024, 14, False, 1), (512, 14, False, 1), (512, 7, False, 5), (2048, 7, True, 3),
          (2048, 7, False, 1)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    dev = torch.device("blackwell", 0)
    peak = 6.45e12
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = json.load(open(p))["hbm_gbs"] * 1e9
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    q = torch.b200.current_queue()

    def time_us(fn):
        fn()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            a, b = torch.b200.Notifier(), torch.b200.Notifier()
            a.place(q); fn(); b.place(q); b.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    tot = {"fwd": [0.0, 0.0], "bwd": [0.0, 0.0]}
    print(f"copy bandwidth used for the bound: {peak / 1e12:.2f} TB/s")
    print(f"{'shape':28s} {'pass':5s} {'us':>8s} {'GB/s':>8s} {'of copy':>8s}")
    for C, H, res, count in SHAPES:
        N = args.batch
        x = torch.randn(N, C, H, H, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        r = torch.randn_like(x) if res else None
        g = torch.randn_like(x)
        w = torch.ones(C, device=dev); b = torch.zeros(C, device=dev)
        rm = torch.zeros(C, device=dev); rv = torch.ones(C, device=dev)
        sums = torch.stack([x.float().sum((0, 2, 3)), (x.float() ** 2).sum((0, 2, 3))]).double().reshape(-1).contiguous()
        out = {}

        def fwd():
            out["r"] = torch.ops.catch_b200.batch_norm_act_mask(x, w, b, rm, rv, r, True, 0.1, 1e-5, 1, sums)

        t_f = time_us(fwd)
        y, mean, invstd, mask = out["r"]

        def bwd():
            torch.ops.catch_b200.batch_norm_act_backward(g, mask, x, w, rm, mean, invstd, True, 1, res)

        t_b = time_us(bwd)
        T = x.numel() * 2
        bytes_f = T * (3 if res else 2) + T / 16
        bytes_b = T * 2 + T / 16 + T * (4 if res else 3) + T / 16  # reduce: dy, x, mask; apply: dy, x, mask -> dx (+ dres)
        name = f"{C}x{H}x{H}{' +res' if res else ''} (x{count})"
        for tag, t, by in (("fwd", t_f, bytes_f), ("bwd", t_b, bytes_b)):
            print(f"{name:28s} {tag:5s} {t:8.1f} {by / t / 1e3:8.0f} {by / t * 1e6 / peak:8.2f}")
            tot[tag][0] += t * count
            tot[tag][1] += by / peak * 1e6 * count
        del x, r, g, y, mask, out
    for tag in ("fwd", "bwd"):
        print(f"TOTAL {tag}: {tot[tag][0] / 1e3:.2f} ms over ResNet-50's batch norms; bytes at copy bandwidth: {tot[tag][1] / 1e3:.2f} ms")


if __name__ == "__main__":
    main()
