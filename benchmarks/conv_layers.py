"""Per-layer convolution timings for the ResNet-50 shapes (batch 256, bf16, NHWC):
this backend's tcgen05 kernels against stock PyTorch (cuDNN) on the same GPU.

    python benchmarks/conv_layers.py [--batch 256] [--iters 10] [--no-stock] [--layer IDX]

Prints, for forward / data-gradient / weight-gradient of each distinct layer shape,
microseconds, TFLOP/s and the bound implied by the measured peaks (time at the bf16
GEMM peak vs time to move the operands once at the copy bandwidth).
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.nn.functional as F

import catch_b200  # noqa: F401

# (Cin, H, Cout, R, stride, pad, count in ResNet-50)
LAYERS = [
    (3, 224, 64, 7, 2, 3, 1),
    (64, 56, 64, 1, 1, 0, 1), (64, 56, 64, 3, 1, 1, 3), (64, 56, 256, 1, 1, 0, 4), (256, 56, 64, 1, 1, 0, 2),
    (256, 56, 128, 1, 1, 0, 1), (128, 56, 128, 3, 2, 1, 1), (128, 28, 512, 1, 1, 0, 4), (256, 56, 512, 1, 2, 0, 1),
    (512, 28, 128, 1, 1, 0, 3), (128, 28, 128, 3, 1, 1, 3),
    (512, 28, 256, 1, 1, 0, 1), (256, 28, 256, 3, 2, 1, 1), (256, 14, 1024, 1, 1, 0, 6), (512, 28, 1024, 1, 2, 0, 1),
    (1024, 14, 256, 1, 1, 0, 5), (256, 14, 256, 3, 1, 1, 5),
    (1024, 14, 512, 1, 1, 0, 1), (512, 14, 512, 3, 2, 1, 1), (512, 7, 2048, 1, 1, 0, 3), (1024, 14, 2048, 1, 2, 0, 1),
    (2048, 7, 512, 1, 1, 0, 2), (512, 7, 512, 3, 1, 1, 2),
]


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def time_fn(fn, iters, sync, ev, rec, flush):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush()
        a, b = ev(), ev()
        rec(a); fn(); rec(b)
        sync()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2] * 1e3  # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--no-stock", action="store_true")
    ap.add_argument("--layer", type=int, default=-1, help="index into the layer table; -1 = all")
    args = ap.parse_args()
    bw, fl, src = peaks()
    N = args.batch
    dev = torch.device("blackwell", 0)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    cflush = None if args.no_stock else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    tot = {"ours": 0.0, "stock": 0.0, "bound": 0.0}
    print(f"peaks ({src}): {bw / 1e12:.2f} TB/s, {fl / 1e12:.0f} TFLOP/s")
    print(f"{'layer':34s} {'pass':6s} {'ours us':>9s} {'TF/s':>7s} {'stock us':>9s} {'bound us':>9s} {'ours/bound':>10s}")
    for (C, H, K, R, s, p, cnt) in (LAYERS if args.layer < 0 else [LAYERS[args.layer]]):
        P = (H + 2 * p - R) // s + 1
        x = torch.randn(N, C, H, H).bfloat16()
        w = (torch.randn(K, C, R, R) / (C * R * R) ** 0.5).bfloat16()
        gy = torch.randn(N, K, P, P).bfloat16()
        flops = 2.0 * N * P * P * K * C * R * R
        bytes_ = 2.0 * (N * C * H * H + K * C * R * R + N * K * P * P)
        bound = max(flops / fl, bytes_ / bw) * 1e6
        res = {}
        for arm in (["ours"] if args.no_stock else ["ours", "stock"]):
            d = dev if arm == "ours" else torch.device("cuda", 0)
            xd = x.to(d).contiguous(memory_format=torch.channels_last)
            wd = w.to(d).contiguous(memory_format=torch.channels_last)
            gd = gy.to(d).contiguous(memory_format=torch.channels_last)
            if arm == "ours":
                sync, ev, rec = torch.b200.synchronize, (lambda: torch.b200.Notifier()), (lambda e: e.place())
                flush = lambda: flush_buf.zero_()  # noqa: E731
                bwd = lambda m: torch.ops.aten.convolution_backward(gd, xd, wd, None, [s, s], [p, p], [1, 1], False, [0, 0], 1, m)  # noqa: E731
            else:
                torch.backends.cudnn.benchmark = True
                sync, ev, rec = torch.cuda.synchronize, (lambda: torch.cuda.Event(enable_timing=True)), (lambda e: e.record())
                flush = lambda: cflush.zero_()  # noqa: E731
                bwd = lambda m: torch.ops.aten.convolution_backward(gd, xd, wd, None, [s, s], [p, p], [1, 1], False, [0, 0], 1, m)  # noqa: E731
            t_f = time_fn(lambda: F.conv2d(xd, wd, None, s, p), args.iters, sync, ev, rec, flush)
            t_d = time_fn(lambda: bwd([True, False, False]), args.iters, sync, ev, rec, flush) if C >= 8 else 0.0
            t_w = time_fn(lambda: bwd([False, True, False]), args.iters, sync, ev, rec, flush)
            res[arm] = (t_f, t_d, t_w)
        name = f"{C}x{H}x{H}->{K} k{R} s{s} (x{cnt})"
        for i, ps in enumerate(("fprop", "dgrad", "wgrad")):
            o = res["ours"][i]
            st = res["stock"][i] if "stock" in res else 0.0
            if o == 0.0:
                continue
            print(f"{name:34s} {ps:6s} {o:9.1f} {flops / o / 1e6:7.1f} {st:9.1f} {bound:9.1f} {o / bound:10.2f}")
            tot["ours"] += o * cnt; tot["stock"] += st * cnt; tot["bound"] += bound * cnt
    print(f"TOTAL over ResNet-50 (weighted by layer count): ours {tot['ours'] / 1e3:.2f} ms, stock {tot['stock'] / 1e3:.2f} ms, "
          f"bound {tot['bound'] / 1e3:.2f} ms")


if __name__ == "__main__":
    main()
