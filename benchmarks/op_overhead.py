"""Host-side cost per operator call: tiny tensors, many calls, wall time per call with the device kept busy.

    python benchmarks/op_overhead.py [--stock]

Launch-bound models (BERT-base at batch 32: about 700 launches in a 15 ms step) run at the speed of this number.
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--stock", action="store_true")
    ap.add_argument("--calls", type=int, default=20000)
    args = ap.parse_args()
    if args.stock:
        dev, sync = torch.device("cuda", 0), torch.cuda.synchronize
    else:
        import catch_b200  # noqa: F401

        dev, sync = torch.device("blackwell", 0), torch.b200.synchronize
    x = torch.randn(64, 64, device=dev)
    y = torch.randn(64, 64, device=dev)
    h = torch.randn(64, 64, device=dev).half()
    w = torch.randn(64, 64, device=dev).half()
    ln = torch.nn.LayerNorm(64).to(dev)
    cases = {
        "add": lambda: x + y,
        "add_": lambda: x.add_(y, alpha=0.0),
        "relu": lambda: torch.relu(x),
        "mul scalar": lambda: x * 2.0,
        "mm fp16 64^3": lambda: h @ w,
        "layer_norm": lambda: ln(x),
        "sum": lambda: x.sum(),
        "view + transpose + contiguous": lambda: x.view(8, 8, 64).transpose(0, 1).contiguous(),
        "empty": lambda: torch.empty(64, 64, device=dev),
    }
    print(f"{'stock torch.cuda' if args.stock else 'catch_b200'}: microseconds of host time per call ({args.calls} calls each)")
    with torch.no_grad():
        for name, fn in cases.items():
            for _ in range(200):
                fn()
            sync()
            t0 = time.perf_counter()
            for _ in range(args.calls):
                fn()
            t1 = time.perf_counter()
            sync()
            print(f"  {name:32s} {(t1 - t0) / args.calls * 1e6:6.2f}")


if __name__ == "__main__":
    main()
