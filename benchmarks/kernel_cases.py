"""One hot kernel at a time on an input larger than the L2 cache, device-timed, with its roofline fraction.

    python benchmarks/kernel_cases.py --case gemm_ffn [--iters 5]
    python benchmarks/kernel_cases.py --list

Each case is also the small, single-kernel workload used for `ncu --set full --clock-control none -k regex:<kernel>
-c 1` captures (a few hundred MB on the device, a handful of launches).  The denominators are the measured copy
bandwidth and cuBLAS bf16 burst throughput of MEASURED_PEAKS.json when that file exists, else 6.65 TB/s and
1.59 PFLOP/s ("fallback").
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.nn.functional as F

import catch_b200  # noqa: F401

DEV = "blackwell"


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def rnd(*shape, dtype=torch.bfloat16):
    return torch.randn(*shape).to(dtype).to(DEV)


def case_gemm_ffn():
    a, b = rnd(4096, 768), rnd(768, 3072)
    return (lambda: a @ b), 2.0 * 4096 * 768 * 3072, (4096 * 768 + 768 * 3072 + 4096 * 3072) * 2, "gemm_tcgen05_kernel"


def case_gemm_ffn_wgrad():
    # weight gradient of the same layer: K = 4096 tokens, split among CTAs, fp32 reduce-add epilogue
    x, g = rnd(4096, 768), rnd(4096, 3072)
    w = rnd(3072, 768)
    acc = torch.zeros(3072 * 768, device=DEV)
    fn = lambda: torch.ops.catch_b200.linear_backward_fp32w(g, x, w, False, True, False, acc, None)
    return fn, 2.0 * 4096 * 768 * 3072, (4096 * 768 + 4096 * 3072) * 2 + 3072 * 768 * 4, "gemm_tcgen05_kernel"


def case_gemm_square():
    a, b = rnd(8192, 8192), rnd(8192, 8192)
    return (lambda: a @ b), 2.0 * 8192 ** 3, 3 * 8192 * 8192 * 2, "gemm_tcgen05_kernel"


def _bn_tensors():
    x = rnd(256, 256, 56, 56).contiguous(memory_format=torch.channels_last)  # 411 MB
    bn = torch.nn.BatchNorm2d(256).to(DEV)
    return x, bn


def case_bn_fwd():
    x, bn = _bn_tensors()
    fn = lambda: torch.ops.catch_b200.batch_norm_act(x, bn.weight, bn.bias, bn.running_mean, bn.running_var, None, True, 0.1,
                                                    1e-5, 1)
    return fn, 0, x.numel() * 2 * 3, "bn_"  # statistics pass + apply pass (read, read, write)


def case_bn_bwd():
    x, bn = _bn_tensors()
    out, mean, rstd = torch.ops.catch_b200.batch_norm_act(x, bn.weight, bn.bias, bn.running_mean, bn.running_var, None, True,
                                                          0.1, 1e-5, 1)[:3]
    gy = torch.randn_like(out)
    fn = lambda: torch.ops.catch_b200.batch_norm_act_backward(gy, out, x, bn.weight, None, mean, rstd, True, 1, False)
    return fn, 0, x.numel() * 2 * 5, "bn_bwd"  # reduce (dy, x) + apply (dy, x -> dx)


def case_softmax_xent():
    logits = rnd(8192, 30522)  # 500 MB
    target = torch.randint(0, 30522, (8192,)).to(DEV)
    fn = lambda: torch.ops.catch_b200.softmax_cross_entropy(logits, target, -100, 0.0)
    return fn, 0, logits.numel() * 2 * 2, "softmax_xent"  # logits read once, gradient written once


def case_layernorm():
    h, r = rnd(262144, 768), rnd(262144, 768)  # 400 MB each
    ln = torch.nn.LayerNorm(768).to(DEV)
    fn = lambda: torch.ops.catch_b200.dropout_add_layer_norm(h, r, ln.weight, ln.bias, 0.1, True, 1e-5)
    return fn, 0, h.numel() * 2 * 4 + h.numel() // 8, "dropout_add_layernorm"  # h, r -> s, y (+ bit mask)


def case_maxpool():
    x = rnd(256, 64, 112, 112).contiguous(memory_format=torch.channels_last)  # 411 MB
    fn = lambda: F.max_pool2d(x, 3, 2, 1)
    return fn, 0, x.numel() * 2 * 1.25, "maxpool_fwd"


def case_sgd():
    n = 64 << 20  # 64 M parameters: 256 MB each of params, grads, momentum
    p, g, m = torch.randn(n).to(DEV), torch.randn(n).to(DEV), torch.zeros(n).to(DEV)
    lowp = torch.empty(n, dtype=torch.bfloat16, device=DEV)
    fn = lambda: torch.ops.catch_b200.fused_sgd_step([p], [g], [m], [lowp], 0.1, 0.9, 0.0, 1e-4, False, False, 1.0)
    return fn, 0, n * (4 * 5 + 2), "sgd_kernel"


def case_add():
    a, b = rnd(256, 256, 56, 56), rnd(256, 256, 56, 56)
    return (lambda: a + b), 0, a.numel() * 2 * 3, "ew_vec"


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="gemm_ffn")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--list", action="store_true")
    args = ap.parse_args()
    if args.list:
        print("\n".join(CASES))
        return
    bw, fl, which = peaks()
    with torch.no_grad():
        fn, flops, nbytes, kernel = CASES[args.case]()
        flush = torch.empty(192 << 20, dtype=torch.uint8, device=DEV)
        for _ in range(3):
            fn()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            a, b = torch.b200.Notifier(), torch.b200.Notifier()
            a.place(); fn(); b.place()
            torch.b200.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
    ts.sort()
    us = ts[len(ts) // 2]
    line = f"{args.case}: {us:.1f} us (kernel regex {kernel})"
    if flops:
        line += f", {flops / us / 1e6:.0f} TFLOP/s = {flops / us / 1e-6 / fl:.2f} of {which} cuBLAS bf16"
    line += f", {nbytes / us / 1e3:.0f} GB/s algorithmic = {nbytes / us / 1e-6 / bw:.2f} of {which} copy bandwidth"
    print(line)


if __name__ == "__main__":
    main()
