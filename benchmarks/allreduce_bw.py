"""All-reduce bus bandwidth of the bwccl kernels (nccl-tests definition:
busbw = algbw * 2 (n-1) / n, algbw = bytes / time), device-timed, max over ranks.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/allreduce_bw.py [--nccl]

``--nccl`` measures stock NCCL on torch.cuda tensors on the same GPUs for comparison.
Sizes sweep 1 KB ... 1 GB (symmetric-memory in-place path: no staging copies).
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--nccl", action="store_true")
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    dtype = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    es = 4 if args.dtype == "fp32" else 2
    sizes = [1 << k for k in range(10, 31) if (1 << k) <= args.max_mb << 20]
    if args.nccl:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl")
        dev = torch.device("cuda", local)
        buf = torch.zeros(max(sizes) // es, dtype=dtype, device=dev)
        sync = torch.cuda.synchronize
        mk = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
        rec = lambda e: e.record()  # noqa: E731
        run = lambda t: dist.all_reduce(t)  # noqa: E731
    else:
        import catch_b200  # noqa: F401
        from catch_b200.distributed import get_backend

        os.environ.setdefault("CATCH_B200_SYMM_USER_MB", str(args.max_mb + 64))
        torch.b200.set_device(local)
        dist.init_process_group("bwccl")
        dev = torch.device("blackwell", local)
        pg = get_backend()
        buf = pg.symm_empty(max(sizes) // es, dtype)
        buf.zero_()
        sync = torch.b200.synchronize
        mk = lambda: torch.b200.Notifier()  # noqa: E731
        rec = lambda e: e.place()  # noqa: E731
        run = lambda t: pg.allreduce_symm(t).wait()  # noqa: E731
    if rank == 0:
        print(f"# {'nccl' if args.nccl else 'bwccl'} all-reduce, {world} ranks, {args.dtype}")
        print(f"{'bytes':>12s} {'us':>10s} {'algbw GB/s':>11s} {'busbw GB/s':>11s}")
    for nbytes in sizes:
        t = buf[: nbytes // es]
        for _ in range(3):
            run(t)
        dist.barrier()
        sync()
        a, b = mk(), mk()
        rec(a)
        for _ in range(args.iters):
            run(t)
        rec(b)
        sync()
        ms = torch.tensor([a.elapsed_time(b) / args.iters], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        us = ms.item() * 1e3
        alg = nbytes / (us * 1e-6) / 1e9
        if rank == 0:
            print(f"{nbytes:12d} {us:10.1f} {alg:11.1f} {alg * 2 * (world - 1) / world:11.1f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
