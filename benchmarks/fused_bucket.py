"""Time of the fused bucket kernel (gradient reduce-scatter + 1/world + SGD-momentum + parameter all-gather
with the bf16 copy) for one 25 MB gradient bucket, against its NVLink bound.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/fused_bucket.py

Per rank and direction the peer-memory kernel moves (N-1)/N of the bucket's gradients in and (N-1)/N of the
fp32 parameters plus their bf16 copy out; with the multicast mapping the switch does the fan-in / fan-out and a
rank receives 1/N of the gradients and sends 1/N of the parameters (the other direction carries the whole
bucket once).  bound = bytes of the busier direction / 770 GB/s (the measured peer-copy rate per direction);
the optimizer arithmetic is far below that (a few FLOP per byte), so the link is the roofline.
Device-timed, max over ranks.  The kernel uses peer loads / stores unless CATCH_B200_NVLS_FUSED=1 asks for the
in-switch (multimem) variant.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=float, default=25.0)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--grad-dtype", default="fp32", choices=["fp32", "bf16"])
    args = ap.parse_args()
    import catch_b200  # noqa: F401
    from catch_b200.distributed import get_backend

    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.b200.set_device(local)
    dist.init_process_group("bwccl")
    dev = torch.device("blackwell", local)
    pg = get_backend()
    n = int(args.mb * 1024 * 1024 / 4)
    gdt = torch.float32 if args.grad_dtype == "fp32" else torch.bfloat16
    pad = max(pg.shard_elems(n, torch.float32), pg.shard_elems(n, gdt)) * world
    params = pg.symm_empty(pad, torch.float32)[:n]
    lowp = pg.symm_empty(pad, torch.bfloat16)[:n]
    comm = pg.symm_empty(pad, gdt)
    local_grads = torch.empty(pad, dtype=torch.float32, device=dev) if gdt != torch.float32 else None
    shard = pg.shard_elems(n, gdt)
    state = torch.zeros(shard, device=dev)
    params.normal_()
    (local_grads if local_grads is not None else comm).normal_()
    dist.barrier()
    mc = pg.multicast_enabled() and os.environ.get("CATCH_B200_NVLS_FUSED") == "1"

    def run(step):
        return pg.fused_allreduce_step(comm[:n], params, state, torch.empty(0, device=dev), 0, 0.1, 0.9, 0.0, 1e-4, 0.9, 0.999,
                                       1e-8, step, False, step == 1, 1.0 / world, lowp=lowp, cast_src=local_grads,
                                       zero_grads=True)

    for i in range(3):
        run(i + 1).wait()
    dist.barrier()
    torch.b200.synchronize()
    a, b = torch.b200.Notifier(), torch.b200.Notifier()
    a.place()
    for i in range(args.iters):
        run(i + 4).wait()
    b.place()
    torch.b200.synchronize()
    ms = torch.tensor([a.elapsed_time(b) / args.iters], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    us = ms.item() * 1e3
    ges = 4 if gdt == torch.float32 else 2
    if mc:
        ingress = n * ges / world + n * 6 * (world - 1) / world   # my reduced shard + everybody else's parameters
        egress = n * ges * (world - 1) / world + n * 6 / world    # my gradients to the switch + my parameter shard
    else:
        ingress = n * ges * (world - 1) / world + n * 6 * (world - 1) / world / 1  # gradients pulled + parameters pushed to me
        egress = ingress
    bound_us = max(ingress, egress) / 770e9 * 1e6
    if rank == 0:
        print(f"fused bucket kernel, {world} ranks, {args.mb:.0f} MB bucket, gradients cross as {args.grad_dtype}, "
              f"{'multicast (NVLS)' if mc else 'peer loads / stores'}")
        print("us per bucket | MB per rank and direction | bound us at 770 GB/s | fraction of bound")
        print(f"{us:13.1f} | {max(ingress, egress) / 1e6:25.1f} | {bound_us:20.1f} | {bound_us / us:17.2f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
