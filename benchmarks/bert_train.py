"""BERT-base training throughput (sequences/sec): seq 128, per-GPU batch 32, bf16
autocast, AdamW(lr 2e-5, wd 0.01), 2-class head, synthetic token ids.

    python benchmarks/bert_train.py [--stock] [--steps 10]                       (1 GPU)
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bert_train.py

Ours: the blackwell device with the fused all-reduce + AdamW data-parallel wrapper.
``--stock``: the same model definition on torch.cuda with NCCL DDP and torch.optim.AdamW.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import importlib.util

import torch
import torch.distributed as dist

# The model definition is loaded by path so that the --stock arm never imports the package
# (registering a PrivateUse1 backend changes which accelerator autograd's stream logic tracks).
_spec = importlib.util.spec_from_file_location(
    "_bert_def", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "catch_b200", "models", "bert.py"))
_bert = importlib.util.module_from_spec(_spec)
sys.modules["_bert_def"] = _bert
_spec.loader.exec_module(_bert)
BertConfig, BertForSequenceClassification = _bert.BertConfig, _bert.BertForSequenceClassification


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--stock", action="store_true")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--no-fuse", action="store_true", help="ours: keep the unfused module definitions")
    args = ap.parse_args()
    rank, local, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.manual_seed(0)
    model = BertForSequenceClassification(BertConfig(num_hidden_layers=args.layers))
    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, 30522, (args.batch, args.seq), generator=g)
    y = torch.randint(0, 2, (args.batch,), generator=g)
    if args.stock:
        torch.cuda.set_device(local)
        dev, dtype_dev = torch.device("cuda", local), "cuda"
        if world > 1:
            dist.init_process_group("nccl")
        model = model.to(dev)
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
        opt = torch.optim.AdamW(net.parameters(), lr=2e-5, weight_decay=0.01)
        sync, mk, rec = torch.cuda.synchronize, (lambda: torch.cuda.Event(enable_timing=True)), (lambda e: e.record())

        def finish():
            opt.step(); opt.zero_grad(set_to_none=True)
    else:
        import catch_b200  # noqa: F401
        from catch_b200.parallel import FusedDataParallel

        torch.b200.set_device(local)
        dev, dtype_dev = torch.device("blackwell", local), "blackwell"
        if world > 1:
            os.environ.setdefault("CATCH_B200_SYMM_USER_MB", "2048")
            dist.init_process_group("bwccl")
        if not args.no_fuse:
            _bert.fuse_bert(model)   # fused residual blocks, copy-free attention products, linears with bucket gradients
        net = FusedDataParallel(model.to(dev), "adamw", lr=2e-5, weight_decay=0.01)
        sync, mk, rec = torch.b200.synchronize, (lambda: torch.b200.Notifier()), (lambda e: e.place())
        finish = net.step
    ids, y = ids.to(dev), y.to(dev)

    def step():
        with torch.autocast(device_type=dtype_dev, dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(net(ids), y)
        loss.backward()
        finish()
        return loss

    for _ in range(args.warmup):
        step()
    if world > 1:
        dist.barrier()
    sync()
    a, b = mk(), mk()
    rec(a)
    for _ in range(args.steps):
        loss = step()
    rec(b)
    sync()
    ms = torch.tensor([a.elapsed_time(b) / args.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    launches = None
    if not args.stock:
        import catch_b200 as _pkg

        _pkg._C._reset_kernel_launch_count()
        step()
        sync()
        launches = int(_pkg._C._kernel_launch_count())
    if rank == 0:
        print(f"{'stock' if args.stock else 'catch_b200'} BERT-base x{world}: {ms.item():.2f} ms/step, "
              f"{world * args.batch / ms.item() * 1e3:.1f} sequences/sec, loss {loss.item():.4f}"
              + (f", {launches} kernel launches per step" if launches is not None else ""))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
