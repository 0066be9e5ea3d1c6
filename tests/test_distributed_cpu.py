"""The bwccl process group on the host-simulated device: collectives, point to
point, DDP end to end against a single-process CPU run, and failure detection
(a rank that never joins -> time-out error on the others).  No GPU needed."""
import datetime
import os

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_ranks

DEV = "blackwell"


def _init(rank, world, timeout_s=60):
    import catch_b200  # noqa: F401

    torch.b200.set_device(rank % torch.b200.device_count())
    dist.init_process_group("bwccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _collectives(rank, world):
    _init(rank, world)
    for dtype in (torch.float32, torch.float64, torch.int64, torch.int32, torch.uint8, torch.bool, torch.bfloat16):
        t = (torch.arange(6) % 2 == 0).to(dtype).to(DEV) if dtype == torch.bool else (torch.arange(6) + rank).to(dtype).to(DEV)
        dist.broadcast(t, 0)
        exp = (torch.arange(6) % 2 == 0).to(dtype) if dtype == torch.bool else torch.arange(6).to(dtype)
        assert torch.equal(t.cpu(), exp), dtype
        outs = [torch.empty_like(t) for _ in range(world)]
        mine = torch.full((6,), rank + 1).to(dtype).to(DEV)
        dist.all_gather(outs, mine)
        for r in range(world):
            assert torch.equal(outs[r].cpu(), torch.full((6,), r + 1).to(dtype)), dtype
    x = torch.full((5, 3), float(rank + 1), device=DEV)
    w = dist.all_reduce(x, async_op=True)
    w.wait()
    assert w.is_completed()
    assert torch.equal(x.cpu(), torch.full((5, 3), float(sum(range(1, world + 1)))))
    for op, exp in ((dist.ReduceOp.PRODUCT, 2.0), (dist.ReduceOp.MIN, 1.0), (dist.ReduceOp.MAX, 2.0)):
        y = torch.full((4,), float(rank + 1), device=DEV)
        dist.all_reduce(y, op=op)
        assert torch.equal(y.cpu(), torch.full((4,), exp)), op
    z = torch.full((4,), float(rank + 1), device=DEV)
    dist.reduce(z, 1)
    if rank == 1:
        assert torch.equal(z.cpu(), torch.full((4,), 3.0))
    big = torch.empty(world * 4, device=DEV)
    dist.all_gather_into_tensor(big, torch.full((4,), float(rank), device=DEV))
    assert torch.equal(big.cpu(), torch.arange(world).repeat_interleave(4).float())
    rs = torch.empty(3, device=DEV)
    dist.reduce_scatter_tensor(rs, torch.arange(world * 3, dtype=torch.float32, device=DEV))
    assert torch.equal(rs.cpu(), world * torch.arange(rank * 3, rank * 3 + 3).float())
    if rank == 0:
        dist.send(torch.tensor([7.0, 8.0], device=DEV), 1)
    else:
        r = torch.zeros(2, device=DEV)
        dist.recv(r, 0)
        assert torch.equal(r.cpu(), torch.tensor([7.0, 8.0]))
    dist.barrier()
    with pytest.raises(Exception, match="destination rank|self"):
        dist.send(torch.zeros(1, device=DEV), rank)
    dist.destroy_process_group()


def test_collectives_two_ranks():
    run_ranks(_collectives, world=2)


def _ddp(rank, world, hook=None):
    _init(rank, world)
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(10, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    ref = torch.nn.Sequential(torch.nn.Linear(10, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    ref.load_state_dict(net.state_dict())
    ddp = torch.nn.parallel.DistributedDataParallel(net.to(DEV))
    if hook is not None:
        from catch_b200.parallel import hooks
        ddp.register_comm_hook(None, getattr(hooks, hook))
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05, momentum=0.9)
    opt_ref = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    g = torch.Generator().manual_seed(1)
    for _ in range(5):
        x = torch.randn(8 * world, 10, generator=g)
        y = torch.randn(8 * world, 4, generator=g)
        opt_ref.zero_grad()
        torch.nn.functional.mse_loss(ref(x), y).backward()
        opt_ref.step()
        xs, ys = x[rank * 8:(rank + 1) * 8].to(DEV), y[rank * 8:(rank + 1) * 8].to(DEV)
        opt.zero_grad()
        torch.nn.functional.mse_loss(ddp(xs), ys).backward()
        opt.step()
    tol = 3e-2 if hook == "bf16_compress_hook" else 3e-3
    for a, b in zip(ref.parameters(), ddp.module.parameters()):
        assert (a - b.cpu()).abs().max().item() < tol
    dist.destroy_process_group()


def test_ddp_matches_single_process_cpu():
    run_ranks(_ddp, world=2)


def _ddp_allreduce_hook(rank, world):
    _ddp(rank, world, "allreduce_hook")


def _ddp_bf16_hook(rank, world):
    _ddp(rank, world, "bf16_compress_hook")


def test_ddp_comm_hooks():
    run_ranks(_ddp_allreduce_hook, world=2)
    run_ranks(_ddp_bf16_hook, world=2)


def _missing_peer(rank, world):
    _init(rank, world, timeout_s=3)
    t = torch.ones(4, device=DEV)
    dist.all_reduce(t)  # both ranks take part once
    if rank == 1:
        os._exit(0)  # leaves between steps, nothing in flight
    try:
        dist.all_reduce(t)
    except Exception as e:  # the surviving rank must get an error, not hang
        assert "imeout" in str(e) or "timed out" in str(e) or "wait" in str(e).lower(), str(e)
        os._exit(0)
    os._exit(3)


def test_rank_that_leaves_is_detected():
    run_ranks(_missing_peer, world=2, timeout=60)


def _heartbeat(rank, world):
    import time

    _init(rank, world, timeout_s=30)
    from catch_b200.distributed import get_backend

    t = torch.ones(4, device=DEV)
    dist.all_reduce(t)
    pg = get_backend()
    assert pg.dead_peer() == -1
    if rank == 1:
        os._exit(0)  # leaves between steps without a goodbye
    deadline = time.time() + 20
    while pg.dead_peer() < 0 and time.time() < deadline:
        time.sleep(0.1)
    assert pg.dead_peer() == 1, "the watchdog did not notice the missing heartbeat"
    t0 = time.time()
    try:
        dist.all_reduce(t)
    except Exception as e:  # raised on the host, before anything is launched and without waiting for the group timeout
        assert "heartbeat" in str(e), str(e)
        assert time.time() - t0 < 5
        os._exit(0)
    os._exit(3)


def test_watchdog_reports_a_rank_that_stopped_heartbeating():
    run_ranks(_heartbeat, world=2, env={"CATCH_B200_HEARTBEAT_MS": "200", "CATCH_B200_HEARTBEAT_TIMEOUT_MS": "1500"})


# ---- FusedDataParallel over several ranks (the bucket step runs on the host under host simulation) ----------
def _fdp_net():
    torch.manual_seed(11)
    return torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.ReLU(), torch.nn.Flatten(),
                               torch.nn.Linear(8 * 6 * 6, 32), torch.nn.Tanh(), torch.nn.Linear(32, 5))


def _fdp_data(steps, world, per_rank=4):
    g = torch.Generator().manual_seed(12)
    return [(torch.randn(world * per_rank, 3, 6, 6, generator=g), torch.randint(0, 5, (world * per_rank,), generator=g))
            for _ in range(steps)]


def _fdp(rank, world, kind, grad_dtype):
    import copy

    from catch_b200.parallel import FusedDataParallel

    _init(rank, world)
    ref = _fdp_net()
    net = copy.deepcopy(ref).to(DEV)
    if rank == 1:  # the wrapper has to take rank 0's parameters
        with torch.no_grad():
            for p in net.parameters():
                p.add_(1.0)
    hp = dict(lr=0.05, momentum=0.9, weight_decay=1e-4) if kind == "sgd" else dict(lr=1e-2, weight_decay=0.01)
    fdp = FusedDataParallel(net, kind, bucket_mb=0.0005, grad_dtype=grad_dtype, **hp)
    assert len(fdp.buckets) >= 3
    opt = torch.optim.SGD(ref.parameters(), **hp) if kind == "sgd" else torch.optim.AdamW(ref.parameters(), **hp)
    data = _fdp_data(5, world)
    per = data[0][0].shape[0] // world
    loss_fn = torch.nn.CrossEntropyLoss()
    for it, (x, t) in enumerate(data[:4]):
        opt.zero_grad()
        loss_fn(ref(x), t).backward()          # the whole batch on one process
        opt.step()
        xs, ts = x[rank * per:(rank + 1) * per].to(DEV), t[rank * per:(rank + 1) * per].to(DEV)
        if it == 2:                            # gradient accumulation: two half micro-batches, the first without exchange
            h = per // 2
            with fdp.no_sync():
                (loss_fn(fdp(xs[:h]), ts[:h]) * 0.5).backward()
            (loss_fn(fdp(xs[h:]), ts[h:]) * 0.5).backward()
        else:
            loss_fn(fdp(xs), ts).backward()
        fdp.step()
    tol = 2e-5 if grad_dtype == torch.float32 else 2e-2
    for (n, p), q in zip(ref.named_parameters(), fdp.module.parameters()):
        assert (p.detach() - q.detach().cpu()).abs().max().item() < tol * max(1.0, p.abs().max().item()), (n, kind, grad_dtype)
        if fdp.lowp_dtype is not None:       # the 16-bit copies follow the masters on every rank
            assert torch.equal(q._b200_lowp.cpu(), q.detach().to(fdp.lowp_dtype).cpu()), n
    for bk in fdp.buckets:
        assert float(bk.grads.abs().max()) == 0.0
    # the sharded optimizer state gathers into the stock layout, and a stock optimizer continues from it
    sd = fdp.optimizer_state_dict()
    if grad_dtype == torch.float32:
        resumed = _fdp_net()
        resumed.load_state_dict({k: v.cpu() for k, v in fdp.module.state_dict().items()})
        opt2 = torch.optim.SGD(resumed.parameters(), **hp) if kind == "sgd" else torch.optim.AdamW(resumed.parameters(), **hp)
        opt2.load_state_dict(sd)
        x, t = data[4]
        for m, o in ((ref, opt), (resumed, opt2)):
            o.zero_grad(); loss_fn(m(x), t).backward(); o.step()
        for p, q in zip(ref.parameters(), resumed.parameters()):
            assert (p - q).abs().max().item() < 5e-5 * max(1.0, p.abs().max().item())
        # ... and loads back into a wrapper (each rank keeps its own shard)
        fdp.load_optimizer_state_dict(opt.state_dict())
    dist.barrier()
    dist.destroy_process_group()


def _fdp_sgd(rank, world):
    _fdp(rank, world, "sgd", torch.float32)


def _fdp_adamw(rank, world):
    _fdp(rank, world, "adamw", torch.float32)


def _fdp_sgd_bf16(rank, world):
    _fdp(rank, world, "sgd", torch.bfloat16)


def test_fused_data_parallel_matches_single_process():
    """Two and three ranks (an odd world size exercises the shard padding), SGD and AdamW, fp32 and 16-bit exchange."""
    run_ranks(_fdp_sgd, world=2)
    run_ranks(_fdp_adamw, world=3)
    run_ranks(_fdp_sgd_bf16, world=2)


def _fdp_unused(rank, world):
    from catch_b200.parallel import FusedDataParallel

    class Two(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(16, 16)
            self.unused = torch.nn.Linear(16, 16)
            self.b = torch.nn.Linear(16, 4)

        def forward(self, x):
            return self.b(torch.tanh(self.a(x)))

    _init(rank, world)
    torch.manual_seed(0)
    net = Two()
    before = {k: v.clone() for k, v in net.state_dict().items()}
    fdp = FusedDataParallel(net.to(DEV), "sgd", lr=0.1, bucket_mb=0.0005, lowp_dtype=None)
    order = []
    launch = fdp._launch
    fdp._launch = lambda b: (order.append(b.index), launch(b))[1]
    g = torch.Generator().manual_seed(rank)
    fdp(torch.randn(4, 16, generator=g).to(DEV)).sum().backward()
    fdp.step()
    # every rank launches every bucket, in bucket order (ranks pair launches by sequence number)
    assert order == sorted(order) and len(order) == len(fdp.buckets), order
    after = {k: v.cpu() for k, v in fdp.module.state_dict().items()}
    assert torch.equal(after["unused.weight"], before["unused.weight"])
    assert not torch.equal(after["a.weight"], before["a.weight"])
    # all ranks hold the same parameters afterwards
    flat = torch.cat([v.flatten() for v in after.values()]).to(DEV)
    both = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(both, flat)
    assert all(torch.equal(both[0].cpu(), b.cpu()) for b in both[1:])
    fdp(torch.randn(4, 16).to(DEV)).sum().backward()
    with pytest.raises(RuntimeError, match="no_sync"):
        fdp(torch.randn(4, 16).to(DEV)).sum().backward()
    dist.destroy_process_group()


def test_fused_data_parallel_unused_parameters_and_second_backward():
    run_ranks(_fdp_unused, world=2)


def _fdp_fused_convnet(rank, world):
    """The fused convolution / batch-norm modules inside FusedDataParallel: weight gradients added straight into the
    buckets, 16-bit weight copies written by the bucket step, gradient sinks.  Both ranks see the same batch, so the
    averaged gradients equal those of one process and the runs can be compared step by step."""
    import copy

    import torchvision

    from catch_b200 import fusion
    from catch_b200.fusion import StatsConv2d, fuse_bn_act
    from catch_b200.parallel import FusedDataParallel

    _init(rank, world)
    fusion.fused_ops_on_host(True)
    torch.manual_seed(21)
    base = torchvision.models.resnet.ResNet(torchvision.models.resnet.BasicBlock, [1, 1, 0, 0], num_classes=7)
    base.layer3, base.layer4 = torch.nn.Identity(), torch.nn.Identity()
    base.fc = torch.nn.Linear(128, 7)
    ref = fuse_bn_act(copy.deepcopy(base)).to(DEV).to(memory_format=torch.channels_last)
    net = fuse_bn_act(copy.deepcopy(base)).to(DEV).to(memory_format=torch.channels_last)
    hp = dict(lr=0.02, momentum=0.9, weight_decay=1e-4)
    opt = torch.optim.SGD(ref.parameters(), **hp)
    fdp = FusedDataParallel(net, "sgd", bucket_mb=0.05, **hp)
    assert len(fdp.buckets) >= 3
    convs = [m for m in net.modules() if isinstance(m, StatsConv2d)]
    assert all(m.weight._b200_lowp.dtype == torch.bfloat16 and m.weight._b200_grad_acc is not None for m in convs)
    g = torch.Generator().manual_seed(22)
    loss_fn = torch.nn.CrossEntropyLoss()
    for _ in range(3):
        x = torch.randn(4, 3, 32, 32, generator=g).to(DEV)
        t = torch.randint(0, 7, (4,), generator=g).to(DEV)
        with torch.autocast(DEV, dtype=torch.bfloat16):
            la = loss_fn(ref(x), t)
            lb = loss_fn(fdp(x), t)
        opt.zero_grad()
        la.backward(); opt.step()
        lb.backward(); fdp.step()
        assert abs(float(la.detach()) - float(lb.detach())) < 2e-2
    for (n, p), q in zip(ref.named_parameters(), fdp.module.parameters()):
        err = (p.detach().cpu() - q.detach().cpu()).norm() / (p.detach().cpu().norm() + 1e-6)
        assert err < 2e-3, (n, float(err))
    for m in convs:
        assert torch.equal(m.weight._b200_lowp.cpu(), m.weight.detach().to(torch.bfloat16).cpu())
    dist.barrier()
    dist.destroy_process_group()


def test_fused_data_parallel_with_fused_convolution_modules():
    run_ranks(_fdp_fused_convnet, world=2)


def _composed_collectives(rank, world):
    """gather / scatter / all_to_all: composed from all-gather and broadcast (equal sizes)."""
    _init(rank, world)
    for dtype in (torch.float32, torch.bfloat16, torch.int64):
        inp = (torch.arange(world * 2) + rank * 10).to(dtype).to(DEV)
        out = torch.empty_like(inp)
        dist.all_to_all_single(out, inp)
        exp = torch.cat([torch.arange(rank * 2, rank * 2 + 2) + r * 10 for r in range(world)]).to(dtype)
        assert torch.equal(out.cpu(), exp), dtype
    ins = [torch.full((2, 3), float(rank * 10 + r), device=DEV) for r in range(world)]
    outs = [torch.empty(2, 3, device=DEV) for _ in range(world)]
    w = dist.all_to_all(outs, ins, async_op=True)
    w.wait()
    assert all(torch.equal(outs[r].cpu(), torch.full((2, 3), float(r * 10 + rank))) for r in range(world))
    t = torch.full((3,), float(rank), device=DEV)
    got = [torch.empty(3, device=DEV) for _ in range(world)] if rank == 1 else None
    dist.gather(t, got, dst=1)
    if rank == 1:
        assert all(torch.equal(got[r].cpu(), torch.full((3,), float(r))) for r in range(world))
    piece = torch.empty(2, 2, device=DEV)
    src = [torch.full((2, 2), float(r + 1), device=DEV) for r in range(world)] if rank == 0 else None
    dist.scatter(piece, src, src=0)
    assert torch.equal(piece.cpu(), torch.full((2, 2), float(rank + 1)))
    # the coalescing manager (used by sharded-training libraries) wraps a group of collectives in one Work
    a, b = torch.full((3,), float(rank), device=DEV), torch.full((5,), 2.0 * rank, device=DEV)
    with dist._coalescing_manager(device=torch.device(DEV)):
        dist.all_reduce(a)
        dist.all_reduce(b)
    assert a.cpu()[0] == sum(range(world)) and b.cpu()[0] == 2 * sum(range(world))
    with dist._coalescing_manager(device=torch.device(DEV), async_ops=True) as cm:
        dist.all_reduce(a)
    cm.wait()
    with pytest.raises(Exception, match="equal splits"):
        dist.all_to_all_single(torch.empty(world, device=DEV), torch.ones(world, device=DEV), [1] * world, [1] * world)
    dist.barrier()
    dist.destroy_process_group()


def test_gather_scatter_all_to_all():
    run_ranks(_composed_collectives, world=3)


def _fsdp(rank, world):
    """Sharded data parallelism (absent from the reference): torch's FullyShardedDataParallel needs
    all_gather_into_tensor, reduce_scatter_tensor and the stream / event surface of the device module."""
    import copy

    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP

    _init(rank, world)
    dev = torch.device(DEV, torch.b200.current_device())
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    net = FSDP(copy.deepcopy(ref).to(dev), device_id=dev)
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    opt_ref = torch.optim.SGD(ref.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(1)
    for _ in range(3):
        x, y = torch.randn(8 * world, 16, generator=g), torch.randn(8 * world, 4, generator=g)
        opt_ref.zero_grad()
        torch.nn.functional.mse_loss(ref(x), y).backward()
        opt_ref.step()
        opt.zero_grad()
        torch.nn.functional.mse_loss(net(x[rank * 8:(rank + 1) * 8].to(dev)), y[rank * 8:(rank + 1) * 8].to(dev)).backward()
        opt.step()
    with FSDP.summon_full_params(net):
        for a, b in zip(ref.parameters(), net.parameters()):
            assert (a - b.cpu()).abs().max().item() < 1e-5
    dist.barrier()
    dist.destroy_process_group()


def test_fully_sharded_data_parallel_runs_on_the_backend():
    run_ranks(_fsdp, world=2)
