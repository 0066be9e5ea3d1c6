"""bwccl on real GPUs (needs >= 2 B200s): collectives over peer-mapped memory,
stock DDP, the fused all-reduce + optimizer path, and the bounded device-side
wait (a rank withholds its signal; peers report a time-out and stay usable)."""
import datetime
import os

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_ranks

pytestmark = pytest.mark.gpu
DEV = "blackwell"


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


WORLD = min(int(os.environ.get("CATCH_B200_TEST_WORLD", "2")), max(_ngpu(), 1))
needs2 = pytest.mark.skipif(_ngpu() < 2, reason="needs two GPUs")
# NCCL's own NVLS stays off in these child processes.  This backend's multicast mapping is forced on (by default it
# starts at four ranks) wherever the GPUs support it, except in the test that makes a wait run out: that one runs
# on plain peer loads and stores.
ENV = {"NCCL_NVLS_ENABLE": "0", "CATCH_B200_NVLS": "1", "CATCH_B200_NVLS_FUSED": "1"}
ENV_NO_MULTICAST = {"NCCL_NVLS_ENABLE": "0", "CATCH_B200_NVLS": "0"}


def _init(rank, world):
    import catch_b200  # noqa: F401

    assert torch.b200.backend_name() == "cuda"
    torch.b200.set_device(rank)
    dist.init_process_group("bwccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))


def _collectives(rank, world):
    _init(rank, world)
    for dtype in (torch.float32, torch.bfloat16, torch.int64, torch.uint8):
        t = (torch.arange(1000) % 100 + rank).to(dtype).to(DEV)
        dist.broadcast(t, 0)
        assert torch.equal(t.cpu(), (torch.arange(1000) % 100).to(dtype)), dtype
        outs = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(outs, torch.full((1000,), rank + 1).to(dtype).to(DEV))
        for r in range(world):
            assert torch.equal(outs[r].cpu(), torch.full((1000,), r + 1).to(dtype))
    for n in (1, 7, 4096, 1 << 20, (1 << 24) + 3):
        x = torch.full((n,), float(rank + 1), device=DEV)
        dist.all_reduce(x)
        assert torch.equal(x.cpu(), torch.full((n,), float(sum(range(1, world + 1))))), n
    torch.manual_seed(5)
    xb = torch.randn(100000).bfloat16()
    dxb = (xb * (rank + 1)).to(DEV)
    dist.all_reduce(dxb)
    ref = sum((xb * (r + 1)).float() for r in range(world))
    assert (dxb.float().cpu() - ref).abs().max() <= 0.02 * ref.abs().max()
    y = torch.full((33,), float(rank + 1), device=DEV)
    dist.all_reduce(y, op=dist.ReduceOp.MAX)
    assert torch.equal(y.cpu(), torch.full((33,), float(world)))
    z = torch.full((4,), float(rank + 1), device=DEV)
    dist.reduce(z, 0)
    if rank == 0:
        assert torch.equal(z.cpu(), torch.full((4,), float(sum(range(1, world + 1)))))
    zi = torch.full((5,), (rank + 1) * world, dtype=torch.int64).to(DEV)
    dist.all_reduce(zi, op=dist.ReduceOp.AVG)
    assert torch.equal(zi.cpu(), torch.full((5,), sum(range(1, world + 1)), dtype=torch.int64))
    strided = [torch.empty(6, 2, device=DEV)[:, 0] for _ in range(world)]
    dist.all_gather(strided, torch.full((6,), float(rank), device=DEV))
    for r in range(world):
        assert torch.equal(strided[r].cpu(), torch.full((6,), float(r)))
    rs = torch.empty(3, device=DEV)
    dist.reduce_scatter_tensor(rs, torch.arange(world * 3, dtype=torch.float32, device=DEV))
    assert torch.equal(rs.cpu(), world * torch.arange(rank * 3, rank * 3 + 3).float())
    if rank == 0:
        dist.send(torch.arange(5000, dtype=torch.float32, device=DEV), 1)
    elif rank == 1:
        r = torch.zeros(5000, device=DEV)
        dist.recv(r, 0)
        assert torch.equal(r.cpu(), torch.arange(5000, dtype=torch.float32))
    dist.barrier()
    torch.b200.synchronize()
    dist.destroy_process_group()


@needs2
def test_collectives():
    run_ranks(_collectives, world=WORLD, env=ENV, timeout=240)


def _ddp(rank, world):
    _init(rank, world)
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 8))
    ref = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 8))
    ref.load_state_dict(net.state_dict())
    ddp = torch.nn.parallel.DistributedDataParallel(net.to(DEV))
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05, momentum=0.9)
    opt_ref = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    g = torch.Generator().manual_seed(1)
    for _ in range(5):
        x = torch.randn(16 * world, 64, generator=g)
        y = torch.randn(16 * world, 8, generator=g)
        opt_ref.zero_grad()
        torch.nn.functional.mse_loss(ref(x), y).backward()
        opt_ref.step()
        opt.zero_grad()
        torch.nn.functional.mse_loss(ddp(x[rank * 16:(rank + 1) * 16].to(DEV)), y[rank * 16:(rank + 1) * 16].to(DEV)).backward()
        opt.step()
    for a, b in zip(ref.parameters(), ddp.module.parameters()):
        assert (a - b.cpu()).abs().max().item() < 3e-3
    dist.destroy_process_group()


@needs2
def test_stock_ddp_matches_cpu():
    run_ranks(_ddp, world=WORLD, env=ENV, timeout=240)


def _fused(rank, world, kind, grad_dtype="fp32"):
    from catch_b200.parallel import FusedDataParallel

    gd = torch.bfloat16 if grad_dtype == "bf16" else torch.float32

    _init(rank, world)
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.Tanh(), torch.nn.Linear(256, 8))
    ref = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.Tanh(), torch.nn.Linear(256, 8))
    ref.load_state_dict(net.state_dict())
    if kind == "sgd":
        fdp = FusedDataParallel(net.to(DEV), "sgd", lr=0.05, momentum=0.9, weight_decay=1e-4, bucket_mb=0.005, grad_dtype=gd)
        opt_ref = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
    else:
        fdp = FusedDataParallel(net.to(DEV), "adamw", lr=1e-3, weight_decay=0.01, bucket_mb=0.005, grad_dtype=gd)
        opt_ref = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.01)
    assert len(fdp.buckets) > 1
    g = torch.Generator().manual_seed(1)
    for it in range(5):
        x = torch.randn(16 * world, 64, generator=g)
        y = torch.randn(16 * world, 8, generator=g)
        opt_ref.zero_grad()
        torch.nn.functional.mse_loss(ref(x), y).backward()
        opt_ref.step()
        xs, ys = x[rank * 16:(rank + 1) * 16].to(DEV), y[rank * 16:(rank + 1) * 16].to(DEV)
        if it == 2:  # the same batch as two accumulated halves
            with fdp.no_sync():
                (0.5 * torch.nn.functional.mse_loss(fdp(xs[:8]), ys[:8])).backward()
            (0.5 * torch.nn.functional.mse_loss(fdp(xs[8:]), ys[8:])).backward()
        else:
            torch.nn.functional.mse_loss(fdp(xs), ys).backward()
        fdp.step()
    torch.b200.synchronize()
    tol = 3e-3 if grad_dtype == "fp32" else 2e-2
    for a, b in zip(ref.parameters(), fdp.module.parameters()):
        assert (a - b.cpu()).abs().max().item() < tol, (a - b.cpu()).abs().max().item()
    for p in fdp.module.parameters():  # 16-bit copies written by the peers' kernels
        assert torch.equal(p._b200_lowp.cpu(), p.detach().to(torch.bfloat16).cpu())
    for bk in fdp.buckets:  # cleared by the kernel
        assert float(bk.grads.abs().max()) == 0.0
    # optimizer state gathered from the shards loads into the stock optimizer
    sd = fdp.optimizer_state_dict()
    opt_chk = type(opt_ref)(ref.parameters(), **{k: v for k, v in opt_ref.defaults.items() if k in ("lr", "momentum", "weight_decay")})
    opt_chk.load_state_dict(sd)
    key = "momentum_buffer" if kind == "sgd" else "exp_avg"
    for pr in ref.parameters():
        assert (opt_chk.state[pr][key] - opt_ref.state[pr][key]).abs().max().item() < tol
    # every rank holds bit-identical parameters
    flat = torch.cat([p.detach().reshape(-1) for p in fdp.module.parameters()])
    outs = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(outs, flat)
    assert all(torch.equal(outs[0].cpu(), o.cpu()) for o in outs)
    dist.destroy_process_group()


@needs2
@pytest.mark.parametrize("kind,grad_dtype", [("sgd", "fp32"), ("adamw", "fp32"), ("sgd", "bf16")])
def test_fused_allreduce_optimizer(kind, grad_dtype):
    run_ranks(_fused, world=WORLD, args=(kind, grad_dtype), env=ENV, timeout=240)


def _bounded_wait(rank, world):
    from catch_b200.distributed import get_backend

    _init(rank, world)
    pg = get_backend()
    t = pg.symm_empty(1024, torch.float32)
    t.fill_(1.0)
    dist.barrier()
    pg.allreduce_symm(t).wait()
    torch.b200.synchronize()
    assert torch.equal(t.cpu(), torch.full((1024,), float(world)))
    pg.set_wait_limit_ms(500)
    # rank 0 withholds its "ready" signal: every device-side wait on it must run out
    pg.allreduce_symm(t, 0, 1.0, rank == 0)
    torch.b200.synchronize()
    assert pg.status_word() & 0xFF == 1, pg.status_word()
    pg.clear_status()
    dist.barrier()  # the context and the communicator are still usable
    t.fill_(2.0)
    dist.barrier()
    pg.allreduce_symm(t).wait()
    torch.b200.synchronize()
    assert torch.equal(t.cpu(), torch.full((1024,), 2.0 * world))
    dist.destroy_process_group()


@needs2
def test_device_wait_is_bounded():
    run_ranks(_bounded_wait, world=WORLD, env=ENV_NO_MULTICAST, timeout=240)


def _multicast(rank, world, expect_on):
    from catch_b200.distributed import get_backend

    _init(rank, world)
    pg = get_backend()
    on = pg.multicast_enabled()
    if not expect_on:
        assert not on
    # sums and averages of every floating type through whichever path the arena has, below and above the
    # size at which the in-switch kernels take over
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 2e-2), (torch.float16, 2e-3)):
        for n in (1000, 70001, (1 << 20) + 8, 3 << 20):
            torch.manual_seed(n)
            base = torch.randn(n)
            t = pg.symm_empty(n, dtype)
            t.copy_((base * (rank + 1)).to(dtype))
            dist.barrier()
            pg.allreduce_symm(t, 0, 0.5).wait()
            torch.b200.synchronize()
            ref = sum((base * (r + 1)).to(dtype).float() for r in range(world)) * 0.5
            err = (t.float().cpu() - ref).abs().max().item()
            assert err <= tol * max(1.0, ref.abs().max().item()), (dtype, n, err, on)
    dist.barrier()
    torch.b200.synchronize()
    if rank == 0:
        print(f"multicast mapping in use: {on}")
    dist.destroy_process_group()


@needs2
@pytest.mark.parametrize("multicast", [True, False])
def test_allreduce_with_and_without_multicast(multicast):
    run_ranks(_multicast, world=WORLD, args=(multicast,), env=ENV if multicast else ENV_NO_MULTICAST, timeout=240)


def _composed(rank, world):
    """gather / scatter / all_to_all, which this backend composes from all-gather and broadcast."""
    _init(rank, world)
    for dtype in (torch.float32, torch.bfloat16, torch.int64):
        inp = (torch.arange(world * 1000) % 50 + rank * 3).to(dtype).to(DEV)
        out = torch.empty_like(inp)
        dist.all_to_all_single(out, inp)
        exp = torch.cat([(torch.arange(rank * 1000, (rank + 1) * 1000) % 50 + r * 3) for r in range(world)]).to(dtype)
        assert torch.equal(out.cpu(), exp), dtype
    ins = [torch.full((5, 7), float(rank * 10 + r), device=DEV) for r in range(world)]
    outs = [torch.empty(5, 7, device=DEV) for _ in range(world)]
    dist.all_to_all(outs, ins)
    assert all(torch.equal(outs[r].cpu(), torch.full((5, 7), float(r * 10 + rank))) for r in range(world))
    t = torch.full((333,), float(rank), device=DEV)
    got = [torch.empty(333, device=DEV) for _ in range(world)] if rank == world - 1 else None
    dist.gather(t, got, dst=world - 1)
    if rank == world - 1:
        assert all(torch.equal(got[r].cpu(), torch.full((333,), float(r))) for r in range(world))
    piece = torch.empty(9, 9, device=DEV)
    src = [torch.full((9, 9), float(r + 1), device=DEV) for r in range(world)] if rank == 0 else None
    dist.scatter(piece, src, src=0)
    assert torch.equal(piece.cpu(), torch.full((9, 9), float(rank + 1)))
    dist.barrier()
    torch.b200.synchronize()
    dist.destroy_process_group()


@needs2
def test_gather_scatter_all_to_all():
    run_ranks(_composed, world=WORLD, env=ENV, timeout=240)
