"""The script converter: golden output and report."""
import os

from catch_b200.tools import gpu2blackwell

SRC = '''import os
import torch
import torch.distributed as dist

def main():
    dev = torch.device("cuda:0")
    x = torch.randn(2).cuda()
    dist.init_process_group("nccl")
    use_gpu = torch.cuda.is_available()  # GPU / CUDA
'''


def test_convert_tree(tmp_path):
    d = tmp_path / "proj"
    (d / "sub").mkdir(parents=True)
    (d / "train.py").write_text(SRC)
    (d / "sub" / "data.txt").write_text("cuda stays here")
    out, report = gpu2blackwell.convert_tree(str(d))
    assert out == str(d) + "_blackwell"
    conv = open(os.path.join(out, "train.py")).read()
    assert "import torch\nimport catch_b200\n" in conv
    assert 'torch.device("blackwell:0")' in conv and ".blackwell()" in conv and '"bwccl"' in conv
    assert "use_gpu" in conv and "# GPU / CUDA" in conv  # untouched without --strict
    assert open(os.path.join(out, "sub", "data.txt")).read() == "cuda stays here"
    rep = open(report).read()
    assert "| 1 | train.py:2 | add \"import catch_b200\" |" in rep
    assert rep.count("\n| ") >= 5


def test_strict_mode(tmp_path):
    d = tmp_path / "p"
    d.mkdir()
    (d / "a.py").write_text(SRC)
    out, _ = gpu2blackwell.convert_tree(str(d), strict=True)
    conv = open(os.path.join(out, "a.py")).read()
    assert "use_blackwell" in conv and "# BLACKWELL / BLACKWELL" in conv
    assert gpu2blackwell.main(["-i", str(d), "-s"]) == 0


def test_operator_coverage_table_is_current_and_has_no_fallback_rows():
    """Every operator of the reference's device list runs on a device kernel, a composite of device kernels or a
    renamed equivalent; the committed table is what the generator prints today.  Running the generator also loads
    the library with every device kernel registered, which checks each kernel's signature against its schema."""
    import subprocess
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, CATCH_B200_CHECK_REGISTRATIONS="1", CATCH_B200_BACKEND="hostsim")
    r = subprocess.run([sys.executable, os.path.join(here, "op_coverage.py"), "--check"], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [line for line in r.stdout.splitlines() if line.startswith("| `")]
    assert len(rows) == 270
    assert not [line for line in rows if "| fallback |" in line]
    with open(os.path.join(here, "OP_COVERAGE.md")) as f:
        assert f.read().strip() == r.stdout.strip()


GPU_SCRIPT = '''import torch
import torch.nn as nn
import torch.backends.cudnn as cudnn

assert torch.cuda.is_available()
cudnn.benchmark = True
torch.cuda.set_device(0)
torch.manual_seed(0); torch.cuda.manual_seed_all(0)
device = torch.device("cuda:0")
print(torch.cuda.get_device_name(0), torch.cuda.device_count(), torch.cuda.get_device_capability())
model = nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.BatchNorm2d(8), nn.ReLU(), nn.AdaptiveAvgPool2d(1), nn.Flatten(),
                      nn.Linear(8, 4)).cuda()
opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
scaler = torch.cuda.amp.GradScaler(enabled=False)
start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
side = torch.cuda.Stream()
torch.cuda.reset_peak_memory_stats()
for step in range(2):
    x = torch.randn(4, 3, 8, 8).pin_memory().cuda(non_blocking=True)
    y = torch.randint(0, 4, (4,)).to(device, non_blocking=True)
    start.record()
    torch.cuda.nvtx.range_push("step")
    with torch.cuda.amp.autocast(dtype=torch.bfloat16):
        loss = nn.functional.cross_entropy(model(x), y)
    opt.zero_grad(set_to_none=True)
    scaler.scale(loss).backward()
    scaler.step(opt); scaler.update()
    torch.cuda.nvtx.range_pop()
    end.record()
    with torch.cuda.stream(side):
        z = x * 2
    torch.cuda.current_stream().wait_stream(side)
    z.record_stream(torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert start.elapsed_time(end) >= 0 and float(loss) == float(loss)
assert torch.cuda.max_memory_allocated() > 0 and torch.cuda.memory_reserved() >= 0
state = torch.cuda.get_rng_state(); torch.cuda.set_rng_state(state)
torch.cuda.set_per_process_memory_fraction(0.9)
torch.save(model.state_dict(), "CKPT")
sd = torch.load("CKPT", map_location="cuda:0")
assert next(iter(sd.values())).device.type != "cpu"
torch.cuda.empty_cache()
assert torch.cuda.memory_summary()
print("script finished on", next(model.parameters()).device)
'''


def test_converted_gpu_script_runs(tmp_path):
    """A training script that uses the usual torch.cuda surface (events, streams, record_stream, nvtx, amp, memory
    statistics, RNG state, checkpoints with a map_location) runs unchanged after the converter."""
    import subprocess
    import sys

    d = tmp_path / "proj"
    d.mkdir()
    (d / "train.py").write_text(GPU_SCRIPT.replace("CKPT", str(tmp_path / "model.pt")))
    out, _ = gpu2blackwell.convert_tree(str(d))
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CATCH_B200_BACKEND="hostsim", PYTHONPATH=repo)
    r = subprocess.run([sys.executable, os.path.join(out, "train.py")], env=env, capture_output=True, text=True, timeout=300,
                       cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-3000:]
    assert "script finished on blackwell:0" in r.stdout


DDP_SCRIPT = '''import os
import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel as DDP
from torch.utils.data import DataLoader, TensorDataset
from torch.utils.data.distributed import DistributedSampler

def main():
    local_rank = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    dist.init_process_group(backend="nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 4)).cuda(local_rank)
    model = DDP(model, device_ids=[local_rank], output_device=local_rank)
    ds = TensorDataset(torch.randn(64, 16), torch.randint(0, 4, (64,)))
    sampler = DistributedSampler(ds, num_replicas=world, rank=rank, shuffle=True)
    loader = DataLoader(ds, batch_size=8, sampler=sampler, pin_memory=True)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    for epoch in range(2):
        sampler.set_epoch(epoch)
        for x, y in loader:
            x, y = x.cuda(local_rank, non_blocking=True), y.cuda(local_rank, non_blocking=True)
            loss = nn.functional.cross_entropy(model(x), y)
            opt.zero_grad(); loss.backward(); opt.step()
    t = torch.tensor([float(rank)], device=f"cuda:{local_rank}")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    objs = [None] * world
    dist.all_gather_object(objs, {"rank": rank, "loss": float(loss)})
    lst = [{"cfg": 1}] if rank == 0 else [None]
    dist.broadcast_object_list(lst, src=0)
    dist.barrier()
    if rank == 0:
        torch.save(model.module.state_dict(), os.environ["OUT_CKPT"])
        print("done", t.item(), [o["rank"] for o in objs], lst[0])
    dist.destroy_process_group()

if __name__ == "__main__":
    main()
'''


def test_converted_ddp_script_runs_on_two_ranks(tmp_path):
    """A stock multi-process script (nccl backend, DistributedSampler, DDP with device_ids, tensor and object
    collectives, rank-0 checkpoint), converted and launched with torch.distributed.run on two host-simulated ranks."""
    import socket
    import subprocess
    import sys

    d = tmp_path / "proj"
    d.mkdir()
    (d / "ddp.py").write_text(DDP_SCRIPT)
    out, _ = gpu2blackwell.convert_tree(str(d))
    conv = open(os.path.join(out, "ddp.py")).read()
    assert 'backend="bwccl"' in conv and ".blackwell(local_rank" in conv
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ckpt = str(tmp_path / "model.pt")
    env = dict(os.environ, CATCH_B200_BACKEND="hostsim", PYTHONPATH=repo, OUT_CKPT=ckpt, OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(out, "ddp.py")], env=env, capture_output=True,
                       text=True, timeout=600, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-3000:]
    assert "done 1.0 [0, 1] {'cfg': 1}" in r.stdout
    import torch

    assert set(torch.load(ckpt, map_location="cpu")) == {"0.weight", "0.bias", "2.weight", "2.bias"}


def test_converter_lists_data_parallel_call_sites_as_needing_attention():
    """nn.DataParallel works for CUDA tensors only: the converter leaves the call as it is and says so in the report;
    DistributedDataParallel lines get no such note."""
    report = gpu2blackwell.Report()
    src = "import torch\nm = torch.nn.DataParallel(net.cuda())\nd = torch.nn.parallel.DistributedDataParallel(net)\n"
    out = gpu2blackwell.convert_source(src, "train.py", False, report)
    assert "torch.nn.DataParallel(net.blackwell())" in out
    notes = [e for e in report.entries if e[2].startswith("needs attention")]
    assert [(p, n) for p, n, _ in notes] == [("train.py", 2)] and "DistributedDataParallel" in notes[0][2]
