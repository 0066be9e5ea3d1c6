"""bench.py as a script: the JSON line it has to print (keys, types, whole-job aggregates), walked on the
host-simulated device with a small model (the numbers mean nothing there), on one process and on two ranks, and the
reference arm's "unavailable" line."""
import json
import os
import socket
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = ["--model", "resnet18", "--batch", "2", "--steps", "2", "--warmup", "3", "--no-stock"]
KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
        "dtype", "data", "config", "clocks", "e2e", "gpu_launches"}


def _run(args, timeout=900):
    env = dict(os.environ, CATCH_B200_BACKEND="hostsim", CATCH_B200_BENCH_DRY_RUN="1", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable] + args, env=env, capture_output=True, text=True, timeout=timeout, cwd=REPO)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout          # ONE JSON line, from rank 0
    return json.loads(lines[0])


def _check(d, world):
    assert KEYS <= set(d), KEYS - set(d)
    assert d["n_gpus"] == world and d["steps"] == 2 and d["warmup"] == 3
    assert d["higher_is_better"] is True and d["scaling"] == "weak" and d["dtype"] == "bf16" and "synthetic" in d["data"]
    assert d["config"]["global_batch"] == 2 * world and d["config"]["parallelism"] == f"dp{world}"
    # the value is the whole job's rate: global batch over the step time
    assert abs(d["value"] - 2 * world / (d["ms_per_step"] / 1e3)) <= 0.06 * d["value"] + 0.1
    e = d["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] == 2 * 3 * 224 * 224 * 4 + 2 * 8 and e["d2h_bytes_per_step"] == 4
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
    assert d["kernel_error_flag"] == 0 and d["final_loss"] == d["final_loss"]


def test_single_process_line():
    _check(_run(["bench.py"] + SMALL), 1)


def test_two_rank_line():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    d = _run(["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port",
              str(port), "bench.py", "--gpus", "2"] + SMALL)
    _check(d, 2)
    assert d["params_identical_across_ranks"] is True


def test_reference_arm_says_why_it_cannot_run():
    env = dict(os.environ, CATCH_B200_BACKEND="hostsim")
    r = subprocess.run([sys.executable, "bench.py", "--impl", "reference"], env=env, capture_output=True, text=True, timeout=300,
                       cwd=REPO)
    assert r.returncode == 0
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and d["unavailable"]
