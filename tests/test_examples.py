"""The example scripts run end to end on the host-simulated device (small model, small images)."""
import os
import socket
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = ["--model", "resnet18", "--image", "64", "--batch", "2"]


def _run(args, timeout=600):
    env = dict(os.environ, CATCH_B200_BACKEND="hostsim", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable] + args, env=env, capture_output=True, text=True, timeout=timeout, cwd=REPO)
    assert r.returncode == 0, r.stderr[-3000:]
    return r.stdout


def test_single_card_training_example(tmp_path):
    ckpt = str(tmp_path / "checkpoint.pt")
    out = _run(["examples/single_card_train.py", "--iters", "2", "--checkpoint", ckpt] + SMALL)
    assert "loss" in out
    import torch

    saved = torch.load(ckpt, map_location="cpu")
    assert {"epoch", "model_state_dict", "optimizer_state_dict"} <= set(saved)


def test_eager_and_fusion_mode_inference_examples():
    assert "top-1:" in _run(["examples/eager_eval.py"] + SMALL)
    out = _run(["examples/jit_eval.py"] + SMALL)
    assert "fusion groups:" in out and "top-1:" in out


@pytest.mark.parametrize("fused", [False, True])
def test_multi_card_training_example(fused):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = _run(["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                "--master-port", str(port), "examples/multi_card_train.py", "--iters", "2"] + SMALL + (["--fused"] if fused else []))
    assert "iter 1: loss" in out


def test_bert_benchmark_script_walks_through_with_fused_layers():
    env = dict(os.environ, CATCH_B200_BACKEND="hostsim", CATCH_B200_FUSION_ON_HOSTSIM="1", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "benchmarks/bert_train.py", "--steps", "2", "--warmup", "1", "--batch", "2", "--seq", "16",
                        "--layers", "1"], env=env, capture_output=True, text=True, timeout=600, cwd=REPO)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "sequences/sec" in r.stdout and "loss" in r.stdout
