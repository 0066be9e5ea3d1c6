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
