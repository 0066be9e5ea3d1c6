"""Dump tool, profiler, prefetch loader and fusion passes on the host-simulated device."""
import os

import torch

import catch_b200  # noqa: F401
from catch_b200 import dumptool, jit, profiler
from catch_b200.utils import PrefetchLoader

DEV = "blackwell"


def test_dump_tool_files(tmp_path):
    x = torch.arange(12.0).reshape(3, 4).to(DEV)
    d = str(tmp_path / "dump")
    with dumptool.Dumper(d, enable=True, use_cpu=True, level=2):
        y = torch.relu(x - 5.0)
    ops = sorted(os.listdir(d))
    assert any(o.endswith("aten__sub") or "sub" in o for o in ops) and any("relu" in o for o in ops)
    relu_dir = os.path.join(d, [o for o in ops if "relu" in o][0])
    files = sorted(os.listdir(relu_dir))
    assert "dev_0" in files and "dev_result_0" in files and "cpu_result_0" in files
    head, *vals = open(os.path.join(relu_dir, "dev_result_0")).read().splitlines()
    assert head == "Tensor : Type = Float : Shape = [3, 4] : Stride = [4, 1] : Dumped = 12"
    assert [float(v) for v in vals] == torch.relu(torch.arange(12.0) - 5).tolist()
    errs, ok = dumptool.compare_dump(relu_dir)
    assert ok and errs
    # level 0: first ten values; a second dump goes to "<dir>1"
    with dumptool.Dumper(d, level=0):
        torch.relu(x)
    assert os.path.isdir(d + "1")
    sub = os.path.join(d + "1", os.listdir(d + "1")[0])
    assert open(os.path.join(sub, "dev_0")).read().splitlines()[0].endswith("Dumped = 10")
    assert y.device.type == DEV


def test_profiler_reports_device_time():
    x = torch.randn(64, 64, device=DEV)
    with profiler.profile(record_shapes=True, profile_memory=True) as prof:
        y = (x @ x).relu().sum()
    assert y.device.type == DEV
    names = {e.name for e in prof.function_events}
    assert "aten::mm" in names and "aten::relu" in names
    table = prof.key_averages().table(sort_by="self_cpu_time_total")
    assert "aten::mm" in table
    with profiler.timed_region() as t:
        _ = x + 1
    assert t.ms >= 0.0


def test_prefetch_loader_matches_plain():
    data = [(torch.full((4, 3), float(i)), torch.tensor([i] * 4)) for i in range(5)]
    for use_q in (True, False):
        got = list(PrefetchLoader(data, DEV, use_io_queue=use_q))
        assert len(got) == 5
        for i, (a, b) in enumerate(got):
            assert a.device.type == DEV and torch.equal(a.cpu(), data[i][0]) and torch.equal(b.cpu(), data[i][1])


class Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1 = torch.nn.Conv2d(8, 16, 3, padding=1, bias=False)
        self.bn1 = torch.nn.BatchNorm2d(16)
        self.conv2 = torch.nn.Conv2d(16, 16, 3, padding=1, bias=False)
        self.bn2 = torch.nn.BatchNorm2d(16)
        self.skip = torch.nn.Conv2d(8, 16, 1, bias=False)
        self.drop = torch.nn.Dropout(0.5)
        self.fc = torch.nn.Linear(16, 10)

    def forward(self, x):
        y = torch.relu(self.bn1(self.conv1(x)))
        y = self.bn2(self.conv2(y))
        y = torch.relu(y + self.skip(x))
        y = self.drop(y.mean((2, 3)))
        return torch.relu(self.fc(y))


def test_fusion_passes_rewrite_and_segment():
    torch.manual_seed(0)
    m = Block().eval()
    for bn in (m.bn1, m.bn2):
        bn.running_mean.normal_(); bn.running_var.uniform_(0.5, 2.0)
    x = torch.randn(2, 8, 12, 12)
    ref = m(x)
    sm = torch.jit.script(m)
    opt = jit.optimize(sm)
    g = str(opt.graph)
    assert "catch_b200::FusionGroup" in g
    assert "aten::batch_norm" not in g and "aten::dropout" not in g
    inner = "".join(str(n.g("Subgraph")) for n in opt.graph.nodes() if n.kind() == "catch_b200::FusionGroup")
    assert inner.count("catch_b200::conv_bn_act") == 3 and "catch_b200::linear_act" in inner
    assert "aten::conv2d" not in inner and "aten::relu" not in inner.replace("relu_", "")
    out = opt(x)
    assert torch.allclose(out, ref, atol=1e-4), (out - ref).abs().max()
    before = jit.fusion_stats()
    opt(x); opt(torch.randn(3, 8, 12, 12))
    after = jit.fusion_stats()
    assert after["compiles"] >= before["compiles"] + 1  # a new shape compiles a new plan


def test_fusion_of_traced_module_rewrites_underscore_convolution():
    # torch.jit.trace records aten::_convolution; lowering has to turn it into the form the
    # conv+add+relu patterns match, otherwise every relu / add stays a separate kernel.
    torch.manual_seed(0)
    m = Block().eval()
    x = torch.randn(2, 8, 12, 12)
    ref = m(x)
    opt = jit.optimize(torch.jit.trace(m, x))
    inner = "".join(str(n.g("Subgraph")) for n in opt.graph.nodes() if n.kind() == "catch_b200::FusionGroup")
    assert inner.count("catch_b200::conv_bn_act") == 3
    assert "aten::_convolution" not in inner and "aten::relu(" not in inner and "aten::add(" not in inner
    assert torch.allclose(opt(x), ref, atol=1e-4)


def test_torchscript_save_load_roundtrip_and_unfuse(tmp_path):
    """Reference test strategy: test/torch_native_ci/jit/test_save_load.py -- scripted modules round-trip through
    files, to and from the device; an optimised module is saved without its fusion groups and gets them back."""
    import io

    torch.manual_seed(0)
    m = Block().eval()
    x = torch.randn(2, 8, 12, 12)
    ref = m(x)
    # plain scripted module: host file -> device, device file -> host / device
    buf = io.BytesIO(); torch.jit.save(torch.jit.script(m), buf); buf.seek(0)
    dm = torch.jit.load(buf, map_location="blackwell")
    assert next(dm.parameters()).device.type == "blackwell"
    assert torch.allclose(dm(x.to("blackwell")).cpu(), ref, atol=1e-4)
    path = tmp_path / "on_device.pt"
    torch.jit.save(torch.jit.script(Block().eval()).to("blackwell"), str(path))
    assert next(torch.jit.load(str(path), map_location="cpu").parameters()).device.type == "cpu"
    assert next(torch.jit.load(str(path)).parameters()).device.type == "blackwell"
    # optimised module: groups are dissolved for the file and rebuilt on both sides
    opt = jit.optimize(torch.jit.script(m))
    n_groups = str(opt.graph).count("catch_b200::FusionGroup")
    assert n_groups >= 1
    path2 = tmp_path / "optimised.pt"
    jit.save(opt, str(path2))
    assert str(opt.graph).count("catch_b200::FusionGroup") == n_groups
    back = jit.load(str(path2), map_location="blackwell")
    g = str(back.graph)
    assert "catch_b200::FusionGroup" in g
    inner = "".join(str(n.g("Subgraph")) for n in back.graph.nodes() if n.kind() == "catch_b200::FusionGroup")
    assert inner.count("catch_b200::conv_bn_act") == 3
    assert torch.allclose(back(x.to("blackwell")).cpu(), ref, atol=1e-4)
    jit.unfuse_graph(back.graph)
    assert "FusionGroup" not in str(back.graph) and str(back.graph).count("catch_b200::conv_bn_act") == 3
    assert torch.allclose(back(x.to("blackwell")).cpu(), ref, atol=1e-4)


def test_fusion_toggle_and_forced_fallback():
    m = torch.jit.script(Block().eval())
    jit.set_fusion_enabled(False)
    try:
        assert not jit.fusion_enabled() and not torch.b200._jit_can_fuse_on_b200()
        g = str(jit.optimize(m).graph)
        assert "FusionGroup" not in g
    finally:
        torch.b200._jit_override_can_fuse_on_b200(True)
    assert jit.fusion_enabled()


def test_lowering_removes_exception_ifs_and_dropout():
    @torch.jit.script
    def f(x):
        if x.dim() != 2:
            raise RuntimeError("bad rank")
        y = torch.nn.functional.dropout(x, 0.5, False)
        return (y.contiguous() + 1).mean()

    g = f.graph
    jit.lower_graph(g)
    s = str(g)
    assert "prim::RaiseException" not in s and "aten::dropout" not in s and "aten::contiguous" not in s

    # contiguous() stays where something downstream depends on strides: in front of a view, or as a graph output
    @torch.jit.script
    def shuffle(x):
        b, c, h, w = x.shape
        y = x.view(b, 2, c // 2, h, w).transpose(1, 2).contiguous()
        return y.view(b, c, h, w)

    g = shuffle.graph
    jit.lower_graph(g)
    assert str(g).count("aten::contiguous") == 1
    x = torch.randn(2, 8, 3, 3).to("blackwell")
    ref = x.cpu().view(2, 2, 4, 3, 3).transpose(1, 2).contiguous().view(2, 8, 3, 3)
    assert torch.equal(shuffle(x).cpu(), ref)


def test_delayed_scalar_returns_each_value_one_push_later():
    from catch_b200.utils import DelayedScalar

    r = DelayedScalar()
    vals = [torch.tensor(float(i) + 0.5).to("blackwell") for i in range(5)]
    got = [r.push(v) for v in vals]
    assert got[0] is None and got[1:] == [0.5, 1.5, 2.5, 3.5]
    assert r.flush() == 4.5 and r.flush() is None
    assert r.push(torch.tensor([2.0]).to("blackwell").bfloat16().sum()) is None and r.flush() == 2.0


def test_kernel_case_generator_and_replay(tmp_path, capfd):
    """Same flow as the reference's test/cnnl/test_dumptool.py:147-175: levels L1 / L2 write case files, L3 prints,
    anything else raises; on top of that a written case can be replayed."""
    import json

    import pytest

    a, b = torch.randn(2, 2, 6, 6), torch.randn(2, 2, 6, 6)
    for level in ("L1", "L2"):
        d = str(tmp_path / f"gen_case_{level}")
        assert dumptool.dump_gencase(True, level, d) is True
        (a.to(DEV) + b.to(DEV)).view(4, 36)
        torch.nn.functional.conv2d(a.to(DEV).contiguous(memory_format=torch.channels_last), torch.randn(4, 2, 3, 3).to(DEV),
                                   padding=1)
        assert dumptool.dump_gencase(False) is False
        assert os.path.isdir(d)
        add_dir = os.path.join(d, "aten__add.Tensor")
        cases = sorted(f for f in os.listdir(add_dir) if f.endswith(".json"))
        assert cases
        case = json.load(open(os.path.join(add_dir, cases[0])))
        assert case["op"] == "aten::add.Tensor" and case["schema"].startswith("aten::add.Tensor(Tensor self")
        assert case["args"][0]["shape"] == [2, 2, 6, 6] and case["args"][0]["dtype"] == "Float"
        assert case["args"][2]["name"] == "alpha" and case["args"][2]["value"] == 1
        assert ("data" in case["args"][0]) == (level == "L2")
        dev, cpu, errs = dumptool.replay_case(os.path.join(add_dir, cases[0]))
        assert dev[0].device.type == DEV and errs[0] < 1e-6
        if level == "L2":  # the recorded bytes are the operands
            assert torch.equal(cpu[0], a + b)
        conv_dirs = [x for x in os.listdir(d) if "conv" in x]
        assert conv_dirs
        cdir = os.path.join(d, sorted(conv_dirs)[0])
        ccase = json.load(open(os.path.join(cdir, sorted(f for f in os.listdir(cdir) if f.endswith(".json"))[0])))
        assert ccase["args"][0]["format"] == "channels_last"
    # nothing is written once the generator is off
    n = sum(len(fs) for _, _, fs in os.walk(str(tmp_path)))
    a.to(DEV) + b.to(DEV)
    assert sum(len(fs) for _, _, fs in os.walk(str(tmp_path))) == n
    capfd.readouterr()
    assert dumptool.dump_gencase(True, "L3", str(tmp_path / "none"))
    a.to(DEV) + b.to(DEV)
    dumptool.dump_gencase(False)
    assert "[gen_case]" in capfd.readouterr().err and not os.path.exists(str(tmp_path / "none"))
    for level in ("L0", "l1", "L4"):
        with pytest.raises(ValueError):
            dumptool.dump_gencase(True, level)


_MIXED_DEVICE_SCRIPT = r'''
import torch, catch_b200
F = torch.nn.functional
D = "blackwell"
w = torch.empty(3, 4, device=D)
cases = {
    "mm": lambda: torch.empty(2, 3) @ w,
    "addmm": lambda: torch.addmm(torch.empty(4), torch.empty(2, 3, device=D), w),
    "bmm": lambda: torch.bmm(torch.empty(1, 2, 3, device=D), torch.empty(1, 3, 4)),
    "conv weight": lambda: F.conv2d(torch.empty(1, 3, 8, 8, device=D), torch.empty(4, 3, 3, 3)),
    "embedding": lambda: F.embedding(torch.tensor([1]), w),
    "index_select": lambda: w.index_select(0, torch.tensor([1])),
    "gather": lambda: w.gather(0, torch.zeros(1, 4, dtype=torch.long)),
    "scatter": lambda: w.scatter(0, torch.zeros(1, 4, dtype=torch.long), 1.0),
    "scatter_add": lambda: w.scatter_add(0, torch.zeros(1, 4, dtype=torch.long, device=D), torch.ones(1, 4)),
    "masked_select": lambda: w.masked_select(torch.ones(3, 4, dtype=torch.bool)),
    "nll_loss": lambda: F.nll_loss(w, torch.tensor([1, 2, 3])),
    "layer_norm": lambda: F.layer_norm(w, (4,), torch.ones(4)),
    "other device": lambda: w.t() @ torch.empty(3, 2, device="blackwell:1"),
    "linear_act": lambda: torch.ops.catch_b200.linear_act(torch.empty(2, 4), w, None, 0),
    "softmax_cross_entropy": lambda: torch.ops.catch_b200.softmax_cross_entropy(w, torch.tensor([1, 2, 3]), -100, 0.0),
}
bad = []
for name, fn in cases.items():
    try:
        fn()
        bad.append(name + ": no error")
    except RuntimeError as e:
        if "Expected all tensors to be on the same device" not in str(e):
            bad.append(name + ": " + str(e)[:100])
print("BAD", bad)
'''


def test_kernels_that_take_raw_pointers_refuse_arguments_on_another_device():
    """The matrix-product, convolution, normalisation, look-up and loss kernels receive raw pointers: an argument on
    the host or on another device must raise (in the stock backends' words) before a kernel could read it.  The
    kernels are registered without a GPU by the registration-check switch; the check runs in front of the launch."""
    import os
    import subprocess
    import sys

    env = dict(os.environ, CATCH_B200_BACKEND="hostsim", CATCH_B200_CHECK_REGISTRATIONS="1")
    r = subprocess.run([sys.executable, "-c", _MIXED_DEVICE_SCRIPT], env=env, capture_output=True, text=True, timeout=600,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stderr[-2000:]
    assert "BAD []" in r.stdout, r.stdout[-2000:]
    # batch normalisation is registered on the host-simulated device as it is: checked in this process
    import pytest
    import torch

    import catch_b200  # noqa: F401

    with pytest.raises(RuntimeError, match="same device"):
        torch.nn.BatchNorm2d(4).to("blackwell")(torch.empty(2, 4, 3, 3))
