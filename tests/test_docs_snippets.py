"""The code shown in docs/training.md, docs/inference.md and docs/debugging.md, run as written (small model, host-simulated
device): a guide that does not execute is worse than none."""
import torch
import torchvision

import catch_b200  # noqa: F401
from catch_b200 import jit
from catch_b200.fusion import fuse_bn_act
from catch_b200.optim import FusedSGD
from catch_b200.utils import DelayedScalar, PrefetchLoader


def test_guide_snippets_execute(tmp_path):
    CKPT = str(tmp_path / "model.pt")
    # docs/training.md, single GPU
    model = fuse_bn_act(torchvision.models.resnet18(num_classes=10)).to("blackwell").to(memory_format=torch.channels_last)
    opt = FusedSGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    data = [(torch.randn(2, 3, 64, 64), torch.randint(0, 10, (2,))) for _ in range(3)]
    last = DelayedScalar()
    for x, t in PrefetchLoader(data, device="blackwell"):
        with torch.autocast("blackwell", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(model(x), t)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        print("loss one step late:", last.push(loss))
    print("last:", last.flush())

    # docs/inference.md, fusion mode + save/load
    m = torchvision.models.resnet18(num_classes=10).eval().half().to("blackwell").to(memory_format=torch.channels_last)
    example = torch.randn(2, 3, 64, 64).half().to("blackwell").contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        fused = jit.optimize(torch.jit.trace(m, example))
        y = fused(example)
        jit.save(fused, CKPT); fused2 = jit.load(CKPT, map_location="blackwell")
        assert torch.allclose(fused2(example).float().cpu(), y.float().cpu(), atol=1e-2)
    fast = torch.b200.make_graphed_callable(m, (example,))
    with torch.no_grad():
        fast(example)

    # docs/inference.md, int8
    from catch_b200.quantize import quantize_dynamic
    fp = torchvision.models.resnet18(num_classes=10).eval()
    calib = quantize_dynamic(fp, {"per_channel": True, "iteration": 2}, dtype="int8", gen_quant=True, mixed_layer={"conv1": "float"})
    for _ in range(2): calib(torch.randn(2, 3, 64, 64))
    q = quantize_dynamic(fp, mixed_layer={"conv1": "float"})
    q.load_state_dict(calib.state_dict(), strict=False)
    q = q.half().to("blackwell").to(memory_format=torch.channels_last)
    with torch.no_grad():
        fq = jit.optimize(torch.jit.trace(q, example))
        print("int8 out", fq(example).shape)
    # docs/debugging.md
    from catch_b200 import profiler, dumptool
    with profiler.kernel_trace() as tr:
        torch.relu(example)
    with profiler.profile(kernels=True) as prof:
        torch.relu(example)
    print(prof.table()[:60].splitlines()[0])
    print(torch.b200.memory_summary()[:30].splitlines()[0])
    print("snippets ok")
