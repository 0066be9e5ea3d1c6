"""Fusion-mode (TorchScript) ResNet-50 inference (counterpart of examples/inference/jit_eval.py)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torchvision

import catch_b200  # noqa: F401
from catch_b200 import jit

ap = argparse.ArgumentParser()
ap.add_argument("--model", default="resnet50")
ap.add_argument("--batch", type=int, default=16)
ap.add_argument("--image", type=int, default=224)
args = ap.parse_args()
dev = torch.device("blackwell", 0)
# move first, then trace and freeze: freezing turns the weights into graph constants
model = getattr(torchvision.models, args.model)().eval().half().to(dev).to(memory_format=torch.channels_last)
x = torch.randn(args.batch, 3, args.image, args.image).half().to(dev).contiguous(memory_format=torch.channels_last)
with torch.no_grad():
    traced = torch.jit.trace(model, x)
    fused = jit.optimize(traced)
    out = fused(x)
print("fusion groups:", str(fused.graph).count("catch_b200::FusionGroup"), "top-1:", out.argmax(1).cpu().tolist())
print(jit.fusion_stats())
