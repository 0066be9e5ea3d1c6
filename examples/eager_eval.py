"""Eager-mode ResNet-50 inference (counterpart of examples/inference/eager_eval.py)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torchvision

import catch_b200  # noqa: F401

dev = torch.device("blackwell", 0)
model = torchvision.models.resnet50().eval().half().to(dev).to(memory_format=torch.channels_last)
x = torch.randn(16, 3, 224, 224).half().to(dev)
with torch.no_grad():
    out = model(x)
print("top-1:", out.argmax(1).cpu().tolist())
