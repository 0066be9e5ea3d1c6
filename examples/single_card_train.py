"""Train ResNet-50 on synthetic data on one blackwell device (counterpart of the
reference's examples/training/single_card_demo.py)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torchvision

import catch_b200  # noqa: F401
from catch_b200.optim import FusedSGD
from catch_b200.utils import PrefetchLoader


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--image", type=int, default=224)
    ap.add_argument("--checkpoint", default="checkpoint.pt", help="where the final checkpoint goes ('' = do not write one)")
    args = ap.parse_args()
    dev = torch.device("blackwell", 0)
    model = getattr(torchvision.models, args.model)().to(dev).to(memory_format=torch.channels_last)
    opt = FusedSGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    data = torchvision.datasets.FakeData(args.batch * args.iters, (3, args.image, args.image), 1000, torchvision.transforms.ToTensor())
    loader = PrefetchLoader(torch.utils.data.DataLoader(data, batch_size=args.batch), dev)
    model.train()
    for i, (x, y) in enumerate(loader):
        with torch.autocast(device_type="blackwell", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(model(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        print(f"iter {i}: loss {loss.item():.4f}")
    if args.checkpoint:
        torch.save({"epoch": 0, "model_state_dict": model.state_dict(), "optimizer_state_dict": opt.state_dict()}, args.checkpoint)


if __name__ == "__main__":
    main()
