#!/usr/bin/env python
"""The whole stack on a toy problem, after the reference's ``train_mnist`` example: a 3-layer MLP
(784 -> 128 -> 64 -> 10) trained with Adam on synthetic MNIST from this package's own dataset
reader, batched and shuffled by the data loader, driven by ``Learner.fit`` with an accuracy metric.
The synthetic digits are class-dependent patterns plus noise, so the accuracy must climb well
above chance within a few epochs.

    python examples/train_mnist_synthetic.py [--epochs 3] [--samples 1000]
"""
import argparse
import os
import sys

import torch
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200 import vision  # noqa: E402
from ferrotorch_b200.train.learner import AccuracyMetric, Learner, LossMetric  # noqa: E402
from ferrotorch_b200.vision import own_transforms as T  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", type=int, default=3)
    ap.add_argument("--samples", type=int, default=1000)
    ap.add_argument("--batch-size", type=int, default=32)
    a = ap.parse_args()
    torch.manual_seed(0)
    vision.vision_manual_seed(0)
    augment = T.Compose([T.RandomCrop(28, padding=2), vision.VisionNormalize([0.5], [0.5])])
    train = vision.Mnist.synthetic(vision.Split.Train, a.samples, transform=augment)
    test = vision.Mnist.synthetic(vision.Split.Test, a.samples // 4, transform=vision.VisionNormalize([0.5], [0.5]))
    loader = torch.utils.data.DataLoader(train, batch_size=a.batch_size, shuffle=True, generator=torch.Generator().manual_seed(42))
    val = torch.utils.data.DataLoader(test, batch_size=128)
    model = nn.Sequential(nn.Flatten(), nn.Linear(784, 128), nn.ReLU(), nn.Linear(128, 64), nn.ReLU(), nn.Linear(64, 10))
    print("model: 3-layer MLP, %d parameters; %d training samples, %d batches per epoch"
          % (sum(p.numel() for p in model.parameters()), len(train), len(loader)))
    learner = Learner(model, torch.optim.Adam(model.parameters(), lr=1e-3), nn.CrossEntropyLoss(),
                      metrics=[LossMetric(), AccuracyMetric()])
    history = learner.fit(loader, val, epochs=a.epochs)
    for e in history.epochs:
        print("epoch %d: train %s | validation %s" % (e.epoch, {k: round(v, 4) for k, v in e.train.items()},
                                                     {k: round(v, 4) for k, v in (e.val or {}).items()}))
    acc = [v for k, v in (history.epochs[-1].val or {}).items() if "acc" in k.lower() or "top" in k.lower()]
    assert acc and acc[0] > 0.5, "validation accuracy %s did not rise above chance" % acc
    print("final validation accuracy %.3f" % acc[0])


if __name__ == "__main__":
    main()
