"""VGG-19: 16 convolutions + classifier 25088 -> 4096 -> 4096 -> 1000 (143.7 M parameters).

Each convolution is bias-free and followed by ``layers.FusedBiasReLU``, which owns the bias and
applies bias + ReLU (and the 2x2 max pooling where one follows) in one pass of this framework's
kernels; parameter count and maths are those of the usual conv(bias) -> ReLU -> pool stack.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .layers import FusedBiasReLU

CFG19 = [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"]


class VGG(nn.Module):
    def __init__(self, cfg=CFG19, num_classes: int = 1000, hidden: int = 4096, in_hw: int = 224,
                 dropout: float = 0.5):
        super().__init__()
        layers, c = [], 3
        pools = 0
        for i, v in enumerate(cfg):
            if v == "M":
                pools += 1          # folded into the preceding epilogue
                continue
            pooled = i + 1 < len(cfg) and cfg[i + 1] == "M"
            layers += [nn.Conv2d(c, v, 3, padding=1, bias=False), FusedBiasReLU(v, pool=pooled)]
            c = v
        self.features = nn.Sequential(*layers)
        side = in_hw // (2 ** pools)
        self.classifier = nn.Sequential(
            nn.Linear(c * side * side, hidden), nn.ReLU(inplace=True), nn.Dropout(dropout),
            nn.Linear(hidden, hidden), nn.ReLU(inplace=True), nn.Dropout(dropout),
            nn.Linear(hidden, num_classes))
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0, 0.01)
                nn.init.zeros_(m.bias)

    def forward(self, x):
        return self.classifier(torch.flatten(self.features(x), 1))


def vgg19(num_classes: int = 1000) -> VGG:
    return VGG(CFG19, num_classes)


def vgg_tiny(num_classes: int = 10) -> VGG:
    return VGG([8, "M", 16, "M", 16, "M"], num_classes, hidden=64, in_hw=32, dropout=0.0)
