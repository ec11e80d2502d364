"""CIFAR ResNet-20/32/44/56 (He et al. 2016, section 4.2): three stages of
``n`` basic blocks with widths 16/32/64, about 0.27 M parameters for ``n = 3``.

The reference tree has no such model (its ``models/resnet.py`` is the 4-stage,
width-64 family); ResNet-20 is the model named by the CPU/gloo correctness
configuration of the benchmarks.
"""
import torch
import torch.nn as nn

from .layers import BatchNorm2d
import torch.nn.functional as F


class _Block(nn.Module):
    def __init__(self, cin, cout, stride):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.bn1 = BatchNorm2d(cout)
        self.conv2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.bn2 = BatchNorm2d(cout)
        self.proj = None
        if stride != 1 or cin != cout:
            self.proj = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), BatchNorm2d(cout))

    def forward(self, x):
        y = self.bn1(self.conv1(x), relu=True)
        y = self.bn2(self.conv2(y))
        return F.relu(y + (x if self.proj is None else self.proj(x)))


class CifarResNet(nn.Module):
    def __init__(self, blocks_per_stage=3, num_classes=10, widths=(16, 32, 64)):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, widths[0], 3, 1, 1, bias=False), BatchNorm2d(widths[0]), nn.ReLU())
        layers, cin = [], widths[0]
        for i, w in enumerate(widths):
            for b in range(blocks_per_stage):
                layers.append(_Block(cin, w, 2 if (b == 0 and i > 0) else 1))
                cin = w
        self.stages = nn.Sequential(*layers)
        self.fc = nn.Linear(cin, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def forward(self, x):
        x = self.stages(self.stem(x))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def ResNet20(num_classes=10):
    return CifarResNet(3, num_classes)


def ResNet32(num_classes=10):
    return CifarResNet(5, num_classes)


def ResNet56(num_classes=10):
    return CifarResNet(9, num_classes)
