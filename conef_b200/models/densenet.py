"""DenseNet-BC for CIFAR (121/169/201/161 layouts and a small growth-12 variant).

Counterpart of the reference's ``examples/ImageClassification/models/densenet.py:35-103``.
"""
import math

import torch
import torch.nn as nn

from .layers import BatchNorm2d
import torch.nn.functional as F


class _DenseLayer(nn.Module):
    def __init__(self, cin, growth):
        super().__init__()
        self.bn1 = BatchNorm2d(cin)
        self.conv1 = nn.Conv2d(cin, 4 * growth, 1, bias=False)
        self.bn2 = BatchNorm2d(4 * growth)
        self.conv2 = nn.Conv2d(4 * growth, growth, 3, padding=1, bias=False)

    def forward(self, x):
        y = self.conv1(self.bn1(x, relu=True))
        y = self.conv2(self.bn2(y, relu=True))
        return torch.cat([y, x], 1)


class _Transition(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.bn = BatchNorm2d(cin)
        self.conv = nn.Conv2d(cin, cout, 1, bias=False)

    def forward(self, x):
        return F.avg_pool2d(self.conv(self.bn(x, relu=True)), 2)


class DenseNet(nn.Module):
    def __init__(self, nblocks, growth_rate=12, reduction=0.5, num_classes=10):
        super().__init__()
        planes = 2 * growth_rate
        self.conv1 = nn.Conv2d(3, planes, 3, padding=1, bias=False)
        stages = []
        for i, n in enumerate(nblocks):
            for _ in range(n):
                stages.append(_DenseLayer(planes, growth_rate))
                planes += growth_rate
            if i + 1 < len(nblocks):
                out = int(math.floor(planes * reduction))
                stages.append(_Transition(planes, out))
                planes = out
        self.features = nn.Sequential(*stages)
        self.bn = BatchNorm2d(planes)
        self.linear = nn.Linear(planes, num_classes)

    def forward(self, x):
        x = self.features(self.conv1(x))
        x = F.avg_pool2d(self.bn(x, relu=True), 4)
        return self.linear(torch.flatten(x, 1))


def DenseNet121(num_classes=10):
    return DenseNet([6, 12, 24, 16], 32, num_classes=num_classes)


def DenseNet169(num_classes=10):
    return DenseNet([6, 12, 32, 32], 32, num_classes=num_classes)


def DenseNet201(num_classes=10):
    return DenseNet([6, 12, 48, 32], 32, num_classes=num_classes)


def DenseNet161(num_classes=10):
    return DenseNet([6, 12, 36, 24], 48, num_classes=num_classes)


def densenet_cifar(num_classes=10):
    return DenseNet([6, 12, 24, 16], 12, num_classes=num_classes)
