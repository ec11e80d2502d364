"""ResNeXt-29 for CIFAR (grouped 3x3 convolutions; 2x64d, 4x64d, 8x64d, 32x4d).

Counterpart of the reference's ``examples/ImageClassification/models/resnext.py:39-86``.
"""
import torch
import torch.nn as nn

from .layers import BatchNorm2d
import torch.nn.functional as F


class _Block(nn.Module):
    expansion = 2

    def __init__(self, cin, cardinality, width, stride):
        super().__init__()
        g = cardinality * width
        cout = self.expansion * g
        self.conv1 = nn.Conv2d(cin, g, 1, bias=False)
        self.bn1 = BatchNorm2d(g)
        self.conv2 = nn.Conv2d(g, g, 3, stride, 1, groups=cardinality, bias=False)
        self.bn2 = BatchNorm2d(g)
        self.conv3 = nn.Conv2d(g, cout, 1, bias=False)
        self.bn3 = BatchNorm2d(cout)
        self.shortcut = nn.Identity()
        if stride != 1 or cin != cout:
            self.shortcut = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), BatchNorm2d(cout))

    def forward(self, x):
        y = self.bn1(self.conv1(x), relu=True)
        y = self.bn2(self.conv2(y), relu=True)
        return F.relu(self.bn3(self.conv3(y)) + self.shortcut(x))


class ResNeXt(nn.Module):
    def __init__(self, num_blocks, cardinality, bottleneck_width, num_classes=10):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 64, 1, bias=False)
        self.bn1 = BatchNorm2d(64)
        layers, cin, width = [], 64, bottleneck_width
        for stage, n in enumerate(num_blocks):
            for b in range(n):
                layers.append(_Block(cin, cardinality, width, 2 if (b == 0 and stage > 0) else 1))
                cin = _Block.expansion * cardinality * width
            width *= 2
        self.layers = nn.Sequential(*layers)
        self.linear = nn.Linear(cin, num_classes)

    def forward(self, x):
        x = self.layers(self.bn1(self.conv1(x), relu=True))
        return self.linear(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def ResNeXt29_2x64d(num_classes=10):
    return ResNeXt([3, 3, 3], 2, 64, num_classes)


def ResNeXt29_4x64d(num_classes=10):
    return ResNeXt([3, 3, 3], 4, 64, num_classes)


def ResNeXt29_8x64d(num_classes=10):
    return ResNeXt([3, 3, 3], 8, 64, num_classes)


def ResNeXt29_32x4d(num_classes=10):
    return ResNeXt([3, 3, 3], 32, 4, num_classes)
