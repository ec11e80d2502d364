"""CIFAR variants of ResNet-18/34/50/101/152 (3x3 stem, four stages of width 64..512).

Same family as the reference's ``examples/ImageClassification/models/resnet.py:98-115``.
"""
import torch
import torch.nn as nn

from .layers import BatchNorm2d
import torch.nn.functional as F


def _shortcut(cin, cout, stride):
    if stride == 1 and cin == cout:
        return nn.Identity()
    return nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), BatchNorm2d(cout))


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, cin, planes, stride=1):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, planes, 3, stride, 1, bias=False)
        self.bn1 = BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, 1, 1, bias=False)
        self.bn2 = BatchNorm2d(planes)
        self.shortcut = _shortcut(cin, planes, stride)

    def forward(self, x):
        y = self.bn1(self.conv1(x), relu=True)
        return F.relu(self.bn2(self.conv2(y)) + self.shortcut(x))


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin, planes, stride=1):
        super().__init__()
        cout = planes * self.expansion
        self.conv1 = nn.Conv2d(cin, planes, 1, bias=False)
        self.bn1 = BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, stride, 1, bias=False)
        self.bn2 = BatchNorm2d(planes)
        self.conv3 = nn.Conv2d(planes, cout, 1, bias=False)
        self.bn3 = BatchNorm2d(cout)
        self.shortcut = _shortcut(cin, cout, stride)

    def forward(self, x):
        y = self.bn1(self.conv1(x), relu=True)
        y = self.bn2(self.conv2(y), relu=True)
        return F.relu(self.bn3(self.conv3(y)) + self.shortcut(x))


class ResNet(nn.Module):
    def __init__(self, block, num_blocks, num_classes=10):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 64, 3, 1, 1, bias=False)
        self.bn1 = BatchNorm2d(64)
        layers, cin = [], 64
        for stage, (planes, n) in enumerate(zip((64, 128, 256, 512), num_blocks)):
            for b in range(n):
                layers.append(block(cin, planes, 2 if (b == 0 and stage > 0) else 1))
                cin = planes * block.expansion
        self.layers = nn.Sequential(*layers)
        self.linear = nn.Linear(cin, num_classes)

    def forward(self, x):
        x = self.layers(self.bn1(self.conv1(x), relu=True))
        return self.linear(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def ResNet18(num_classes=10):
    return ResNet(BasicBlock, [2, 2, 2, 2], num_classes)


def ResNet34(num_classes=10):
    return ResNet(BasicBlock, [3, 4, 6, 3], num_classes)


def ResNet50(num_classes=10):
    return ResNet(Bottleneck, [3, 4, 6, 3], num_classes)


def ResNet101(num_classes=10):
    return ResNet(Bottleneck, [3, 4, 23, 3], num_classes)


def ResNet152(num_classes=10):
    return ResNet(Bottleneck, [3, 8, 36, 3], num_classes)
