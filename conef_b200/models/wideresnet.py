"""Wide ResNet for CIFAR (Zagoruyko & Komodakis 2016): pre-activation basic
blocks, ``depth = 6n + 4``, widths ``16k / 32k / 64k``.

Same architecture as the reference's ``examples/ImageClassification/models/
wideresnet.py:44-83`` (conv biases included, dropout between the two convs of
a block, BatchNorm momentum 0.9) so that parameter shapes — and therefore the
compression plan — match: WRN-28-10 with 100 classes has 36,546,980 parameters.
The class count is an argument here; the reference's ``WideResNet40_10``
factory hard-codes 28-10 with 10 classes (``wideresnet.py:86-87``).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import BatchNorm2d, Conv2d


class WideBlock(nn.Module):
    def __init__(self, cin, cout, dropout, stride):
        super().__init__()
        self.bn1 = BatchNorm2d(cin, momentum=0.9)
        self.conv1 = Conv2d(cin, cout, 3, padding=1, bias=True)
        self.drop = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        self.bn2 = BatchNorm2d(cout, momentum=0.9)
        self.conv2 = Conv2d(cout, cout, 3, stride=stride, padding=1, bias=True)
        self.shortcut = None
        if stride != 1 or cin != cout:
            self.shortcut = Conv2d(cin, cout, 1, stride=stride, bias=True)

    def forward(self, x):
        y = self.drop(self.conv1(self.bn1(x, relu=True)))
        y = self.conv2(self.bn2(y, relu=True))
        return y + (x if self.shortcut is None else self.shortcut(x))


class WideResNet(nn.Module):
    def __init__(self, depth=28, widen_factor=10, dropout=0.3, num_classes=10):
        super().__init__()
        assert (depth - 4) % 6 == 0, "depth must be 6n + 4"
        n = (depth - 4) // 6
        widths = [16, 16 * widen_factor, 32 * widen_factor, 64 * widen_factor]
        self.conv1 = Conv2d(3, widths[0], 3, padding=1, bias=True)
        blocks, cin = [], widths[0]
        for stage, w in enumerate(widths[1:]):
            for b in range(n):
                blocks.append(WideBlock(cin, w, dropout, stride=(1 if stage == 0 else 2) if b == 0 else 1))
                cin = w
        self.blocks = nn.Sequential(*blocks)
        self.bn = BatchNorm2d(cin, momentum=0.9)
        self.linear = nn.Linear(cin, num_classes)

    def forward(self, x):
        x = self.blocks(self.conv1(x))
        x = self.bn(x, relu=True)
        x = F.adaptive_avg_pool2d(x, 1)
        return self.linear(torch.flatten(x, 1))


def WideResNet28_10(num_classes=100, dropout=0.3):
    return WideResNet(28, 10, dropout, num_classes)


def WideResNet40_10(num_classes=10, dropout=0.3):
    """Name kept from the reference, where it builds a 28-10 network."""
    return WideResNet(28, 10, dropout, num_classes)
