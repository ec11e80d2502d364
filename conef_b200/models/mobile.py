"""MobileNetV2 and ShuffleNetV2 for 32x32 inputs.

Counterparts of the reference's ``examples/ImageClassification/models/mobilenetv2.py:39-76`` and
``shufflenetv2.py:95-151``.
"""
import torch
import torch.nn as nn

from .layers import BatchNorm2d
import torch.nn.functional as F


class _InvertedResidual(nn.Module):
    def __init__(self, cin, cout, expansion, stride):
        super().__init__()
        mid = cin * expansion
        self.stride = stride
        self.conv1 = nn.Conv2d(cin, mid, 1, bias=False)
        self.bn1 = BatchNorm2d(mid)
        self.conv2 = nn.Conv2d(mid, mid, 3, stride, 1, groups=mid, bias=False)
        self.bn2 = BatchNorm2d(mid)
        self.conv3 = nn.Conv2d(mid, cout, 1, bias=False)
        self.bn3 = BatchNorm2d(cout)
        self.shortcut = None
        if stride == 1 and cin != cout:
            self.shortcut = nn.Sequential(nn.Conv2d(cin, cout, 1, bias=False), BatchNorm2d(cout))
        self.identity = stride == 1 and cin == cout

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = F.relu(self.bn2(self.conv2(y)))
        y = self.bn3(self.conv3(y))
        if self.stride == 1:
            y = y + (x if self.identity else self.shortcut(x))
        return y


class MobileNetV2(nn.Module):
    # (expansion, out channels, blocks, stride); strides adapted to 32x32 images
    cfg = [(1, 16, 1, 1), (6, 24, 2, 1), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]

    def __init__(self, num_classes=10):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 32, 3, 1, 1, bias=False)
        self.bn1 = BatchNorm2d(32)
        layers, cin = [], 32
        for t, c, n, s in self.cfg:
            for i in range(n):
                layers.append(_InvertedResidual(cin, c, t, s if i == 0 else 1))
                cin = c
        self.layers = nn.Sequential(*layers)
        self.conv2 = nn.Conv2d(320, 1280, 1, bias=False)
        self.bn2 = BatchNorm2d(1280)
        self.linear = nn.Linear(1280, num_classes)

    def forward(self, x):
        x = self.layers(F.relu(self.bn1(self.conv1(x))))
        x = F.relu(self.bn2(self.conv2(x)))
        return self.linear(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def _channel_shuffle(x, groups=2):
    n, c, h, w = x.shape
    return x.view(n, groups, c // groups, h, w).transpose(1, 2).reshape(n, c, h, w)


class _ShuffleUnit(nn.Module):
    """Stride 1: split channels, transform one half.  Stride 2: transform both branches."""

    def __init__(self, cin, cout, stride):
        super().__init__()
        self.stride = stride
        mid = cout // 2
        inp = cin if stride == 2 else cin // 2

        def branch(c_in):
            return nn.Sequential(
                nn.Conv2d(c_in, mid, 1, bias=False), BatchNorm2d(mid), nn.ReLU(inplace=True),
                nn.Conv2d(mid, mid, 3, stride, 1, groups=mid, bias=False), BatchNorm2d(mid),
                nn.Conv2d(mid, mid, 1, bias=False), BatchNorm2d(mid), nn.ReLU(inplace=True))
        self.right = branch(inp)
        self.left = None
        if stride == 2:
            self.left = nn.Sequential(
                nn.Conv2d(cin, cin, 3, 2, 1, groups=cin, bias=False), BatchNorm2d(cin),
                nn.Conv2d(cin, mid, 1, bias=False), BatchNorm2d(mid), nn.ReLU(inplace=True))

    def forward(self, x):
        if self.stride == 1:
            a, b = x.chunk(2, dim=1)
            out = torch.cat([a, self.right(b)], 1)
        else:
            out = torch.cat([self.left(x), self.right(x)], 1)
        return _channel_shuffle(out)


class ShuffleNetV2(nn.Module):
    configs = {0.5: (48, 96, 192, 1024), 1: (116, 232, 464, 1024), 1.5: (176, 352, 704, 1024), 2: (224, 488, 976, 2048)}

    def __init__(self, net_size=1, num_classes=10):
        super().__init__()
        c1, c2, c3, c4 = self.configs[net_size]
        self.conv1 = nn.Conv2d(3, 24, 3, 1, 1, bias=False)
        self.bn1 = BatchNorm2d(24)
        layers, cin = [], 24
        for cout, n in ((c1, 3), (c2, 7), (c3, 3)):
            layers.append(_ShuffleUnit(cin, cout, 2))
            layers += [_ShuffleUnit(cout, cout, 1) for _ in range(n)]
            cin = cout
        self.layers = nn.Sequential(*layers)
        self.conv2 = nn.Conv2d(cin, c4, 1, bias=False)
        self.bn2 = BatchNorm2d(c4)
        self.linear = nn.Linear(c4, num_classes)

    def forward(self, x):
        x = self.layers(F.relu(self.bn1(self.conv1(x))))
        x = F.relu(self.bn2(self.conv2(x)))
        return self.linear(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))
