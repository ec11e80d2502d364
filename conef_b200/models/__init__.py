"""Model zoo of the example workloads (framework-layer PyTorch code)."""
from .resnet_cifar import CifarResNet, ResNet20, ResNet32, ResNet56
from .wideresnet import WideResNet, WideResNet28_10, WideResNet40_10

__all__ = ["CifarResNet", "ResNet20", "ResNet32", "ResNet56", "WideResNet", "WideResNet28_10", "WideResNet40_10"]
