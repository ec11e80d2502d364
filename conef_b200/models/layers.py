"""Layers shared by the model zoo.

``Conv2d`` is ``torch.nn.Conv2d`` (same parameters, same ``state_dict``) whose backward pass computes the
bias gradient with the library's column-sum kernel when the output gradient lies in channels-last memory
on a GPU; everything else (the convolution itself, the input and weight gradients) stays with cuDNN.
The reference's Wide ResNet keeps a bias on every convolution
(examples/ImageClassification/models/wideresnet.py:10-13), and PyTorch's generic reduction spends 13 % of
a WRN-28-10 training step on those 28 bias gradients.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import native
from ..ops.colsum import channel_sum


class _ConvBiasFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding, dilation, groups):
        y = F.conv2d(x, weight, bias, stride, padding, dilation, groups)      # autocast applies as usual
        ctx.save_for_backward(x, weight)
        ctx.conf = (stride, padding, dilation, groups)
        ctx.bias_dtype = bias.dtype
        return y

    @staticmethod
    def backward(ctx, gy):
        x, weight = ctx.saved_tensors
        stride, padding, dilation, groups = ctx.conf
        if not gy.is_contiguous(memory_format=torch.channels_last):
            gy = gy.contiguous(memory_format=torch.channels_last)
        xx = x if x.dtype == gy.dtype else x.to(gy.dtype)
        ww = weight if weight.dtype == gy.dtype else weight.to(gy.dtype)
        gx, gw, _ = torch.ops.aten.convolution_backward(
            gy, xx, ww, None, list(stride), list(padding), list(dilation), False, [0, 0], groups,
            [ctx.needs_input_grad[0], ctx.needs_input_grad[1], False])
        gb = channel_sum(gy).to(ctx.bias_dtype) if ctx.needs_input_grad[2] else None
        return gx, gw, gb, None, None, None, None


class Conv2d(nn.Conv2d):
    """``nn.Conv2d`` with the bias gradient computed by ``conef_b200.ops.colsum.channel_sum``."""

    def forward(self, x):
        if (self.bias is not None and x.is_cuda and x.dim() == 4 and self.padding_mode == "zeros"
                and not isinstance(self.padding, str) and torch.is_grad_enabled() and self.bias.requires_grad
                and x.is_contiguous(memory_format=torch.channels_last) and native.available()):
            return _ConvBiasFn.apply(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)
        return super().forward(x)
