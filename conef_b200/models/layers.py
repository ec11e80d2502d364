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
        from ..ops.colsum import bias_add_, cast_like_autocast
        if torch.is_autocast_enabled():      # cast once here (vectorised copy) and keep the casts for the backward pass
            dt = torch.get_autocast_dtype("cuda")
            x = cast_like_autocast(x, dt)
            weight = cast_like_autocast(weight, dt)
        y = F.conv2d(x, weight, None, stride, padding, dilation, groups)
        if not bias_add_(y, bias):      # the library adds it with a broadcasting kernel that is not vectorised
            y = y + bias.to(y.dtype).view(1, -1, 1, 1)
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


class _BatchNormFn(torch.autograd.Function):
    """Training-mode batch norm over a channels-last activation, optionally fused with the ReLU behind it.
    All four passes run on the library's column kernels (``csrc/colsum.cu``): statistics (before this
    function), the normalisation (+ ReLU) in one pass, the backward sums of dy and dy (x - mean) with dy
    masked by the ReLU, and the input gradient in one pass.  Anything the kernels do not take goes through
    ``batch_norm_elemt`` / ``batch_norm_backward_reduce`` / ``batch_norm_backward_elemt`` (the ops
    SyncBatchNorm is built from) and a separate ReLU."""

    @staticmethod
    def forward(ctx, x, weight, bias, mean, invstd, eps, count, relu):
        from ..ops.colsum import bn_apply
        y = bn_apply(x, mean, invstd, weight, bias, relu)
        if y is None:
            y = torch.batch_norm_elemt(x, weight, bias, mean, invstd, eps)
            if relu:
                y = torch.relu(y)
        ctx.save_for_backward(x, weight, bias, mean, invstd, count)
        ctx.relu = relu
        return y

    @staticmethod
    def backward(ctx, gy):
        from ..ops.colsum import bn_backward_apply, channel_dot, channel_dot_relu
        x, weight, bias, mean, invstd, count = ctx.saved_tensors
        relu = ctx.relu
        if gy.dtype != x.dtype:
            gy = gy.to(x.dtype)
        if not gy.is_contiguous(memory_format=torch.channels_last):
            gy = gy.contiguous(memory_format=torch.channels_last)
        sums = channel_dot_relu(gy, x, mean, invstd, weight, bias) if relu else channel_dot(gy, x, mean, invstd)
        native_mask = sums is not None
        if sums is None:
            if relu:      # mask by the recomputed activation, then the unfused ops
                gy = gy * (torch.batch_norm_elemt(x, weight, bias, mean, invstd, 0.0) > 0)
            sums = torch.batch_norm_backward_reduce(gy, x, mean, invstd, weight, True, True, True)
        sum_dy, sum_dy_xmu, gw, gb = sums
        gx = None
        if ctx.needs_input_grad[0]:
            gx = bn_backward_apply(gy, x, mean, invstd, weight, bias, sum_dy, sum_dy_xmu, relu and native_mask)
            if gx is None:
                if relu and native_mask:
                    gy = gy * (torch.batch_norm_elemt(x, weight, bias, mean, invstd, 0.0) > 0)
                gx = torch.batch_norm_backward_elemt(gy, x, mean, invstd, weight, sum_dy, sum_dy_xmu, count)
        return gx, gw.to(weight.dtype), gb.to(weight.dtype), None, None, None, None, None


class BatchNorm2d(nn.BatchNorm2d):
    """``nn.BatchNorm2d`` (same parameters, buffers and ``state_dict``) whose training-mode passes run on
    ``conef_b200.ops.colsum`` when the input lies in channels-last memory on a GPU; ``forward(x, relu=True)``
    applies the ReLU that follows in the same passes.  PyTorch's channels-last statistics kernels reach
    about 0.8 TB/s on WRN-28-10's bf16 activations (55-59 us per 42 MB pass), and batch norm + ReLU cost
    two passes over the activation in each direction."""

    def forward(self, x, relu: bool = False):
        if (self.training and self.track_running_stats and self.affine and self.momentum is not None
                and x.is_cuda and x.dim() == 4 and torch.is_grad_enabled() and native.available()
                and x.is_contiguous(memory_format=torch.channels_last)):
            from ..ops.colsum import channel_stats
            stats = channel_stats(x, self.eps, self.running_mean, self.running_var, self.momentum)
            if stats is not None:
                if self.num_batches_tracked is not None:
                    self.num_batches_tracked.add_(1)
                n = x.numel() // x.shape[1]
                key = (n, x.device)
                if getattr(self, "_count_key", None) != key:
                    self._count = torch.full((1,), n, dtype=torch.int32, device=x.device)
                    self._count_key = key
                return _BatchNormFn.apply(x, self.weight, self.bias, stats[0], stats[1], self.eps, self._count, relu)
        y = super().forward(x)
        return F.relu(y) if relu else y


class _LinearFn(torch.autograd.Function):
    """``F.linear`` whose bias gradient (a column sum over all tokens) runs on ``channel_sum``; PyTorch uses
    its generic reduction there (20 us per 16 MB gradient of BERT-large, 146 of them per step)."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        if torch.is_autocast_enabled():      # cast once here and keep the casts for the backward pass
            from ..ops.colsum import cast_like_autocast
            dt = torch.get_autocast_dtype("cuda")
            x = cast_like_autocast(x, dt)
            weight = cast_like_autocast(weight, dt)
        y = F.linear(x, weight, bias)
        ctx.save_for_backward(x, weight)
        ctx.bias_dtype = bias.dtype
        return y

    @staticmethod
    def backward(ctx, gy):
        x, weight = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        if g2.dtype != weight.dtype:
            g2 = g2.to(weight.dtype)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        gx = g2.matmul(weight).view(x.shape) if ctx.needs_input_grad[0] else None
        gw = g2.t().matmul(x.reshape(-1, x.shape[-1])) if ctx.needs_input_grad[1] else None
        gb = channel_sum(g2).to(ctx.bias_dtype) if ctx.needs_input_grad[2] else None
        return gx, gw, gb


class Linear(nn.Linear):
    """``nn.Linear`` (same parameters and ``state_dict``) with the bias gradient computed by
    ``conef_b200.ops.colsum.channel_sum`` on a GPU."""

    def forward(self, x):
        if (self.bias is not None and x.is_cuda and torch.is_grad_enabled() and self.bias.requires_grad
                and x.dim() >= 2 and self.out_features % 8 == 0 and native.available()):
            return _LinearFn.apply(x, self.weight, self.bias)
        return super().forward(x)


class _LayerNormFn(torch.autograd.Function):
    """Layer norm whose weight and bias gradients (column sums over all tokens) run on
    ``ops.colsum.layer_norm_wgrad``; the forward pass and the input gradient stay with PyTorch."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        if torch.is_autocast_enabled():      # autocast runs layer norm in fp32
            x = x.float()
        x = x.contiguous()
        y, mean, rstd = torch.native_layer_norm(x, [x.shape[-1]], weight, bias, eps)
        ctx.save_for_backward(x, weight, bias, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, gy):
        from ..ops.colsum import layer_norm_wgrad
        x, weight, bias, mean, rstd = ctx.saved_tensors
        if gy.dtype != x.dtype:
            gy = gy.to(x.dtype)
        gy = gy.contiguous()
        grads = layer_norm_wgrad(gy, x, mean, rstd) if (ctx.needs_input_grad[1] or ctx.needs_input_grad[2]) else None
        mask = [ctx.needs_input_grad[0], grads is None and ctx.needs_input_grad[1], grads is None and ctx.needs_input_grad[2]]
        gx, gw, gb = torch.ops.aten.native_layer_norm_backward(gy, x, [x.shape[-1]], mean, rstd, weight, bias, mask)
        if grads is not None:
            gw, gb = grads[0].to(weight.dtype), grads[1].to(bias.dtype)
        return gx, gw, gb, None


class LayerNorm(nn.LayerNorm):
    """``nn.LayerNorm`` (same parameters and ``state_dict``) over the last dimension with the weight and bias
    gradients on the library's column kernel when the input is on a GPU."""

    def forward(self, x):
        if (self.elementwise_affine and self.bias is not None and len(self.normalized_shape) == 1 and x.is_cuda
                and torch.is_grad_enabled() and self.weight.requires_grad and native.available()
                and self.normalized_shape[0] % 8 == 0 and self.normalized_shape[0] <= 2048):
            return _LayerNormFn.apply(x, self.weight, self.bias, self.eps)
        return super().forward(x)
