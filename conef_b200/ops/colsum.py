"""Channel sums of a channels-last activation gradient (= the bias gradient of a convolution).

PyTorch's convolution backward computes the bias gradient with its generic reduction kernel, which
reaches about 0.5 TB/s on the bf16 gradients of WRN-28-10 (78 us for 42 MB; 28 convolutions with a
bias add up to 2.3 ms of an 18 ms step).  ``channel_sum`` streams the gradient once with 16-byte
loads (``csrc/colsum.cu``) and falls back to ``Tensor.sum`` for anything the kernel does not take.
"""
from __future__ import annotations

import torch

from . import native

_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
_MAX_PARTS = 592      # four CTAs per SM (the second stage adds the partial rows with 64 of them in flight)


def _rows_cols(t: torch.Tensor):
    """(rows, cols) when ``t`` is a dense (N, C, H, W) tensor in channels-last memory or a contiguous
    2-D matrix whose columns are the channels; else None."""
    if t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last):
        n, c, h, w = t.shape
        return n * h * w, c
    if t.dim() == 2 and t.is_contiguous():
        return t.shape[0], t.shape[1]
    return None


def channel_sum(t: torch.Tensor) -> torch.Tensor:
    """fp32 sums over every dimension but the channel dimension (dim 1 of a 4-D tensor, the columns of
    a matrix)."""
    rc = _rows_cols(t) if t.is_cuda and t.dtype in _DTYPES and native.available() else None
    if rc is not None:
        rows, cols = rc
        if cols % 8 == 0 and cols <= 2048 and t.data_ptr() % 16 == 0 and rows > 0:
            nparts = int(max(1, min(_MAX_PARTS, rows // 32)))
            partial = torch.empty(nparts * cols, dtype=torch.float32, device=t.device)
            out = torch.empty(cols, dtype=torch.float32, device=t.device)
            native.check(native.lib().conef_colsum(t.data_ptr(), _DTYPES[t.dtype], rows, cols, partial.data_ptr(),
                                                   nparts, out.data_ptr(), native.stream_ptr(t.device)), "colsum")
            return out
    dims = [d for d in range(t.dim()) if d != 1] if t.dim() != 2 else [0]
    return t.float().sum(dim=dims)


def _native_shape(t: torch.Tensor):
    """(rows, cols) when the native kernels take ``t``; else None."""
    if not (t.is_cuda and t.dtype in _DTYPES and native.available()):
        return None
    rc = _rows_cols(t)
    if rc is None:
        return None
    rows, cols = rc
    if cols % 8 != 0 or cols > 2048 or t.data_ptr() % 16 != 0 or rows <= 0:
        return None
    return rows, cols


def channel_stats(x: torch.Tensor, eps: float, running_mean=None, running_var=None, momentum: float = 0.1):
    """Batch-norm statistics of a channels-last activation: ``(mean, invstd)`` in fp32 with
    ``invstd = 1 / sqrt(biased variance + eps)``, and the momentum update of the running statistics in
    place (unbiased variance), as ``torch.batch_norm`` does in training mode.  Returns None when the
    native kernel does not take the input (the caller then uses the library)."""
    rc = _native_shape(x)
    if rc is None:
        return None
    for r in (running_mean, running_var):
        if r is not None and not (r.is_cuda and r.dtype == torch.float32 and r.is_contiguous()):
            return None
    rows, cols = rc
    nparts = int(max(1, min(_MAX_PARTS, rows // 32)))
    partial = torch.empty(nparts * 2 * cols, dtype=torch.float32, device=x.device)
    mean = torch.empty(cols, dtype=torch.float32, device=x.device)
    invstd = torch.empty(cols, dtype=torch.float32, device=x.device)
    native.check(native.lib().conef_colstats(
        x.data_ptr(), _DTYPES[x.dtype], rows, cols, float(eps), float(momentum), partial.data_ptr(), nparts,
        mean.data_ptr(), invstd.data_ptr(), native.ptr(running_mean), native.ptr(running_var),
        native.stream_ptr(x.device)), "colstats")
    return mean, invstd


def channel_dot(dy: torch.Tensor, x: torch.Tensor, mean: torch.Tensor, invstd: torch.Tensor):
    """``(sum_dy, sum_dy_xmu, grad_weight, grad_bias)`` of the batch-norm backward pass, all fp32; None
    when the native kernel does not take the inputs."""
    rc = _native_shape(x)
    if rc is None or dy.dtype != x.dtype or dy.shape != x.shape or _native_shape(dy) != rc:
        return None
    rows, cols = rc
    nparts = int(max(1, min(_MAX_PARTS, rows // 32)))
    dev = x.device
    partial = torch.empty(nparts * 2 * cols, dtype=torch.float32, device=dev)
    out = torch.empty(4, cols, dtype=torch.float32, device=dev)
    native.check(native.lib().conef_coldot(
        dy.data_ptr(), x.data_ptr(), _DTYPES[x.dtype], rows, cols, mean.data_ptr(), invstd.data_ptr(),
        partial.data_ptr(), nparts, out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), out[3].data_ptr(),
        native.stream_ptr(dev)), "coldot")
    return out[0], out[1], out[2], out[3]


def _elem_parts(rows: int) -> int:
    return int(max(1, min(4 * _MAX_PARTS, rows // 16)))


def bn_apply(x, mean, invstd, weight, bias, relu: bool):
    """``relu?((x - mean) * invstd * weight + bias)`` in one pass over a channels-last activation; None
    when the native kernel does not take the input."""
    rc = _native_shape(x)
    if rc is None:
        return None
    rows, cols = rc
    y = torch.empty_like(x)      # keeps the channels-last strides
    if y.data_ptr() % 16 != 0:
        return None
    native.check(native.lib().conef_bn_apply(
        x.data_ptr(), y.data_ptr(), _DTYPES[x.dtype], rows, cols, mean.data_ptr(), invstd.data_ptr(),
        native.ptr(weight), native.ptr(bias), int(bool(relu)), _elem_parts(rows), native.stream_ptr(x.device)),
        "bn_apply")
    return y


def channel_dot_relu(dy, x, mean, invstd, weight, bias):
    """:func:`channel_dot` with ``dy`` masked where the ReLU behind the batch norm is inactive."""
    rc = _native_shape(x)
    if rc is None or dy.dtype != x.dtype or dy.shape != x.shape or _native_shape(dy) != rc:
        return None
    rows, cols = rc
    nparts = int(max(1, min(_MAX_PARTS, rows // 32)))
    dev = x.device
    partial = torch.empty(nparts * 2 * cols, dtype=torch.float32, device=dev)
    out = torch.empty(4, cols, dtype=torch.float32, device=dev)
    native.check(native.lib().conef_coldot_relu(
        dy.data_ptr(), x.data_ptr(), _DTYPES[x.dtype], rows, cols, mean.data_ptr(), invstd.data_ptr(),
        native.ptr(weight), native.ptr(bias), partial.data_ptr(), nparts, out[0].data_ptr(), out[1].data_ptr(),
        out[2].data_ptr(), out[3].data_ptr(), native.stream_ptr(dev)), "coldot_relu")
    return out[0], out[1], out[2], out[3]


def bn_backward_apply(gy, x, mean, invstd, weight, bias, sum_dy, sum_dy_xmu, relu: bool):
    """Input gradient of batch norm (+ ReLU) in one pass; None when the native kernel does not take the inputs."""
    rc = _native_shape(x)
    if rc is None or gy.dtype != x.dtype or _native_shape(gy) != rc:
        return None
    rows, cols = rc
    gx = torch.empty_like(x)
    if gx.data_ptr() % 16 != 0:
        return None
    native.check(native.lib().conef_bn_backward_apply(
        gy.data_ptr(), x.data_ptr(), gx.data_ptr(), _DTYPES[x.dtype], rows, cols, mean.data_ptr(), invstd.data_ptr(),
        native.ptr(weight), native.ptr(bias), sum_dy.data_ptr(), sum_dy_xmu.data_ptr(), int(bool(relu)),
        _elem_parts(rows), native.stream_ptr(x.device)), "bn_backward_apply")
    return gx


def bias_add_(y: torch.Tensor, bias: torch.Tensor) -> bool:
    """``y[:, c] += bias[c]`` in place on a channels-last activation; False when the native kernel does
    not take the input (nothing is changed then)."""
    rc = _native_shape(y)
    if rc is None or not (bias.is_cuda and bias.dtype == torch.float32 and bias.is_contiguous()):
        return False
    rows, cols = rc
    native.check(native.lib().conef_bias_add(y.data_ptr(), _DTYPES[y.dtype], rows, cols, bias.data_ptr(),
                                             _elem_parts(rows), native.stream_ptr(y.device)), "bias_add")
    return True


def layer_norm_wgrad(dy: torch.Tensor, x: torch.Tensor, mean: torch.Tensor, rstd: torch.Tensor):
    """``(dgamma, dbeta)`` (fp32) of a layer norm over the last dimension; ``mean`` / ``rstd`` are the per-row
    statistics its forward pass saved.  None when the native kernel does not take the inputs."""
    if not (x.is_cuda and x.dtype in _DTYPES and dy.dtype == x.dtype and native.available()
            and x.is_contiguous() and dy.is_contiguous() and dy.shape == x.shape):
        return None
    cols = x.shape[-1]
    rows = x.numel() // cols
    if (cols % 8 != 0 or cols > 2048 or rows <= 0 or x.data_ptr() % 16 != 0 or dy.data_ptr() % 16 != 0
            or mean.numel() != rows or rstd.numel() != rows or mean.dtype != torch.float32 or rstd.dtype != torch.float32
            or not mean.is_contiguous() or not rstd.is_contiguous()):
        return None
    nparts = int(max(1, min(_MAX_PARTS, rows // 32)))
    partial = torch.empty(nparts * 2 * cols, dtype=torch.float32, device=x.device)
    out = torch.empty(2, cols, dtype=torch.float32, device=x.device)
    native.check(native.lib().conef_ln_wgrad(
        dy.data_ptr(), x.data_ptr(), _DTYPES[x.dtype], rows, cols, mean.data_ptr(), rstd.data_ptr(),
        partial.data_ptr(), nparts, out[0].data_ptr(), out[1].data_ptr(), native.stream_ptr(x.device)), "ln_wgrad")
    return out[0], out[1]


def cast_like_autocast(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``t.to(dtype)``; the fp32 -> bf16 case of a dense CUDA tensor runs on the library's vectorised copy
    (PyTorch's kernel for this pair of types reaches 0.5 TB/s)."""
    if t.dtype == dtype:
        return t
    if (t.dtype == torch.float32 and dtype == torch.bfloat16 and t.is_cuda and native.available()
            and (t.is_contiguous() or t.is_contiguous(memory_format=torch.channels_last)) and t.data_ptr() % 16 == 0):
        out = torch.empty_like(t, dtype=dtype)      # same strides
        if out.data_ptr() % 16 == 0:
            native.check(native.lib().conef_cast_f32_bf16(t.data_ptr(), out.data_ptr(), t.numel(),
                                                          native.stream_ptr(t.device)), "cast")
            return out
    return t.to(dtype)
