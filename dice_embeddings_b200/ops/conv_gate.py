"""Fused convolution → batch normalisation → ReLU of the convolutional gate models (ConEx, AConEx, ConvQ, AConvQ,
ConvO, AConvO) as one autograd function over the sm_100a kernels of ``csrc/conv_gate.cu``.

The reference builds the ``[B, 1, 2k, d/k]`` image with ``torch.cat``, runs ``nn.Conv2d(1, C, 3, padding=1)``,
``nn.BatchNorm2d(C)`` and ``relu`` as separate library kernels and keeps the convolution output, its normalised copy
and the ReLU output for autograd (``dicee/models/complex.py:47-66``, ``dicee/models/quaternion.py:262-283``,
``dicee/models/octonion.py:214-236``).  Here only the image and the final feature map exist in memory: every pass
recomputes the nine-tap convolution from the image in shared memory (it costs less than reading a stored copy), and
the batch statistics, the weight gradient and the image gradient come out of the same passes.

``conv_gate_features`` is used by ``residual_convolution`` when the tensors are on a B200, the kernel is 3x3, the
channel count is at most 8 and no feature-map dropout is active; other cases take the PyTorch layers.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import _lib
from . import kernels as K


def supported(x: torch.Tensor, conv: nn.Conv2d, bn: nn.BatchNorm2d, H: int, W: int) -> bool:
    """True when the fused kernels cover this call (device, dtype, kernel size, channel count, plane size)."""
    if not (x.is_cuda and x.dtype == torch.float32 and _lib.available()):
        return False
    if torch.cuda.get_device_capability(x.device)[0] != 10:
        return False
    if tuple(conv.kernel_size) != (3, 3) or tuple(conv.padding) != (1, 1) or tuple(conv.stride) != (1, 1):
        return False
    if conv.in_channels != 1 or conv.bias is None or conv.groups != 1 or tuple(conv.dilation) != (1, 1):
        return False
    if not bn.training and bn.running_mean is None:
        return False
    if bn.momentum is None:   # cumulative moving average is not implemented in the kernel
        return False
    return bool(_lib.lib().dice_conv_gate_supported(int(x.shape[0]), int(H), int(W), int(conv.out_channels)))


class _ConvGateFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, gamma, beta, run_mean, run_var, training, momentum, eps, H, W):
        B, C = x.shape[0], weight.shape[0]
        x = x.contiguous()
        w = weight.detach().reshape(C, 9).contiguous()
        b = bias.detach().contiguous()
        dev = x.device
        stats = torch.empty(2 * C, dtype=torch.float64, device=dev)
        fold = torch.empty(4 * C, dtype=torch.float32, device=dev)
        out = torch.empty(B, C * H * W, dtype=torch.float32, device=dev)
        K._call("dice_conv_gate_forward", x, B, H, W, C, int(training), x.data_ptr(), w.data_ptr(), b.data_ptr(),
                K._ptr(gamma), K._ptr(beta), K._ptr(run_mean), K._ptr(run_var), float(momentum), float(eps),
                stats.data_ptr(), fold.data_ptr(), out.data_ptr(), others=(w, b, gamma, beta, run_mean, run_var))
        ctx.save_for_backward(x, w, b, fold)
        ctx.shape = (B, H, W, C, bool(training))
        ctx.has_affine = gamma is not None
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, w, b, fold = ctx.saved_tensors
        B, H, W, C, training = ctx.shape
        dev = x.device
        g = grad_out.contiguous()
        bstats = torch.empty(2 * C, dtype=torch.float64, device=dev)
        dwb = torch.empty(10 * C, dtype=torch.float64, device=dev)
        dx = torch.empty_like(x)
        K._call("dice_conv_gate_backward", x, B, H, W, C, int(training), x.data_ptr(), w.data_ptr(), b.data_ptr(),
                fold.data_ptr(), g.data_ptr(), bstats.data_ptr(), dx.data_ptr(), dwb.data_ptr(), others=(w, b, fold, g))
        dweight = dwb[: 9 * C].to(torch.float32).reshape(C, 1, 3, 3)
        dbias = dwb[9 * C:].to(torch.float32)
        dgamma = bstats[:C].to(torch.float32) if ctx.has_affine else None
        dbeta = bstats[C:].to(torch.float32) if ctx.has_affine else None
        return dx, dweight, dbias, dgamma, dbeta, None, None, None, None, None, None, None


def conv_gate_features(x: torch.Tensor, conv: nn.Conv2d, bn: nn.BatchNorm2d, H: int, W: int) -> torch.Tensor:
    """``relu(bn(conv(x.view(B, 1, H, W)))).view(B, -1)`` for ``x`` of shape ``[B, H·W]``.

    In training mode the batch statistics are used and ``bn.running_mean`` / ``running_var`` /
    ``num_batches_tracked`` are updated exactly as ``nn.BatchNorm2d`` does."""
    training = bn.training or bn.running_mean is None
    run_mean: Optional[torch.Tensor] = bn.running_mean if bn.track_running_stats else None
    run_var: Optional[torch.Tensor] = bn.running_var if bn.track_running_stats else None
    if training and bn.track_running_stats and bn.num_batches_tracked is not None:
        bn.num_batches_tracked.add_(1)
    return _ConvGateFunction.apply(x, conv.weight, conv.bias, bn.weight, bn.bias, run_mean, run_var, training,
                                   bn.momentum, bn.eps, H, W)
