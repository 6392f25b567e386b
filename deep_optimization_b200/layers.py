"""Drop-in conv / linear modules (Activation_Compression/layers.py:11-188).

Constructor signatures match the reference (including its `out_channesl` and
`in_chanels` spellings being positional).  In eval mode they are the stock
modules; in training they call the save-for-backward Functions.  Conv1d/3d use
`clamp_alpha` for the PACT clamp (the reference reads an undefined `pact_alpha`
and forgets `.apply`).  The conv modules take a trailing `bias` keyword (default
False, the reference's fixed choice) so that a biased convolution can be swapped
without losing its bias.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .modules.ops import GroupPACTClampFn, _DOConv1d, _DOConv2d, _DOConv3d, _DOLinear


class DOLinear(nn.Linear):
    def __init__(self, in_features, out_features, clamp_alpha=3.0, target_name=None, meta={}):
        super().__init__(in_features, out_features)
        self.clamp_alpha, self.target_name, self.meta = clamp_alpha, target_name, meta
        self.ema_grad_meta = None

    def forward(self, x):
        if self.training:
            return _DOLinear.apply(x, self.weight, self.clamp_alpha, self.target_name, self.meta,
                                   self.ema_grad_meta, self.bias)
        return super().forward(x)


class _DOConvMixin:
    _fn = None
    _pact = False

    def _init_do(self, clamp_alpha, target_name, meta):
        self.clamp_alpha, self.target_name, self.meta = clamp_alpha, target_name, meta
        self.ema_grad_meta = None
        self.learnable_scale = None

    def forward(self, x):
        if not self.training:
            return super().forward(x)
        if self._pact:
            x = GroupPACTClampFn.apply(x, self.clamp_alpha, self.meta[f"{self.target_name}"]["group_size"],
                                       self.meta, self.target_name)
        padding = self.padding
        if self.padding_mode != "zeros":
            x = F.pad(x, self._reversed_padding_repeated_twice, mode=self.padding_mode)
            padding = 0
        return self._fn.apply(x, self.weight, self.learnable_scale, self.stride, padding, self.dilation,
                              self.groups, self.clamp_alpha, self.target_name, self.meta, self.ema_grad_meta,
                              self.bias)


class DOConv1d(_DOConvMixin, nn.Conv1d):
    _fn, _pact = _DOConv1d, True

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 padding_mode="zeros", clamp_alpha=3.0, target_name=None, meta={}, bias=False):
        nn.Conv1d.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups,
                           bias=bias, padding_mode=padding_mode)
        self._init_do(clamp_alpha, target_name, meta)


class DOConv2d(_DOConvMixin, nn.Conv2d):
    _fn = _DOConv2d

    def __init__(self, in_channels, out_channesl, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 padding_mode="zeros", clamp_alpha=3.0, target_name=None, meta={}, bias=False):
        nn.Conv2d.__init__(self, in_channels, out_channesl, kernel_size, stride, padding, dilation, groups,
                           bias=bias, padding_mode=padding_mode)
        self._init_do(clamp_alpha, target_name, meta)


class DOConv3d(_DOConvMixin, nn.Conv3d):
    _fn, _pact = _DOConv3d, True

    def __init__(self, in_chanels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 padding_mode="zeros", clamp_alpha=3.0, target_name=None, meta={}, bias=False):
        nn.Conv3d.__init__(self, in_chanels, out_channels, kernel_size, stride, padding, dilation, groups,
                           bias=bias, padding_mode=padding_mode)
        self._init_do(clamp_alpha, target_name, meta)


class DODepthPointConv2d(nn.Module):
    """Depth-wise conv followed by a 1x1 conv, both compressed (layers.py:170-188; the
    reference forwards an `acc_var` keyword its DOConv2d does not take)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 padding_mode="zeros", acc_var=5.0, target_name=None, meta={}):
        super().__init__()
        self.depth_quanconv2d = DOConv2d(in_channels, in_channels, kernel_size, stride=stride, padding=padding,
                                         dilation=dilation, groups=in_channels, padding_mode=padding_mode,
                                         clamp_alpha=acc_var, target_name=target_name, meta=meta)
        self.point_quanconv2d = DOConv2d(in_channels, out_channels, 1, clamp_alpha=acc_var,
                                         target_name=target_name, meta=meta)

    def forward(self, x):
        return self.point_quanconv2d(self.depth_quanconv2d(x))


class RMSNorm(nn.Module):
    def __init__(self, dims, eps=1e-8):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dims))
        self.eps = eps

    def forward(self, x):
        return x * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps).to(x.dtype) * self.weight
