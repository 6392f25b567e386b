"""Activation Functions that keep only compressed state for backward.

ReLU / ReLU6 keep a 1-bit mask; SiLU and GELU keep their *derivative*,
quantised, so backward is `dy * unpack(derivative)` -- the scheme of
Activation_Compression/modules/activations/act_ops.py:16-164.  The element-wise
maths is plain PyTorch; the compressed state goes through the CUDA codec.
"""
from __future__ import annotations

import math

import torch
from torch.amp import custom_bwd, custom_fwd
from torch.autograd import Function

from ..module_utils import unified_dequantize, unified_quantize


class _DOReLU(Function):
    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, input, relu, relu6, target_name, meta):
        if relu6 and not relu:
            mask = (input > 0) & (input < 6)
        else:
            mask = input > 0
        y = torch.where(mask, input, torch.zeros((), dtype=input.dtype, device=input.device))
        m = dict(meta[f"{target_name}"])
        m["pack_only"], m["bits"] = True, 1
        q_tensors, q_meta, _ = unified_quantize(mask.to(torch.int8), None, target_name,
                                                {f"{target_name}": m}, clamp=False, clamp_alpha=0.0)
        ctx.q_meta = q_meta
        ctx.save_for_backward(q_tensors[0])
        return y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, dy):
        (packed,) = ctx.saved_tensors
        mask = unified_dequantize((packed, None, None), ctx.q_meta, None)
        return dy * mask.to(dy.dtype), None, None, None, None


def _save_derivative(ctx, deriv, target_name, meta):
    q_tensors, q_meta, _ = unified_quantize(deriv.to(torch.bfloat16), None, target_name, meta,
                                            clamp=False, clamp_alpha=0.0)
    ctx.q_meta = q_meta
    ctx.save_for_backward(q_tensors[0], q_tensors[1], q_tensors[2])


def _apply_derivative(ctx, dy):
    packed, scale, mn = ctx.saved_tensors
    deriv = unified_dequantize((packed, scale, mn), ctx.q_meta, None)
    return dy * deriv.to(dy.dtype)


class _DOSiLU(Function):
    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, input, target_name, meta):
        x = input.float()
        sig = torch.sigmoid(x)
        y = (x * sig).to(input.dtype)
        _save_derivative(ctx, sig + x * sig * (1.0 - sig), target_name, meta)
        return y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, dy):
        return _apply_derivative(ctx, dy), None, None


class _DOGELU(Function):
    """tanh-approximated GELU, as the reference's kernel
    (Activation_Compression/modules/activations/kernel_implementation.py:433-465)."""

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, input, target_name, meta):
        x = input.float()
        k = math.sqrt(2.0 / math.pi)
        inner = k * (x + 0.044715 * x * x * x)
        th = torch.tanh(inner)
        y = (0.5 * x * (1.0 + th)).to(input.dtype)
        deriv = 0.5 * (1.0 + th) + 0.5 * x * (1.0 - th * th) * k * (1.0 + 3 * 0.044715 * x * x)
        _save_derivative(ctx, deriv, target_name, meta)
        return y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, dy):
        return _apply_derivative(ctx, dy), None, None
