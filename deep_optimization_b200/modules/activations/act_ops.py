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

from ... import act_kernels, codec
from ..module_utils import unified_dequantize, unified_quantize


class _DOReLU(Function):
    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, input, relu, relu6, target_name, meta):
        m = meta[f"{target_name}"]
        ctx.fused = not m["act_padding"] and input.numel() % max(m["group_size"], 32) == 0
        if ctx.fused:
            # one pass: y and the 1-bit mask (act_ops.py:31-38 of the reference)
            y, packed, N, G = act_kernels.op("relu_fwd_fused_pack")(input, relu, relu6, 1, m["group_size"])
            ctx.meta_ngs = (N, G, m["group_size"])
            ctx.channels_last = codec.is_channels_last(input)      # the mask follows the input's memory order
            ctx.save_for_backward(packed)
            return y
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
        if ctx.fused:
            N, G, gs = ctx.meta_ngs
            if ctx.channels_last:
                dy = dy.contiguous(memory_format=torch.channels_last)
            elif codec.is_channels_last(dy):
                dy = dy.contiguous()
            return act_kernels.op("relu_bwd_fused_unpack")(packed, dy, 1, N, G, gs), None, None, None, None
        mask = unified_dequantize((packed, None, None), ctx.q_meta, None)
        return dy * mask.to(dy.dtype), None, None, None, None


def _save_derivative(ctx, deriv, target_name, meta):
    q_tensors, q_meta, _ = unified_quantize(deriv.to(torch.bfloat16), None, target_name, meta,
                                            clamp=False, clamp_alpha=0.0)
    ctx.q_meta = q_meta
    ctx.save_for_backward(q_tensors[0], q_tensors[1], q_tensors[2])


def _fused_ok(input, m):
    return not m["act_padding"] and not m.get("AVG_ALAM", False) and input.numel() % m["group_size"] == 0


def _fused_forward(ctx, input, kind, m):
    """activation + derivative codec in one kernel (flat grouping)."""
    if kind in ("gelu", "gelu_erf"):
        y, packed, scale, mn, N, G = act_kernels.op("gelu_fwd_fused_quan_pack")(input, m["bits"], m["group_size"],
                                                                                kind == "gelu_erf")
    else:
        y, packed, scale, mn, N, G = act_kernels.op("silu_fwd_quan_pack")(input, m["bits"], m["group_size"],
                                                                          False, False, 0)[:6]
    ctx.fused_meta = (N, G, m["bits"], m["group_size"])
    ctx.save_for_backward(packed, scale, mn)
    return y


def _apply_derivative(ctx, dy):
    packed, scale, mn = ctx.saved_tensors
    if getattr(ctx, "fused_meta", None) is not None:
        N, G, bits, gs = ctx.fused_meta
        return act_kernels.op("gelu_bwd_fused_dequan_unpack")(packed, dy, scale, mn, bits, N, G, gs)
    deriv = unified_dequantize((packed, scale, mn), ctx.q_meta, None)
    return dy * deriv.to(dy.dtype)


class _DOSiLU(Function):
    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, input, target_name, meta):
        ctx.fused_meta = None
        if _fused_ok(input, meta[f"{target_name}"]):
            return _fused_forward(ctx, input, "silu", meta[f"{target_name}"])
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
    """GELU: the tanh approximation of the reference's kernel
    (Activation_Compression/modules/activations/kernel_implementation.py:433-465) or, with
    `exact`, x * Phi(x), so that a module built from nn.GELU() keeps its function."""

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, input, target_name, meta, exact=False):
        ctx.fused_meta = None
        if _fused_ok(input, meta[f"{target_name}"]):
            return _fused_forward(ctx, input, "gelu_erf" if exact else "gelu", meta[f"{target_name}"])
        x = input.float()
        if exact:
            cdf = 0.5 * (1.0 + torch.erf(x * math.sqrt(0.5)))
            y = (x * cdf).to(input.dtype)
            deriv = cdf + x * torch.exp(-0.5 * x * x) * (1.0 / math.sqrt(2.0 * math.pi))
        else:
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
        return _apply_derivative(ctx, dy), None, None, None


class _DOMaxPool2d(Function):
    """max_pool2d of a channels-last activation whose saved state is a 4-bit argmax per output
    (PyTorch keeps an int64 index per output).  The caller checks `codec.maxpool_supported`."""

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, input, kernel_size, stride, padding):
        y, idx = codec.maxpool_fwd(input, kernel_size, stride, padding)
        ctx.geom = (tuple(input.shape), kernel_size, stride, padding)
        ctx.save_for_backward(idx)
        return y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        shape, k, s, pad = ctx.geom
        return codec.maxpool_bwd(idx, dy, shape, k, s, pad), None, None, None
