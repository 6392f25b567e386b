"""The quantise boundary every save-for-backward Function calls.

`quantize / dequantize / unified_quantize / unified_dequantize` keep the
signatures, the `(tensors, 14-tuple meta)` return layout and the DIVISION
residual of Activation_Compression/modules/module_utils.py:28-102; the kernels
behind `torch.ops.act_lib.*` are the CUDA ones registered by `act_kernels` (reached through
`act_kernels.op`, which skips the dispatcher in eager mode).

q_meta order (module_utils.py:37,68):
  (bits, pack_only, group_size, act_padding, N, G, new_H, new_W,
   spatial_pad_elig, spatial_reshape_elig, channel_mean, avg_alam, alam_bits, ori_shape)
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _lib, act_kernels, codec
from .tensor_act_reshape_utils import (
    spatical_aware_act_tensor_reshape,
    spatical_aware_act_tensor_reshape_back,
    spatical_aware_act_tensor_reshape_eligibility,
)

_TILE = {64: 8, 256: 16, 1024: 32}


class ChannelsLastShape(tuple):
    """The `ori_shape` entry of q_meta for an activation that was stored channels-last: the
    logical [N, C, H, W] shape, tagged so that `dequantize` rebuilds the same memory format.
    Such a tensor is grouped flat over its NHWC memory order (no conversion copy either way)."""


def _tiled_in_place(input, group_size, act_padding, pack_only, avg_alam):
    """Spatial grouping that the tiled kernels read and write in place (no permute copy): the
    spatial branch of the reshape helpers, in the two fixed-point modes."""
    if pack_only or avg_alam or act_kernels.get_mode() == "ref_compat" or not codec.tiles_supported(input, group_size):
        return False
    pad_elig, reshape_elig = spatical_aware_act_tensor_reshape_eligibility(input, group_size, act_padding)
    return reshape_elig and not pad_elig


def quantize(input, bits, pack_only, group_size, act_padding, N, avg_alam, alam_bits, clamp, clamp_alpha):
    if codec.is_channels_last(input):
        # [N, H*W*C] view of the memory as it lies; flat groups; the shape entry records the format
        n = input.shape[0]
        tensors, q_meta = quantize(input.permute(0, 2, 3, 1).reshape(n, -1), bits, pack_only, group_size,
                                   act_padding, N, avg_alam, alam_bits, clamp, clamp_alpha)
        return tensors, q_meta[:-1] + (ChannelsLastShape(input.shape),)
    if _tiled_in_place(input, group_size, act_padding, pack_only, avg_alam):
        t = _TILE[group_size]
        n, C, H, W = input.shape
        G = C * (H // t) * (W // t)
        flags = _lib.ACT_FLAG_ROUND_NEAREST if act_kernels.get_mode() == "nearest" else 0
        out, scaler, ema_min = codec.quant_pack_tiles(input, bits, t, flags=flags)
        return (out, scaler.view(n, G), ema_min.view(n, G)), (bits, pack_only, group_size, act_padding, n, G, H // t,
                                                              W // t, False, True, False, avg_alam, alam_bits,
                                                              input.shape)
    groups, N, G, new_H, new_W, ori_shape, pad_elig, reshape_elig, channel_mean = \
        spatical_aware_act_tensor_reshape(input, Group_Size=group_size, act_padding=act_padding,
                                          pack_only=pack_only)
    if pack_only:
        out = act_kernels.op("pack_triton")(groups, bits, group_size)
        # the reference records (0, 0, False, False) here although it grouped spatially,
        # which scrambles masks on the way back; the real grouping is recorded instead
        return (out, None, None), (bits, pack_only, group_size, act_padding, N, G, new_H, new_W, pad_elig,
                                   reshape_elig, channel_mean, None, None, ori_shape)
    out, scaler, ema_min = act_kernels.op("quant_pack_triton")(groups, bits, group_size, avg_alam,
                                                               alam_bits, clamp, clamp_alpha)
    return (out, scaler, ema_min), (bits, pack_only, group_size, act_padding, N, G, new_H, new_W,
                                    pad_elig, reshape_elig, channel_mean, avg_alam, alam_bits, ori_shape)


def unified_quantize(input, input_l, target_name, meta, clamp, clamp_alpha):
    m = meta[f"{target_name}"]
    tensors, q_meta = quantize(input, m["bits"], m["pack_only"], m["group_size"], m["act_padding"],
                               m["N"], m["AVG_ALAM"], m["ALAM_BITS"], clamp, clamp_alpha)
    return tensors, q_meta, input_l


def dequantize(quantized_tensor, quantized_meta):
    q_input, q_scale, ema_mn = quantized_tensor
    (q_bits, pack_only, group_size, act_padding, N, G, new_H, new_W, pad_elig, reshape_elig,
     channel_mean, avg_alam, alam_bits, input_shape) = quantized_meta
    if isinstance(input_shape, ChannelsLastShape):
        n, C, H, W = input_shape
        flat = dequantize(quantized_tensor, tuple(quantized_meta[:-1]) + (torch.Size((n, H * W * C)),))
        return flat.view(n, H, W, C).permute(0, 3, 1, 2)
    if (not pack_only and reshape_elig and not pad_elig and not avg_alam and group_size in _TILE
            and q_input.is_cuda and len(input_shape) == 4):
        return codec.dequant_unpack_tiles(q_input, q_scale.reshape(-1), ema_mn.reshape(-1), q_bits,
                                          _TILE[group_size], tuple(input_shape))
    if pack_only:
        unpack = act_kernels.op("unpack_triton")(q_input, q_bits, N, G, group_size)
    else:
        unpack = act_kernels.op("dequant_unpack_triton")(q_input, q_scale, ema_mn, q_bits, group_size,
                                                         avg_alam, alam_bits)
    return spatical_aware_act_tensor_reshape_back(unpack, input_shape, group_size, new_H, new_W,
                                                  act_padding, pad_elig, reshape_elig, channel_mean)


def low_pass_upsampled(input_l, input_shape):
    """The stored low-pass part of a DIVISION layer, nearest-upsampled to the layer input's
    shape (module_utils.py:91-102).  Forward subtracts exactly this tensor before the codec
    and backward adds it back, so the pair cancels whatever the e4m3 storage lost."""
    if len(input_shape) == 4:
        size = (input_shape[-2], input_shape[-1])
    elif len(input_shape) == 3:
        size = input_shape[2]
    else:
        size = input_shape[0]
    return F.interpolate(input_l.to(torch.bfloat16), size=size, mode="nearest")


def unified_dequantize(ori_quantized_tensor, ori_quantized_meta, input_l):
    input_shape = ori_quantized_meta[-1]
    x = dequantize(ori_quantized_tensor, ori_quantized_meta)
    if input_l is None:
        return x
    # DIVISION: residual + low-pass part
    return x + low_pass_upsampled(input_l, input_shape).to(x.dtype)
