"""Grouping of activations into `[N, G, group_size]` and back.

Same functions, argument orders and return tuples as
Activation_Compression/modules/tensor_act_reshape_utils.py:17-154:

* flat grouping: `[N, ...] -> [N, G, gs]`, zero-padding each sample's tail to a
  multiple of gs when `act_padding` is set;
* spatial grouping for 4-D activations whose H and W are multiples of
  sqrt(gs): each group is one sqrt(gs) x sqrt(gs) tile of one channel.

`channel_mean` is always False (the reference's channel-averaging branch is
commented out) and is carried only to keep the tuple layout.  The reference's
inverse of the spatial grouping views the tile grid as (new_W, new_H), which is
wrong for H != W; the inverse here uses (new_H, new_W).
"""
from __future__ import annotations

import math
from typing import Tuple

import torch
import torch.nn.functional as F
from torch import Tensor


def default_act_tensor_reshape(X: Tensor, Group_Size: int, act_padding: bool, pack_only: bool):
    N = X.shape[0]
    shape = X.shape
    if act_padding:
        flat = X.reshape(N, -1)
        pad = (-flat.size(1)) % Group_Size
        if pad:
            flat = F.pad(flat, (0, pad))
        X = flat
    x2 = X.reshape(N, -1, Group_Size)
    return x2, N, x2.shape[1], shape, False


def default_act_tensor_reshape_back(X: Tensor, _shape, act_padding: bool, channel_mean: bool) -> Tensor:
    N = _shape[0]
    flat = X.reshape(N, -1)
    if act_padding:
        flat = flat[:, :math.prod(_shape[1:])]
    out = flat.reshape(*_shape)
    if channel_mean:
        out = out.repeat(1, 2, 1, 1)
    return out


def act_tensor_reshape_pad_hepler(X: Tensor, H: int, W: int, sgs: int):
    pad_h, pad_w = (-H) % sgs, (-W) % sgs
    if pad_h or pad_w:
        X = F.pad(X, (0, pad_w, 0, pad_h), "constant", 0)
    return X, X.shape[2] // sgs, X.shape[3] // sgs


def spatical_aware_act_tensor_reshape_eligibility(X: Tensor, Group_Size: int, act_padding: bool) -> Tuple[bool, bool]:
    if act_padding or X.dim() != 4:
        return False, False
    sgs = int(math.isqrt(Group_Size))
    H, W = X.shape[2], X.shape[3]
    padding_elig = sgs * sgs != Group_Size
    reshape_elig = (H % sgs == 0) and (W % sgs == 0)
    return padding_elig, reshape_elig


def spatical_aware_act_tensor_reshape(X: Tensor, Group_Size: int, act_padding: bool, pack_only: bool):
    padding_elig, reshape_elig = spatical_aware_act_tensor_reshape_eligibility(X, Group_Size, act_padding)
    sgs = int(math.isqrt(Group_Size))
    # a non-square group size cannot be cut into sgs x sgs tiles; the reference
    # reaches its permute with it and fails, here it takes the flat grouping
    if not reshape_elig or padding_elig:
        x2, N, G, shape, cm = default_act_tensor_reshape(X, Group_Size, act_padding, pack_only)
        return x2, N, G, 0, 0, shape, False, False, cm
    N, C, H, W = X.shape
    new_H, new_W = H // sgs, W // sgs
    x2 = X.reshape(N, C, new_H, sgs, new_W, sgs).permute(0, 1, 2, 4, 3, 5)
    x2 = x2.reshape(N, C * new_H * new_W, Group_Size)
    return x2.contiguous(), N, x2.shape[1], new_H, new_W, X.shape, padding_elig, reshape_elig, False


def spatical_aware_act_tensor_reshape_back(X: Tensor, _shape, Group_Size: int, new_H: int, new_W: int,
                                           act_padding: bool, spatical_padding_eligibility: bool,
                                           spatical_reshape_eligibility: bool, channel_mean: bool) -> Tensor:
    if not spatical_reshape_eligibility:
        return default_act_tensor_reshape_back(X, _shape, act_padding, channel_mean).contiguous()
    N, C = _shape[0], _shape[1]
    sgs = int(math.isqrt(Group_Size))
    x2 = X.reshape(N, C, new_H, new_W, sgs, sgs).permute(0, 1, 2, 4, 3, 5)
    x2 = x2.reshape(N, C, new_H * sgs, new_W * sgs)
    if not spatical_padding_eligibility:
        x2 = x2[:, :, :_shape[2], :_shape[3]]
    x2 = x2.reshape(*_shape)
    if channel_mean:
        x2 = x2.repeat(1, 2, 1, 1)
    return x2.contiguous()
