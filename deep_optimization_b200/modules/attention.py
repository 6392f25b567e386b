"""The q/k/v split of a fused qkv projection with a one-pass backward.

`split_heads(qkv, heads)` returns what the reference's attention builds with view, permute and
index (Model/ViT/ViT.py:39-42): three [B, heads, T, head_dim] tensors, here strided views of the
projection's output (no copy).  Its backward hands the three gradients of the attention kernel to
`act_merge_heads`, which writes the gradient of the projection's output directly; autograd's own
route is a stack of the three followed by a strided copy of the result."""
from __future__ import annotations

import ctypes

import torch
from torch.autograd import Function

from .. import _lib


def _merge_heads(grads, B, H, T, Dh, dtype, device):
    out = torch.empty((B, T, len(grads) * H * Dh), dtype=dtype, device=device)
    ptrs = (ctypes.c_void_p * len(grads))(*[g.data_ptr() for g in grads])
    strides = (ctypes.c_int64 * (3 * len(grads)))(*[s for g in grads for s in (g.stride(0), g.stride(1), g.stride(2))])
    with _lib.device_of(out):
        rc = _lib.load().act_merge_heads(ptrs, strides, len(grads), B, H, T, Dh, out.element_size(), out.data_ptr(),
                                         _lib.stream_ptr(out))
    _lib.check(rc, "act_merge_heads")
    return out


def _mergeable(g, Dh):
    es = g.element_size()
    return (g.stride(3) == 1 and g.data_ptr() % 16 == 0 and (Dh * es) % 16 == 0
            and all((g.stride(i) * es) % 16 == 0 for i in range(3)))


class _SplitHeads(Function):
    @staticmethod
    def forward(ctx, qkv, heads):
        B, T, D3 = qkv.shape
        Dh = D3 // (3 * heads)
        ctx.dims = (B, heads, T, Dh)
        return qkv.view(B, T, 3, heads, Dh).permute(2, 0, 3, 1, 4).unbind(0)

    @staticmethod
    def backward(ctx, dq, dk, dv):
        B, H, T, Dh = ctx.dims
        ref = next(g for g in (dq, dk, dv) if g is not None)
        grads = [g if g is not None else torch.zeros((B, H, T, Dh), dtype=ref.dtype, device=ref.device)
                 for g in (dq, dk, dv)]
        if all(g.dtype == ref.dtype for g in grads) and ref.element_size() in (2, 4) \
                and all(_mergeable(g, Dh) for g in grads):
            return _merge_heads(grads, B, H, T, Dh, ref.dtype, ref.device), None
        return torch.stack(grads, 0).permute(1, 3, 0, 2, 4).reshape(B, T, 3 * H * Dh), None


def split_heads(qkv: torch.Tensor, heads: int):
    """q, k, v of shape [B, heads, T, head_dim] from the [B, T, 3 * heads * head_dim] output of a fused
    projection, as views.  On a CUDA tensor that needs a gradient the backward is one gather pass.
    A model that is traced with torch.fx registers the name it imports this under with
    `torch.fx.wrap("split_heads")`, so that the trace keeps the call instead of its branches."""
    B, T, D3 = qkv.shape
    if qkv.is_cuda and qkv.requires_grad and qkv.is_contiguous():
        return _SplitHeads.apply(qkv, heads)
    return qkv.view(B, T, 3, heads, D3 // (3 * heads)).permute(2, 0, 3, 1, 4).unbind(0)
