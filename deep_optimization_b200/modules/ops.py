"""Save-for-backward autograd Functions of the conv / linear layers.

Each Function runs the stock forward op and stores the layer input compressed
(`unified_quantize`) instead of the tensor itself; backward decompresses it
(`unified_dequantize`) and computes the gradients with the stock gradient ops.
Argument orders, saved-tensor orders and the returned gradient tuples follow
Activation_Compression/modules/ops.py:200-387 (`_DOConvnd`), :390-435
(`_DOConv{1,2,3}d`), :438-540 (`_DOLinear`) and :626-680 (`GroupPACTClampFn`).
The dead experiments of that file (Hadamard, low-rank, LARS updates) are not
carried over.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch.amp import custom_bwd, custom_fwd
from torch.autograd import Function
from torch.nn.modules.utils import _pair, _single, _triple

from .. import codec
from ..gemm import dw_from_packed
from .module_utils import low_pass_upsampled, unified_dequantize, unified_quantize


def _patchify_applies(input, weight, stride, padding, dilation, groups) -> bool:
    """A 2-d convolution whose windows tile the input without overlap (kernel = stride, no padding,
    no dilation, one group): the patch embedding of a vision transformer
    (Model/ViT/ViT.py:13 of the reference).  It is a single GEMM on the patches laid out as rows;
    cuDNN's convolution kernels need 1.9 ms forward and 2 ms backward for ViT-B/16's at batch 256,
    the GEMMs 60 us each and the two layout copies 0.1-0.2 ms."""
    if input.dim() != 4 or weight.dim() != 4 or groups != 1 or not input.is_cuda:
        return False
    kh, kw = weight.shape[2], weight.shape[3]
    return (tuple(_pair(stride)) == (kh, kw) and tuple(_pair(padding)) == (0, 0) and tuple(_pair(dilation)) == (1, 1)
            and kh > 1 and kw > 1 and input.shape[2] % kh == 0 and input.shape[3] % kw == 0
            and input.shape[1] == weight.shape[1])


def _to_patches(x, kh, kw):
    """[B, C, H, W] -> [B * H/kh * W/kw, C * kh * kw], a row per window in the weight's (c, i, j) order."""
    B, C, H, W = x.shape
    return x.reshape(B, C, H // kh, kh, W // kw, kw).permute(0, 2, 4, 1, 3, 5).reshape(B * (H // kh) * (W // kw), C * kh * kw)


class _DOConvnd(Function):
    @staticmethod
    def run_forward(ctx, forward_op, input, weight, learnable_scale, stride=1, padding=0, dilation=1,
                    groups=1, clamp_alpha=3.0, target_name=None, meta=None, ema_grad_meta=None, bias=None):
        # `bias` is an addition to the reference's argument list (its conv Functions call the
        # forward op with bias=None, Activation_Compression/modules/ops.py:271-272, so a biased
        # convolution silently loses its bias when swapped): it rides in the convolution itself
        # and its gradient is the sum of dy over everything but the channel axis
        weight_master = weight
        if torch.is_autocast_enabled("cuda"):
            dt = torch.get_autocast_dtype("cuda")
            input = input.to(dt)
            weight_compute = weight.to(dt)
        else:
            weight_compute = weight_master
            input = input.to(weight_master.dtype)      # e.g. the bf16 output of the PACT clamp in an fp32 model
        m = meta[f"{target_name}"]

        # DIVISION: the input is split into a low-pass part (average pool, kept in e4m3) and the
        # residual above it, and only the residual goes through the codec: its range, hence its
        # quantisation step, is smaller.  Backward adds the two back together.  (The reference
        # quantises the whole input and still adds the low-pass part back, modules/ops.py:253-256
        # with the subtraction commented out, which doubles the low frequencies in dW.)
        input_l = None
        to_save = input.to(torch.bfloat16)
        if m["DIVISION"] is not None and not m["pack_only"] and input.dim() == 4:
            k = min(input.shape[-2], input.shape[-1], m["DIVISION"]["pool_kernel_size"])
            input_l = F.avg_pool2d(to_save, k, stride=k, padding=0).to(torch.float8_e4m3fn)
            to_save = to_save - low_pass_upsampled(input_l, input.shape)

        q_tensors, q_meta, input_l = unified_quantize(to_save, input_l, target_name, meta,
                                                      clamp=True, clamp_alpha=clamp_alpha)
        ctx.meta = stride, padding, dilation, groups, ema_grad_meta, clamp_alpha
        # the weight in its compute type is what backward multiplies with: kept, not re-cast
        ctx.weight_compute = weight_compute if weight_compute is not weight_master else None
        ctx.bias_meta = None if bias is None else (bias.dtype, bias.shape[0])
        ctx.save_for_backward(weight_master, q_tensors[0], q_tensors[1], q_tensors[2], input_l, learnable_scale)
        ctx.q_inputs_meta = q_meta
        bias_compute = None if bias is None else bias.to(weight_compute.dtype)
        ctx.patchify = _patchify_applies(input, weight_compute, stride, padding, dilation, groups)
        if ctx.patchify:
            O, _, kh, kw = weight_compute.shape
            B, _, H, W = input.shape
            y2 = F.linear(_to_patches(input, kh, kw), weight_compute.reshape(O, -1), bias_compute)
            return y2.view(B, H // kh, W // kw, O).permute(0, 3, 1, 2)      # a channels-last [B, O, h, w]
        return forward_op(input, weight_compute, bias=bias_compute, stride=stride, padding=padding,
                          dilation=dilation, groups=groups)

    @staticmethod
    def run_backward(ctx, dy, dim, pad_fn):
        q_meta = ctx.q_inputs_meta
        stride, padding, dilation, groups, _, _ = ctx.meta
        weight_master, q_out, q_scale, q_min, input_l, _ = ctx.saved_tensors
        if ctx.weight_compute is not None:
            weight_compute = ctx.weight_compute
            dy = dy.to(weight_compute.dtype)
        elif torch.is_autocast_enabled("cuda"):
            dy = dy.to(torch.get_autocast_dtype("cuda"))
            weight_compute = weight_master.to(torch.bfloat16)
        else:
            weight_compute = weight_master
        stride, padding, dilation = pad_fn(stride), pad_fn(padding), pad_fn(dilation)

        x = unified_dequantize((q_out, q_scale, q_min), q_meta, input_l)
        x = x.to(weight_compute.dtype)
        dy = dy.to(weight_compute.dtype)
        # one backward call on the real input and weight: the library picks its memory format
        # from them (the torch.nn.grad helpers hand it a strideless placeholder, which turns a
        # channels-last gradient back into NCHW with a copy)
        need_dx, need_dw = bool(ctx.needs_input_grad[0]), bool(ctx.needs_input_grad[1])
        need_db = ctx.bias_meta is not None and bool(ctx.needs_input_grad[11])
        dx = dw = db = None
        if getattr(ctx, "patchify", False):
            O, C, kh, kw = weight_compute.shape
            B, _, H, W = x.shape
            dy2 = dy.permute(0, 2, 3, 1).reshape(-1, O)
            if need_dw:
                dw = dy2.t().mm(_to_patches(x, kh, kw)).view(O, C, kh, kw).to(weight_master.dtype)
            if need_dx:
                dx = dy2.mm(weight_compute.reshape(O, -1)).view(B, H // kh, W // kw, C, kh, kw) \
                    .permute(0, 3, 1, 4, 2, 5).reshape(B, C, H, W)
            if need_db:
                dyc = dy2.contiguous()
                db = (codec.col_sum(dyc) if codec.col_sum_applies(dyc) else dyc.sum(0, dtype=torch.float32)).to(ctx.bias_meta[0])
        elif need_dx or need_dw or need_db:
            dx, dw, db = torch.ops.aten.convolution_backward(
                dy, x, weight_compute, [ctx.bias_meta[1]] if need_db else None, list(stride), list(padding),
                list(dilation), False, [0] * dim, groups, [need_dx, need_dw, need_db])
            dw = dw.to(weight_master.dtype) if need_dw else None
            db = db.to(ctx.bias_meta[0]) if need_db else None
            if not need_dx:
                dx = None
        return dx, dw, None, None, None, None, None, None, None, None, None, db


def _make_conv(dim, fwd_op, pad_fn):
    class _Conv(Function):
        @staticmethod
        @custom_fwd(device_type="cuda")
        def forward(ctx, input, weight, learnable_scale, stride=1, padding=0, dilation=1, groups=1,
                    clamp_alpha=3.0, target_name=None, meta=None, ema_grad_meta=None, bias=None):
            return _DOConvnd.run_forward(ctx, fwd_op, input, weight, learnable_scale, stride=stride,
                                         padding=padding, dilation=dilation, groups=groups,
                                         clamp_alpha=clamp_alpha, target_name=target_name, meta=meta,
                                         ema_grad_meta=ema_grad_meta, bias=bias)

        @staticmethod
        @custom_bwd(device_type="cuda")
        def backward(ctx, dy):
            return _DOConvnd.run_backward(ctx, dy, dim, pad_fn)

    _Conv.__name__ = _Conv.__qualname__ = f"_DOConv{dim}d"
    return _Conv


_DOConv1d = _make_conv(1, F.conv1d, _single)
_DOConv2d = _make_conv(2, F.conv2d, _pair)
_DOConv3d = _make_conv(3, F.conv3d, _triple)


# When set (the default), _DOLinear.backward computes dW with the GEMM that decodes the packed
# input in its operand pipeline (gemm.dw_from_packed) wherever the saved state allows it, instead
# of writing the dequantised input out and multiplying: the same speed as dequantise + cuBLAS on
# the ViT-B/16 layers (0.99-1.07x), no [M, K] temporary, about 1 % on the ViT-B/16 step.
# `set_fused_dw(False)` / config key `fused_dw` switch back.
FUSED_DW = True
FUSED_DW_MIN_ROWS = 1024      # below this many rows of dY the reduction is too short to split over the GPU


def set_fused_dw(on: bool) -> None:
    global FUSED_DW
    FUSED_DW = bool(on)


def _fused_dw_applies(q_meta, input_l, dy2, K) -> bool:
    """The packed tensor is the plain flat grouping of a row-major [M, K] input with fp32 scale
    and minimum: no low-pass residual, no padding, no spatial tiling, no sub-group averaging."""
    (bits, pack_only, group_size, act_padding, _N, _G, _h, _w, pad_elig, reshape_elig, _cm, avg_alam,
     _ab, ori_shape) = q_meta
    return (input_l is None and not pack_only and not act_padding and not pad_elig and not reshape_elig
            and not avg_alam and bits in (1, 2, 4, 8) and K % group_size == 0 and K % 8 == 0
            and dy2.dtype == torch.bfloat16 and dy2.shape[1] % 8 == 0 and ori_shape[-1] == K
            and dy2.shape[0] >= FUSED_DW_MIN_ROWS)


class _DOLinear(Function):
    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, input, weight, clamp_alpha, target_name, meta, ema_grad_meta, bias=None):
        # `bias` is an addition to the reference's argument list (Activation_Compression/
        # modules/ops.py:438-479 computes the product without it): handing it to the GEMM
        # keeps the add in the GEMM's epilogue instead of a broadcast pass over the output
        weight_master = weight
        if torch.is_autocast_enabled("cuda"):
            dt = torch.get_autocast_dtype("cuda")
            input = input.to(dt)
            weight_compute = weight.to(dt)
        else:
            weight_compute = weight_master
        bias_compute = None if bias is None else bias.to(weight_compute.dtype)
        m = meta[f"{target_name}"]

        # DIVISION as in the conv Functions: low-pass part beside the compressed residual
        input_l = None
        to_save = input
        if m["DIVISION"] is not None and input.ndim == 3 and not m["pack_only"]:
            k = min(input.shape[2], m["DIVISION"]["pool_kernel_size"])
            input_l = F.avg_pool1d(input.to(torch.bfloat16), k, stride=k, padding=0)
            to_save = (input.to(torch.bfloat16) - low_pass_upsampled(input_l, input.shape)).to(input.dtype)

        q_tensors, q_meta, input_l = unified_quantize(to_save, input_l, target_name, meta, clamp=True,
                                                      clamp_alpha=clamp_alpha)
        ctx.target_name = target_name
        ctx.q_inputs_meta = q_meta
        ctx.meta = input.shape, ema_grad_meta, clamp_alpha
        ctx.bias_dtype = None if bias is None else bias.dtype
        ctx.save_for_backward(weight_master, q_tensors[0], q_tensors[1], q_tensors[2], input_l)
        return F.linear(input, weight_compute, bias_compute)

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, dy):
        q_meta = ctx.q_inputs_meta
        input_shape, _, _ = ctx.meta
        weight_master, q_out, q_scale, q_min, input_l = ctx.saved_tensors
        # the 16-bit copy of the weight is cast again here rather than kept from forward: keeping
        # it cost 0.18 GB on ViT-B/16 and bought no time
        if torch.is_autocast_enabled("cuda"):
            dt = torch.get_autocast_dtype("cuda")
            weight_compute = weight_master.to(dt)
            dy = dy.to(dt)
        else:
            weight_compute = weight_master
        dy = dy.to(weight_compute.dtype)
        dy2 = dy.reshape(-1, dy.shape[-1])
        dw = dx = db = None
        K = weight_master.shape[1]
        if ctx.needs_input_grad[1] and FUSED_DW and q_scale is not None and q_scale.dtype == torch.float32 \
                and _fused_dw_applies(q_meta, input_l, dy2, K):
            dw = dw_from_packed(dy2, q_out, q_scale, q_min, q_meta[0], q_meta[2], K).to(weight_master.dtype)
        elif ctx.needs_input_grad[1]:
            x = unified_dequantize((q_out, q_scale, q_min), q_meta, input_l).to(weight_compute.dtype)
            x2 = x.reshape(-1, x.shape[-1])
            dw = dy2.T.mm(x2).to(weight_master.dtype)
        if ctx.needs_input_grad[0]:
            dx = dy2.mm(weight_compute).view(*input_shape)
        if ctx.bias_dtype is not None and ctx.needs_input_grad[6]:
            # the bias gradient: column sums of dy in one pass (codec.col_sum) where its layout allows
            dyc = dy2 if dy2.is_contiguous() else None
            if dyc is not None and codec.col_sum_applies(dyc):
                db = codec.col_sum(dyc).to(ctx.bias_dtype)
            else:
                db = dy2.sum(0, dtype=torch.float32).to(ctx.bias_dtype)
        return dx, dw, None, None, None, None, db


class GroupPACTClampFn(Function):
    """clamp(x, -alpha, alpha) whose backward mask (|x| <= alpha) is kept 1 bit per element."""

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, x, alpha, group_size, meta, target_name):
        if torch.is_autocast_enabled("cuda"):
            x = x.to(torch.get_autocast_dtype("cuda"))
        alpha = float(alpha)
        inside = (x.abs() <= alpha).to(torch.int8)
        y = x.clamp(-alpha, alpha).to(torch.bfloat16)
        key = f"{target_name}_clamp"
        clamp_meta = {key: {"bits": 1, "pack_only": True, "group_size": group_size,
                            "act_padding": meta[f"{target_name}"]["act_padding"],
                            "N": meta[f"{target_name}"]["N"], "AVG_ALAM": False, "ALAM_BITS": 0}}
        q_tensors, q_meta, _ = unified_quantize(inside, None, key, clamp_meta, clamp=False, clamp_alpha=alpha)
        ctx.save_for_backward(q_tensors[0])
        ctx.q_meta = q_meta
        return y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, dy):
        (packed,) = ctx.saved_tensors
        mask = unified_dequantize((packed, None, None), ctx.q_meta, None)
        return (dy * mask.to(dy.dtype)).to(torch.bfloat16), None, None, None, None
