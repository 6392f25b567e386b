"""BatchNorm Function that saves the normalised activation compressed.

Forward: per-channel batch statistics (fp32), x_hat = (x - mean) * invstd,
y = x_hat * weight + bias (optionally + residual, optionally ReLU); x_hat is stored through
the codec.  Backward: dgamma = sum(dy * x_hat), dbeta = sum(dy),
dx = weight * invstd / M * (M * dy - dbeta - x_hat * dgamma).
Argument order and saved tensors follow
Activation_Compression/modules/normalization/normalization_ops.py:10-171.  Single-GPU batches
of supported shapes (NCHW with HW a multiple of 4, or channels-last with C a multiple of 8) run
on the library's fused kernels, one call per direction (`codec.bn_forward`, `codec.bn_backward`);
other shapes use PyTorch's native batch-norm kernels around the stand-alone codec, and the SyncBN
variant all-gathers (mean, invstd, count) per rank as normalization_ops.py:181-195 does.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch.amp import custom_bwd, custom_fwd
from torch.autograd import Function

from ... import _lib, act_kernels, codec
from ..module_utils import unified_dequantize, unified_quantize


def sync_batch_stats(mean, var, count, process_group, world_size):
    """Combine per-rank (mean, biased var, count) into the statistics of the global batch
    with one all-gather of 2C+1 floats per rank (normalization_ops.py:181-195 of the
    reference gathers mean, invstd and count the same way).  Returns (mean, var, total)."""
    local = torch.cat([mean, var + mean * mean, mean.new_tensor([float(count)])])
    gathered = [torch.empty_like(local) for _ in range(world_size)]
    dist.all_gather(gathered, local, group=process_group)
    g = torch.stack(gathered)
    C = mean.numel()
    counts = g[:, -1:]
    total = counts.sum()
    mean_all = (g[:, :C] * counts).sum(0) / total
    var_all = (g[:, C:2 * C] * counts).sum(0) / total - mean_all * mean_all
    return mean_all, var_all, total


def _channel_view(t):
    return [1, -1] + [1] * (t.dim() - 2)


class _DOBatchNorm(Function):
    """Forward: batch statistics, x_hat = (x - mean) * invstd, y = x_hat * w + b; x_hat goes to
    the codec.  Backward from the decoded x_hat only.  Single-GPU batches use PyTorch's native
    batch-norm kernels for the statistics and the two normalisations (x_hat is batch norm
    without affine; in backward x_hat is handed to the native backward as an input whose mean
    is 0 and inverse deviation 1, and the result is scaled by the true inverse deviation)."""

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, input, weight, bias, running_mean, running_var, exponential_average_factor,
                eps, target_name, meta, ema_grad_meta, process_group=None, world_size=1, fuse_relu=False,
                residual=None, fork=False):
        # fuse_relu (not in the reference's argument list): the module's output is
        # relu(batch_norm(x)); on the fused path the same three kernels do it and keep the mask.
        # residual (with fuse_relu): the output is relu(batch_norm(x) + residual), the end of a
        # residual block; its gradient is dy under the ReLU mask.
        # fork (with a residual): the output is returned twice (the second a view of the first) for
        # a graph in which it has two consumers; backward then receives their two gradients
        # separately and sums them inside the mask pass it runs anyway, instead of autograd adding
        # them with a pass of its own.
        ctx.set_materialize_grads(False)
        ctx.relu_mask = False
        ctx.has_residual = residual is not None
        ctx.fork = bool(fork)
        if residual is not None and not fuse_relu:
            raise ValueError("a residual is fused only together with the ReLU")
        C = input.shape[1]
        shape = _channel_view(input)
        count = input.numel() // C
        m = meta[f"{target_name}"]
        ctx.fused = None
        if (world_size == 1 and not m["act_padding"] and not m.get("AVG_ALAM", False)
                and codec.bn_fused_supported(input, m["group_size"])):
            # fused path: one statistics pass, then normalise + affine + x_hat codec in one kernel
            # (normalization_ops.py:71-98 of the reference: bn_fwd_reduce + bn_fwd_norm_quant_pack_fused)
            # a channels-last activation is normalised and grouped as it lies in memory
            ctx.channels_last = codec.is_channels_last(input) and C % 8 == 0
            x = input if ctx.channels_last else input.contiguous()
            f32 = lambda t: None if t is None else (t if t.dtype == torch.float32 else t.float())
            rm, rv = f32(running_mean), f32(running_var)
            flags = _lib.ACT_FLAG_ROUND_NEAREST if act_kernels.get_mode() != "baseline" else 0
            y, packed, scale, mn, params, relu_mask = codec.bn_forward(
                x, eps, f32(weight), f32(bias), rm, rv, exponential_average_factor or 0.0, m["bits"],
                m["group_size"], flags=flags, relu=fuse_relu,
                residual=None if residual is None else residual.to(x.dtype))
            if rm is not running_mean and running_mean is not None:      # running statistics kept in another type
                running_mean.copy_(rm)
                running_var.copy_(rv)
            out = (y, packed, scale, mn, relu_mask)
            ctx.fused = (m["bits"], m["group_size"], count)
            ctx.sync = (process_group, world_size)
            if fuse_relu:
                ctx.relu_mask = True
                ctx.save_for_backward(weight, packed, scale, mn, params, out[4])
            else:
                ctx.save_for_backward(weight, packed, scale, mn, params)
            return (y, y.view_as(y)) if ctx.fork else y
        if world_size == 1:
            # one native kernel: x_hat and the saved statistics (running stats updated in place)
            x_hat, mean, invstd = torch.native_batch_norm(input, None, None, running_mean, running_var,
                                                           True, exponential_average_factor, eps)
        else:
            x = input.float()
            dims = [0] + list(range(2, x.dim()))
            var, mean = torch.var_mean(x, dim=dims, unbiased=False)
            mean, var, total = sync_batch_stats(mean, var, count, process_group, world_size)
            invstd = torch.rsqrt(var + eps)
            x_hat = ((x - mean.view(shape)) * invstd.view(shape)).to(input.dtype)
            if running_mean is not None:
                n = float(total)
                unbiased = var * (n / max(n - 1.0, 1.0))
                running_mean.mul_(1.0 - exponential_average_factor).add_(mean, alpha=exponential_average_factor)
                running_var.mul_(1.0 - exponential_average_factor).add_(unbiased, alpha=exponential_average_factor)
        if weight is not None:
            y = torch.addcmul(bias.to(x_hat.dtype).view(shape), x_hat, weight.to(x_hat.dtype).view(shape))
        else:
            y = x_hat
        q_tensors, q_meta, _ = unified_quantize(x_hat, None, target_name, meta, clamp=False, clamp_alpha=0.0)
        ctx.q_meta = q_meta
        ctx.sync = (process_group, world_size)
        if residual is not None:
            y = y + residual.to(y.dtype)
        if fuse_relu:
            # unfused shapes: plain ReLU behind the codec path, its mask kept as a bool tensor
            keep = y > 0
            y = torch.where(keep, y, torch.zeros_like(y))
            ctx.relu_mask = True
            ctx.save_for_backward(weight, q_tensors[0], q_tensors[1], q_tensors[2], invstd, keep)
        else:
            ctx.save_for_backward(weight, q_tensors[0], q_tensors[1], q_tensors[2], invstd)
        return (y, y.view_as(y)) if ctx.fork else y

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, dy, dy2=None):
        if dy is None:
            dy, dy2 = dy2, None
        mask = None
        if ctx.relu_mask:
            weight, q_out, q_scale, q_min, invstd, mask = ctx.saved_tensors
        else:
            weight, q_out, q_scale, q_min, invstd = ctx.saved_tensors
        process_group, world_size = ctx.sync
        if ctx.fused is not None:
            # two kernels on the packed x_hat: per-channel sums, then dx (normalization_ops.py:145-163)
            bits, gs, count = ctx.fused
            fmt = torch.channels_last if ctx.channels_last else torch.contiguous_format
            dyc = dy.contiguous(memory_format=fmt)
            dyc2 = None
            if dy2 is not None:
                if ctx.has_residual and mask is not None and dy2.dtype == dy.dtype:
                    dyc2 = dy2.contiguous(memory_format=fmt)      # summed inside the mask pass
                else:
                    dyc = dyc + dy2
            # `invstd` is the whole [C, 4] parameter table on this path; with a residual, dy under
            # the mask is the residual's gradient and the batch norm's dy
            dx, dgamma, dbeta, dres = codec.bn_backward(q_out, q_scale, q_min, dyc, mask, ctx.has_residual,
                                                        bits, gs, invstd, count, dy2=dyc2)
            dw = dgamma.to(weight.dtype) if weight is not None else None
            db = dbeta.to(weight.dtype) if weight is not None else None
            return dx, dw, db, None, None, None, None, None, None, None, None, None, None, dres, None
        if dy2 is not None:
            dy = dy + dy2
        if mask is not None:
            dy = torch.where(mask, dy, torch.zeros_like(dy))
        dres = dy if ctx.has_residual else None
        x_hat = unified_dequantize((q_out, q_scale, q_min), ctx.q_meta, None)
        shape = _channel_view(dy)
        C = dy.shape[1]
        if world_size == 1:
            zeros = torch.zeros(C, device=dy.device, dtype=torch.float32)
            ones = torch.ones(C, device=dy.device, dtype=torch.float32)
            w = weight.float() if weight is not None else None
            dx, dgamma, dbeta = torch.ops.aten.native_batch_norm_backward(
                dy.contiguous(), x_hat.to(dy.dtype), w, None, None, zeros, ones, True, 0.0,
                [True, weight is not None, weight is not None])
            dx = dx * invstd.to(dx.dtype).view(shape)
            dw = dgamma.to(weight.dtype) if weight is not None else None
            db = dbeta.to(weight.dtype) if weight is not None else None
            return dx, dw, db, None, None, None, None, None, None, None, None, None, None, dres, None
        g = dy.float()
        x_hat = x_hat.float()
        dims = [0] + list(range(2, g.dim()))
        dgamma = (g * x_hat).sum(dims)
        dbeta = g.sum(dims)
        both = torch.cat([dgamma, dbeta, dgamma.new_tensor([float(g.numel() // C)])])
        dist.all_reduce(both, group=process_group)
        sum_dg, sum_db, M = both[:C], both[C:2 * C], float(both[-1])
        w = weight.float() if weight is not None else torch.ones_like(invstd)
        dx = (w * invstd / M).view(shape) * (M * g - sum_db.view(shape) - x_hat * sum_dg.view(shape))
        dw = dgamma.to(weight.dtype) if weight is not None else None
        db = dbeta.to(weight.dtype) if weight is not None else None
        return dx.to(dy.dtype), dw, db, None, None, None, None, None, None, None, None, None, None, dres, None


class _DOSyncBatchNorm:
    """Entry with the reference's argument order for the cross-rank variant
    (normalization_ops.py:174-340 there); the work is `_DOBatchNorm` with a process group."""

    @staticmethod
    def apply(input, weight, bias, running_mean, running_var, eps, momentum, process_group,
              world_size, target_name, meta, ema_grad_meta):
        return _DOBatchNorm.apply(input, weight, bias, running_mean, running_var, momentum, eps,
                                  target_name, meta, ema_grad_meta, process_group, world_size)


class _DOLayerNorm(Function):
    """LayerNorm that keeps its input compressed.  The reference's swap list has no LayerNorm
    (Activation_Compression/controller.py:87); the evaluation configuration for ViT-B/16 names
    LayerNorm inputs among the compressed activations, so the input goes through the same
    quantise boundary as a Linear input.  Where the layout allows (last dimension a multiple of
    the group size, at most 1024, flat grouping, one of the two fixed-point modes) forward is one
    kernel that normalises and packs the input it has just read, and backward one kernel that
    decodes it in registers; otherwise forward is ATen's kernel followed by `unified_quantize`,
    backward `unified_dequantize`, ATen's dx and this library's parameter gradients.  The per-row
    mean and inverse deviation are kept in fp32 (8 bytes per row)."""

    @staticmethod
    def _fused(input, normalized_shape, m):
        return (len(normalized_shape) == 1 and normalized_shape[0] == input.shape[-1] and input.dim() in (2, 3)
                and not m["pack_only"] and not m["AVG_ALAM"] and act_kernels.get_mode() in ("baseline", "nearest")
                and input.numel() // input.shape[0] % m["group_size"] == 0
                and codec.ln_fused_applies(input, m["group_size"], m["bits"]))

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, input, normalized_shape, weight, bias, eps, target_name, meta, residual=None):
        """`residual`: the layer normalises (and saves) input + residual and returns that sum as a
        second output; backward then takes the sum's other gradient as a second argument."""
        m = meta[f"{target_name}"]
        ctx.normalized_shape = list(normalized_shape)
        ctx.param_dtypes = (None if weight is None else weight.dtype, None if bias is None else bias.dtype)
        ctx.with_residual = residual is not None
        ctx.set_materialize_grads(False)                     # an unused output brings None, not a tensor of zeros
        input = input.contiguous()
        total = None
        fused = _DOLayerNorm._fused(input, ctx.normalized_shape, m)
        if residual is not None:
            residual = residual.contiguous()
            if not (fused and codec.ln_residual_applies(input, residual)):
                input = total = input + residual          # the kernel cannot take the pair: add first
                residual = None
                fused = _DOLayerNorm._fused(input, ctx.normalized_shape, m)
        done = lambda y: (y, total) if ctx.with_residual else y
        if fused:
            flags = _lib.ACT_FLAG_ROUND_NEAREST if act_kernels.get_mode() == "nearest" else 0
            if residual is not None:
                total, y, mean, rstd, packed, scale, mn = codec.ln_fwd_quant_pack(
                    input, weight, bias, eps, m["bits"], m["group_size"], flags=flags, residual=residual)
            else:
                y, mean, rstd, packed, scale, mn = codec.ln_fwd_quant_pack(input, weight, bias, eps, m["bits"],
                                                                           m["group_size"], flags=flags)
            # the tensors and the 14-entry meta `quantize` returns for a flat grouping of this input
            n = input.shape[0]
            G = input.numel() // n // m["group_size"]
            ctx.q_meta = (m["bits"], False, m["group_size"], m["act_padding"], n, G, 0, 0, False, False, False,
                          m["AVG_ALAM"], m["ALAM_BITS"], input.shape)
            ctx.fused = True
            ctx.save_for_backward(packed, scale.view(n, G), mn.view(n, G), mean, rstd, weight, bias)
            return done(y)
        w = None if weight is None else weight.to(input.dtype)
        b = None if bias is None else bias.to(input.dtype)
        # in the input's own type (statistics are fp32 inside the kernel): under autocast the stock
        # module would first copy a bf16 input to fp32 and return fp32, two passes the next
        # layer's cast back to bf16 undoes
        with torch.autocast("cuda", enabled=False):
            y, mean, rstd = torch.ops.aten.native_layer_norm(input, list(normalized_shape), w, b, eps)
        q_tensors, q_meta, _ = unified_quantize(input, None, target_name, meta, clamp=False, clamp_alpha=0.0)
        ctx.q_meta = q_meta
        ctx.fused = False
        ctx.save_for_backward(q_tensors[0], q_tensors[1], q_tensors[2], mean, rstd, weight, bias)
        return done(y)

    @staticmethod
    @custom_bwd(device_type="cuda")
    def backward(ctx, dy, dtotal=None):
        packed, scale, mn, mean, rstd, weight, bias = ctx.saved_tensors
        wants_x = bool(ctx.needs_input_grad[0]) or (ctx.with_residual and bool(ctx.needs_input_grad[7]))
        mask = [wants_x, weight is not None and bool(ctx.needs_input_grad[2]),
                bias is not None and bool(ctx.needs_input_grad[3])]
        if dy is None:                                       # only the sum was used downstream
            return (dtotal if ctx.needs_input_grad[0] else None, None, None, None, None, None, None,
                    dtotal if ctx.with_residual and ctx.needs_input_grad[7] else None)
        dy = dy.contiguous()

        def result(dx, dw, db):
            wd, bd = ctx.param_dtypes
            out = (dx if ctx.needs_input_grad[0] else None, None, dw.to(wd) if mask[1] else None,
                   db.to(bd) if mask[2] else None, None, None, None)
            # the sum's gradient goes to both of its operands
            return out + ((dx if ctx.needs_input_grad[7] else None,) if ctx.with_residual else (None,))

        if ctx.fused and codec.ln_fused_applies(dy, ctx.q_meta[2], ctx.q_meta[0]):
            dy2 = None
            if dtotal is not None:
                dy2 = dtotal.to(dy.dtype).contiguous()
                if dy2.data_ptr() % 16:
                    dy2 = dy2.clone()
            dx, dw, db = codec.ln_bwd_from_packed(dy, packed, scale, mn, ctx.q_meta[0], ctx.q_meta[2], mean, rstd,
                                                  weight, dy2=dy2)
            return result(dx, dw, db)
        x = unified_dequantize((packed, scale, mn), ctx.q_meta, None).to(dy.dtype).contiguous()
        w = None if weight is None else weight.to(dy.dtype)
        b = None if bias is None else bias.to(dy.dtype)
        # the two parameter gradients are column sums over all rows: this library's one-pass
        # reduction (ATen's kernel for them takes 430 us on bf16 [50432, 768], this one about 30);
        # dx stays ATen's
        own_params = (mask[1] or mask[2]) and len(ctx.normalized_shape) == 1 and codec.col_sum_applies(dy) \
            and codec.col_sum_applies(x)
        with torch.autocast("cuda", enabled=False):
            if own_params:
                dx, _, _ = torch.ops.aten.native_layer_norm_backward(dy, x, ctx.normalized_shape, mean, rstd, w, b,
                                                                       [mask[0], False, False])
                dw, db = codec.ln_bwd_params(dy, x, mean, rstd)
            else:
                dx, dw, db = torch.ops.aten.native_layer_norm_backward(dy, x, ctx.normalized_shape, mean, rstd, w, b, mask)
        if dtotal is not None and dx is not None:
            dx = dx + dtotal.to(dx.dtype)
        return result(dx, dw, db)
