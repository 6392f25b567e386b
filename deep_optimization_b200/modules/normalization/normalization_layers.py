"""Drop-in BatchNorm modules
(Activation_Compression/modules/normalization/normalization_layers.py:8-109)."""
import torch.distributed as dist
from torch import nn

from .normalization_ops import _DOBatchNorm, _DOLayerNorm, _DOSyncBatchNorm


def _ema_factor(mod):
    factor = 0.0 if mod.momentum is None else mod.momentum
    if mod.training and mod.track_running_stats and mod.num_batches_tracked is not None:
        mod.num_batches_tracked.add_(1)
        if mod.momentum is None:
            factor = 1.0 / float(mod.num_batches_tracked)
    return factor


class DOBatchNorm2d(nn.BatchNorm2d):
    def __init__(self, num_features, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True,
                 group=0, target_name=None, meta={}):
        super().__init__(num_features, eps, momentum, affine, track_running_stats)
        self.target_name, self.meta, self.ema_grad_meta = target_name, meta, None
        # set by the Controller when the only consumer is a ReLU: the module then returns
        # relu(batch_norm(x)) and the ReLU node is taken out of the graph
        self.fuse_relu = False
        # set by the Controller where the fused output has exactly two consumers: the module then
        # returns the output twice and its backward adds their two gradients inside its mask pass
        self.fork = False

    def forward(self, x, residual=None):
        # residual: set by the Controller where the graph had relu(batch_norm(x) + residual)
        if not self.training:
            y = super().forward(x)
            if residual is not None:
                y = y + residual
            y = nn.functional.relu(y) if self.fuse_relu else y
            return (y, y) if self.fork else y
        self._check_input_dim(x)
        return _DOBatchNorm.apply(x, self.weight, self.bias, self.running_mean, self.running_var,
                                  _ema_factor(self), self.eps, self.target_name, self.meta,
                                  self.ema_grad_meta, None, 1, self.fuse_relu, residual, self.fork)


class DOSyncBatchNorm2d(nn.SyncBatchNorm):
    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, track_running_stats=True,
                 process_group=None, group=0, target_name=None, meta={}):
        super().__init__(num_features, eps, momentum, affine, track_running_stats, process_group)
        self.target_name, self.meta, self.ema_grad_meta = target_name, meta, None

    def forward(self, x):
        if not self.training:
            return super().forward(x)
        if not x.is_cuda:
            raise ValueError("SyncBatchNorm expected input tensor to be on GPU")
        self._check_input_dim(x)
        factor = _ema_factor(self)
        world_size, group = 1, None
        if dist.is_available() and dist.is_initialized():
            group = self.process_group if self.process_group else dist.group.WORLD
            world_size = dist.get_world_size(group)
        if world_size == 1:
            return _DOBatchNorm.apply(x, self.weight, self.bias, self.running_mean, self.running_var,
                                      factor, self.eps, self.target_name, self.meta, self.ema_grad_meta)
        return _DOSyncBatchNorm.apply(x, self.weight, self.bias, self.running_mean, self.running_var,
                                      self.eps, factor, group, world_size, self.target_name, self.meta,
                                      self.ema_grad_meta)


class DOLayerNorm(nn.LayerNorm):
    """nn.LayerNorm whose input is saved compressed in training (an extension: the reference
    leaves LayerNorm alone).  Eval mode is the stock module."""

    def __init__(self, normalized_shape, eps=1e-5, elementwise_affine=True, bias=True, target_name=None, meta={}):
        super().__init__(normalized_shape, eps, elementwise_affine, bias)
        self.target_name, self.meta = target_name, meta

    def forward(self, x, residual=None):
        """With `residual` the layer normalises s = x + residual and returns (y, s): the Controller
        rewrites `s = a + b; y = norm(s)` into this call, so that the addition happens inside the
        forward kernel and the gradient s receives from its other consumer is added inside the
        backward kernel."""
        if not self.training:
            if residual is None:
                return super().forward(x)
            s = x + residual
            return super().forward(s), s
        if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype):
            s = x + residual                                 # broadcast or promoted: autograd's own addition
            return _DOLayerNorm.apply(s, self.normalized_shape, self.weight, self.bias, self.eps,
                                      self.target_name, self.meta, None), s
        return _DOLayerNorm.apply(x, self.normalized_shape, self.weight, self.bias, self.eps,
                                  self.target_name, self.meta, residual)
