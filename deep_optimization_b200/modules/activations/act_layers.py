"""Drop-in activation modules (Activation_Compression/modules/activations/act_layers.py:7-50).
In eval mode they are the stock modules; in training they save compressed state.
`DOGELU` derives from nn.GELU (the reference derives it from nn.SiLU, which makes
its eval mode compute SiLU)."""
from torch import nn

from ... import codec
from .act_ops import _DOMaxPool2d, _DOGELU, _DOReLU, _DOSiLU


class DOReLU_Variance(nn.ReLU):
    def __init__(self, inplace=False, relu=True, relu6=False, target_name=None, meta={}):
        super().__init__(inplace=inplace)
        self.target_name, self.meta, self.relu, self.relu6 = target_name, meta, relu, relu6

    def forward(self, x):
        if self.training:
            return _DOReLU.apply(x, self.relu, self.relu6, self.target_name, self.meta)
        if self.relu6 and not self.relu:
            return nn.functional.relu6(x)
        return super().forward(x)


class DOSiLU(nn.SiLU):
    def __init__(self, inplace=False, target_name=None, meta={}):
        super().__init__(inplace=inplace)
        self.target_name, self.meta = target_name, meta

    def forward(self, x):
        if self.training:
            return _DOSiLU.apply(x, self.target_name, self.meta)
        return super().forward(x)


class DOGELU(nn.GELU):
    """`approximate` ("tanh", the reference's only form and the default here, or "none") is an
    addition to the reference's constructor: the Controller passes the replaced module's own
    setting, so swapping an nn.GELU() does not change the function the model computes."""

    def __init__(self, inplace=False, target_name=None, meta={}, approximate="tanh"):
        super().__init__(approximate=approximate)
        self.target_name, self.meta = target_name, meta

    def forward(self, x):
        if self.training:
            return _DOGELU.apply(x, self.target_name, self.meta, self.approximate == "none")
        return super().forward(x)


def _square(v):
    if isinstance(v, (tuple, list)):
        return v[0] if len(set(v)) == 1 else None
    return v


class DOMaxPool2d(nn.MaxPool2d):
    """nn.MaxPool2d that, in training on a channels-last activation, saves a 4-bit argmax per
    output instead of PyTorch's int64 index (an extension: the reference leaves pooling to
    PyTorch).  Any other case (NCHW memory, dilation, ceil_mode, return_indices, windows above
    4 x 4, channel counts that are not multiples of 8) is the stock operator."""

    def forward(self, x):
        k, s, p = _square(self.kernel_size), _square(self.stride if self.stride is not None else self.kernel_size), \
            _square(self.padding)
        if (self.training and x.requires_grad and not self.ceil_mode and not self.return_indices
                and _square(self.dilation) == 1 and None not in (k, s, p) and codec.maxpool_supported(x, k, s, p)):
            return _DOMaxPool2d.apply(x, k, s, p)
        return super().forward(x)
