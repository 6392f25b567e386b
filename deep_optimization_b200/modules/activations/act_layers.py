"""Drop-in activation modules (Activation_Compression/modules/activations/act_layers.py:7-50).
In eval mode they are the stock modules; in training they save compressed state.
`DOGELU` derives from nn.GELU (the reference derives it from nn.SiLU, which makes
its eval mode compute SiLU)."""
from torch import nn

from .act_ops import _DOGELU, _DOReLU, _DOSiLU


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
    def __init__(self, inplace=False, target_name=None, meta={}):
        super().__init__(approximate="tanh")
        self.target_name, self.meta = target_name, meta

    def forward(self, x):
        if self.training:
            return _DOGELU.apply(x, self.target_name, self.meta)
        return super().forward(x)
