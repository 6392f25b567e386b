"""Seeded synthetic activations shared by the parity tests and the bench.

They take the shapes and value distributions of the evaluation configurations
(ReLU(N(0,1)) conv activations, GELU(N(0,1)) transformer activations) and stand
in for real datasets, which are not available offline.
"""
from __future__ import annotations

import numpy as np
import torch


def relu_normal(shape, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.relu(torch.randn(shape, generator=g, dtype=torch.float32)).to(dtype)


def gelu_normal(shape, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.nn.functional.gelu(torch.randn(shape, generator=g, dtype=torch.float32)).to(dtype)


def uniform_noise(shape, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(shape, generator=g, dtype=torch.float32)


def to_numpy(t: torch.Tensor):
    """(array, dtype tag) in the form the oracle takes; bf16 travels as uint16 bits."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16), "bf16"
    if t.dtype == torch.float16:
        return t.numpy(), "f16"
    return t.numpy(), "f32"


def adversarial_groups(group_size: int, dtype=torch.float32) -> torch.Tensor:
    """Groups that exercise the degenerate and slow paths: constant groups, signed
    zeros, denormal ranges, huge ranges, infinities and NaN."""
    rows = []
    g = torch.Generator().manual_seed(7)
    base = torch.randn(group_size, generator=g)
    rows.append(torch.zeros(group_size))                       # all +0
    rows.append(torch.full((group_size,), 3.25))               # constant
    z = torch.zeros(group_size); z[1::2] = -0.0; rows.append(z)  # +-0 mix
    rows.append(base * 1e-41)                                  # denormal range
    rows.append(base * 1e-30)                                  # tiny normal range
    rows.append(base * 1e30)                                   # huge range
    rows.append(base.abs() * 3e38 * torch.sign(base))          # range overflows to inf
    r = base.clone(); r[3] = float("inf"); rows.append(r)
    r = base.clone(); r[5] = float("-inf"); rows.append(r)
    r = base.clone(); r[group_size - 1] = float("nan"); rows.append(r)
    r = base.clone(); r[0] = 1e4; rows.append(r)               # one outlier
    rows.append(torch.linspace(-1, 1, group_size))             # exact ladder
    rows.append(torch.arange(group_size, dtype=torch.float32) % 4)  # values on code points
    return torch.stack(rows).to(dtype)
