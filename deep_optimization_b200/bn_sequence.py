"""The kernel sequence of one fused BatchNorm+ReLU layer, forward and backward, on a random
activation: `python -m deep_optimization_b200.bn_sequence N C H W [reps] [bits] [group] [cl]`
(`cl`: the activation is stored channels-last and the kernels run channel-minor).

A small driver for profilers (one process, a handful of launches): batch statistics,
normalise + ReLU + codec, backward sums, backward constants, dx.
"""
from __future__ import annotations

import sys

import torch

from . import codec


def run(shape, reps: int = 3, bits: int = 2, group: int = 256, dtype=torch.bfloat16,
        channels_last: bool = False) -> torch.Tensor:
    dev = torch.device("cuda")
    N, C, H, W = shape
    fmt = torch.channels_last if channels_last else torch.contiguous_format
    xs = [torch.randn(shape, device=dev).to(dtype).contiguous(memory_format=fmt) for _ in range(reps)]
    dys = [torch.randn(shape, device=dev).to(dtype).contiguous(memory_format=fmt) for _ in range(reps)]
    w, b = torch.ones(C, device=dev), torch.zeros(C, device=dev)
    dx = None
    for x, dy in zip(xs, dys):
        params = codec.bn_stats(x, 1e-5, w, b)
        y, packed, scale, mn, mask = codec.bn_fwd_norm_quant_pack(x, None, None, w, b, bits, group,
                                                                  params=params, relu=True)
        s1, s2 = codec.bn_bwd_reduce(packed, scale, mn, dy, bits, group, mask=mask)
        coef = codec.bn_bwd_coef(s1._base, params, N * H * W)
        dx = codec.bn_bwd_dx(packed, scale, mn, dy, None, None, None, bits, group, mask=mask, coef=coef)
    torch.cuda.synchronize()
    return dx


if __name__ == "__main__":
    cl = "cl" in sys.argv[1:]
    a = [int(v) for v in sys.argv[1:] if v != "cl"]
    if len(a) < 4:
        raise SystemExit(__doc__)
    run(tuple(a[:4]), *(a[4:7]), channels_last=cl)
    print("ok")
