"""Mirror of the reference's pybind module `cpp_extension`
(Activation_Compression/cpp_extension/bind.cpp:10-63) on top of the sm_100a library.

Same function names and argument orders, outputs written in place as there:

    pack{1,2,3,4,8}(x[N,G,gs], out, scaler[N,G], min[N*G], beta)
    unpack{1,2,3,4,8}(in, out[N,G,gs], scaler, ema_min, N, G, batchSize)
    min_max_kernel(data[B,N,D]) -> (min[B,N], max[B,N])
    calc_precision(b, C, w, target) -> b

Differences, on purpose: the packed words use this library's layout (code j of a word at
bits [j*b,(j+1)*b)), not the reference's warp-ballot bit planes, and `scaler` holds
(max-min)/(2^b-1) rather than its reciprocal, so data packed here must be unpacked here.
`beta` (an unused EMA coefficient in the reference) is ignored.  3-bit codes are stored as bit
planes (three words per 32 elements, bit l of word p = bit p of the code of element l).  The
ActNN-style `pack_mixed_precision_cuda` / `unpack_mixed_precision_cuda` (caller-supplied
min/max, unused by the reference's Python) are not built and raise NotImplementedError.
"""
from __future__ import annotations

import torch

from . import codec


def _pack(bits, x, out, scaler, min, beta):
    N, G, gs = x.shape
    packed, scale, mn = codec.quant_pack(x, bits, gs, planes3=True)
    out.view(-1)[: packed.numel()].copy_(packed.view(-1))
    scaler.view(-1).copy_(scale.to(scaler.dtype))
    min.view(-1).copy_(mn.to(min.dtype))


def _unpack(bits, inp, out, scaler, ema_min, N, G, batchSize):
    gs = out.shape[-1]
    nwords = N * G * gs * bits // 32
    y = codec.dequant_unpack(inp.view(-1)[:nwords].view(N * G, -1), scaler.reshape(-1).float(),
                             ema_min.reshape(-1).float(), bits, gs, out_dtype=out.dtype, planes3=True)
    out.copy_(y.view_as(out))


def pack1(x, out, scaler, min, beta): _pack(1, x, out, scaler, min, beta)
def pack2(x, out, scaler, min, beta): _pack(2, x, out, scaler, min, beta)
def pack3(x, out, scaler, min, beta): _pack(3, x, out, scaler, min, beta)
def pack4(x, out, scaler, min, beta): _pack(4, x, out, scaler, min, beta)
def pack8(x, out, scaler, min, beta): _pack(8, x, out, scaler, min, beta)
def unpack1(inp, out, scaler, ema_min, N, G, batchSize): _unpack(1, inp, out, scaler, ema_min, N, G, batchSize)
def unpack2(inp, out, scaler, ema_min, N, G, batchSize): _unpack(2, inp, out, scaler, ema_min, N, G, batchSize)
def unpack3(inp, out, scaler, ema_min, N, G, batchSize): _unpack(3, inp, out, scaler, ema_min, N, G, batchSize)
def unpack4(inp, out, scaler, ema_min, N, G, batchSize): _unpack(4, inp, out, scaler, ema_min, N, G, batchSize)
def unpack8(inp, out, scaler, ema_min, N, G, batchSize): _unpack(8, inp, out, scaler, ema_min, N, G, batchSize)


def _not_built(name):
    def f(*args, **kwargs):
        raise NotImplementedError(f"{name} is not built in this backend")
    f.__name__ = name
    return f


pack_mixed_precision_cuda = _not_built("pack_mixed_precision_cuda")
unpack_mixed_precision_cuda = _not_built("unpack_mixed_precision_cuda")
copy_launch = _not_built("copy_launch")


def min_max_kernel(data: torch.Tensor):
    return codec.minmax(data)


def calc_precision(b, C, w, target):
    return codec.calc_precision(b, C, w, float(target))
