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
planes (three words per 32 elements, bit l of word p = bit p of the code of element l).
`pack_mixed_precision_cuda` / `unpack_mixed_precision_cuda` (caller-supplied min/max) do keep
the reference's ballot-plane layout, reciprocal scale and index hash; `copy_launch` is its
debugging copy with a bounds check.
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


_rng_calls = 0


def pack_mixed_precision_cuda(data: torch.Tensor, min: torch.Tensor, max: torch.Tensor, bits: int,
                              stochastic: bool = True, seed: int | None = None, ref_bias: bool = False):
    """data [N, G, gs] with caller-supplied min / max [N, G] in data's dtype ->
    (packed int32 [N*G*(gs/32)*bits], scale [N, G, 1]); the reference's signature
    (cpp_extension/src/quantization_cuda_kernels.cu:111-195) plus two trailing keywords.
    The words are bit planes in the reference's warp-ballot order and the noise is its index
    hash, so the bytes are those its kernel writes for the same seed, up to the last-bit
    freedom its fast-math build has.  The reference draws the seed from PyTorch's CUDA
    generator; here it is `seed`, or a per-call counter mixed with codec's seed.  `stochastic`
    is accepted and, as in the reference's kernel, not consulted.  `ref_bias=True` keeps the
    reference's extra -0.5 (its noise is already centred, so that biases codes down)."""
    global _rng_calls
    if not data.is_cuda:
        raise RuntimeError("data must be a CUDA tensor: there is no CPU path")
    N, G, gs = data.shape
    data = data.contiguous()
    mn, mx = min.to(data.dtype).contiguous(), max.to(data.dtype).contiguous()
    if mn.numel() != N * G or mx.numel() != N * G:
        raise ValueError("min and max must have one entry per group")
    if seed is None:
        _rng_calls += 1
        seed = codec._mix64(codec._stream_seed() + _rng_calls)
    packed = torch.empty(N * G * ((gs + 31) // 32) * bits, dtype=torch.int32, device=data.device)
    scale = torch.empty((N, G, 1), dtype=data.dtype, device=data.device)
    lib = codec._lib.load()
    with codec._device_of(data):
        rc = lib.act_pack_ballot(data.data_ptr(), codec._DTYPES[data.dtype], N * G, gs, bits, mn.data_ptr(), mx.data_ptr(),
                                 seed & 0xFFFFFFFFFFFFFFFF, codec._lib.ACT_FLAG_BALLOT_REF_BIAS if ref_bias else 0,
                                 packed.data_ptr(), scale.data_ptr(), codec._stream_ptr(data))
    codec._lib.check(rc, "act_pack_ballot")
    return packed, scale


def unpack_mixed_precision_cuda(data: torch.Tensor, bits: int, scale: torch.Tensor, min: torch.Tensor,
                                N: int, num_groups: int, group_size: int) -> torch.Tensor:
    """Inverse of pack_mixed_precision_cuda: [N, num_groups, group_size] in scale's dtype
    (cpp_extension/src/quantization_cuda_kernels.cu:248-298)."""
    if not data.is_cuda:
        raise RuntimeError("data must be a CUDA tensor: there is no CPU path")
    scale = scale.contiguous()
    mn = min.to(scale.dtype).contiguous()
    y = torch.empty((N, num_groups, group_size), dtype=scale.dtype, device=data.device)
    lib = codec._lib.load()
    with codec._device_of(data):
        rc = lib.act_unpack_ballot(data.contiguous().data_ptr(), scale.data_ptr(), mn.data_ptr(), codec._DTYPES[scale.dtype],
                                   N * num_groups, group_size, bits, y.data_ptr(), codec._stream_ptr(data))
    codec._lib.check(rc, "act_unpack_ballot")
    return y


def copy_launch(input: torch.Tensor, fake_unpack: torch.Tensor, N: int, G: int) -> None:
    """The reference's debugging copy (cpp_extension/src/copy.cu:50-102): N*G groups of 256
    elements from `input` to `fake_unpack`, here with the bounds check it lacks."""
    if input.dtype != fake_unpack.dtype:
        raise TypeError("input and fake_unpack must have the same dtype")
    nbytes = N * G * 256 * input.element_size()
    lib = codec._lib.load()
    src, dst = input.contiguous(), fake_unpack
    if not dst.is_contiguous():
        raise ValueError("fake_unpack must be contiguous")
    with codec._device_of(src):
        rc = lib.act_copy(src.data_ptr(), dst.data_ptr(), nbytes, src.numel() * src.element_size(),
                          dst.numel() * dst.element_size(), codec._stream_ptr(src))
    codec._lib.check(rc, "act_copy")


def min_max_kernel(data: torch.Tensor):
    return codec.minmax(data)


def calc_precision(b, C, w, target):
    return codec.calc_precision(b, C, w, float(target))
