"""Tensor-level entry to the CUDA codec: thin argument marshalling over the C ABI.

PyTorch supplies device memory and the current stream; every byte of arithmetic
happens in libact_b200.so.  Functions here mirror the four codec operators of
Activation_Compression/act_triton_kernel.py:336-433 with the grouped layout
`[N, G, group_size]` already applied by the caller.
"""
from __future__ import annotations

import contextlib
from typing import Optional, Tuple

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.ACT_DTYPE_F32, torch.bfloat16: _lib.ACT_DTYPE_BF16,
           torch.float16: _lib.ACT_DTYPE_F16}

# successive hash-noise calls draw disjoint counter ranges of one stream
_default_seed = 0x5EED
_next_offset = 0


def manual_seed(seed: int) -> None:
    """Seed of the in-kernel counter hash used when no noise tensor is passed.  In a
    torch.distributed job every rank may pass the same value: the rank is mixed in when
    the seed is used (see `_stream_seed`)."""
    global _default_seed, _next_offset, _seed_for_rank
    _default_seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    _next_offset = 0
    _seed_for_rank = None


_seed_for_rank = None        # (rank, seed mixed with it), computed on first use


def _mix64(z: int) -> int:
    """splitmix64 finaliser (the same mixing function the kernels key their hash with)."""
    z = (z + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 31)


def _stream_seed() -> int:
    """The default seed of this process.  Data-parallel ranks start from the same Python state,
    so with one shared seed they would all draw the same rounding noise per element index and
    their rounding errors would add up across the gradient all-reduce instead of averaging out:
    once a process group exists, the rank is mixed into the seed (rank 0 keeps the plain seed,
    so single-process results do not change)."""
    global _seed_for_rank
    rank = 0
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        rank = torch.distributed.get_rank()
    if _seed_for_rank is None or _seed_for_rank[0] != rank:
        _seed_for_rank = (rank, _default_seed if rank == 0 else _default_seed ^ _mix64(rank))
    return _seed_for_rank[1]


def _bits_consts(bits: int, group_size: int):
    """Same contract as Activation_Compression/act_triton_kernel.py:328-334."""
    if bits not in (1, 2, 4, 8):
        raise ValueError(f"bits must be one of (1,2,4,8). got {bits}")
    vpw = 32 // bits
    return vpw, group_size // vpw, (1 << bits) - 1


def _packed_words(bits: int, group_size: int, planes3: bool) -> int:
    """32-bit words per group.  bits = 3 (stored as bit planes, three words per 32 elements) is
    accepted only from callers that ask for it: the act_lib operators keep the reference's
    bits-in-(1,2,4,8) contract."""
    if bits == 3 and planes3:
        return group_size * 3 // 32
    return _bits_consts(bits, group_size)[1]


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: the codec has no CPU path")


def _stream_ptr(t: torch.Tensor) -> int:
    """Raw handle of PyTorch's current stream on t's device (no Stream object is built)."""
    return torch._C._cuda_getCurrentRawStream(t.device.index)


_NO_SWITCH = contextlib.nullcontext()


def _device_of(t: torch.Tensor):
    """Context that makes t's device current for the launch; free when it already is."""
    if t.device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(t.device)


def quant_pack(x: torch.Tensor, bits: int, group_size: int, noise: Optional[torch.Tensor] = None,
               seed: Optional[int] = None, offset: Optional[int] = None, flags: int = 0,
               clamp_alpha: float = 0.0,
               out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
               planes3: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """x: [..., group_size]-groupable tensor (numel % group_size == 0), fp32/bf16/fp16.
    Returns (packed int32 [NG, group_size*bits/32], scale fp32 [NG], min fp32 [NG]);
    `out` supplies those three buffers instead of allocating them.  planes3=True admits
    bits = 3 (bit-plane layout, the cpp_extension pack3 path)."""
    global _next_offset
    nwords = _packed_words(bits, group_size, planes3)
    _require_cuda(x, "x")
    if x.dtype not in _DTYPES:
        raise TypeError(f"unsupported activation dtype {x.dtype}")
    x = x.contiguous()
    if x.numel() % group_size:
        raise ValueError("numel must be a multiple of group_size")
    ng = x.numel() // group_size
    if out is not None:
        packed, scale, mn = out
        if (packed.dtype != torch.int32 or packed.numel() != ng * nwords or scale.numel() != ng
                or mn.numel() != ng or scale.dtype != torch.float32 or mn.dtype != torch.float32
                or not (packed.is_contiguous() and scale.is_contiguous() and mn.is_contiguous())):
            raise ValueError("out buffers have the wrong size, dtype or layout")
    else:
        packed = torch.empty((ng, nwords), dtype=torch.int32, device=x.device)
        scale = torch.empty((ng,), dtype=torch.float32, device=x.device)
        mn = torch.empty((ng,), dtype=torch.float32, device=x.device)
    if noise is not None:
        _require_cuda(noise, "noise")
        noise = noise.to(torch.float32).contiguous()
        if noise.numel() != x.numel():
            raise ValueError("noise must have as many elements as x")
    if seed is None:
        seed = _stream_seed()
    if offset is None:
        offset = _next_offset
        _next_offset += 1
    with _device_of(x):
        rc = _lib.load().act_quant_pack(
            x.data_ptr(), _DTYPES[x.dtype], ng, group_size, bits,
            noise.data_ptr() if noise is not None else None,
            seed & 0xFFFFFFFFFFFFFFFF, offset & 0xFFFFFFFFFFFFFFFF, flags, float(clamp_alpha),
            packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), _stream_ptr(x))
    _lib.check(rc, "act_quant_pack")
    return packed, scale, mn


def dequant_unpack(packed: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor, bits: int,
                   group_size: int, out_dtype: torch.dtype = torch.bfloat16,
                   out: Optional[torch.Tensor] = None, planes3: bool = False) -> torch.Tensor:
    """Inverse of quant_pack; returns [NG, group_size] of out_dtype (written into `out` if given)."""
    _packed_words(bits, group_size, planes3)
    _require_cuda(packed, "packed")
    packed = packed.contiguous()
    scale = scale.to(torch.float32).contiguous()
    mn = mn.to(torch.float32).contiguous()
    ng = scale.numel()
    if out is not None:
        if out.dtype != out_dtype or out.numel() != ng * group_size or not out.is_contiguous():
            raise ValueError("out buffer has the wrong size, dtype or layout")
        y = out
    else:
        y = torch.empty((ng, group_size), dtype=out_dtype, device=packed.device)
    with _device_of(packed):
        rc = _lib.load().act_dequant_unpack(packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), ng,
                                            group_size, bits, _DTYPES[out_dtype], y.data_ptr(),
                                            _stream_ptr(packed))
    _lib.check(rc, "act_dequant_unpack")
    return y


def quant_pack_avg(x: torch.Tensor, bits: int, group_size: int, avg: int,
                   noise: Optional[torch.Tensor] = None, seed: Optional[int] = None,
                   offset: Optional[int] = None, flags: int = 0, clamp_alpha: float = 0.0
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sub-group averaging (the reference's AVG_ALAM): one code per `avg` consecutive elements.
    Returns (packed int32 [NG, group_size*bits/(32*avg)], scale fp32 [NG], min fp32 [NG])."""
    global _next_offset
    _, nwords, _ = _bits_consts(bits, group_size)
    if avg not in (2, 4, 8) or nwords % avg:
        raise ValueError(f"avg must be 2, 4 or 8 and divide the {nwords} words of a group, got {avg}")
    _require_cuda(x, "x")
    if x.dtype not in _DTYPES:
        raise TypeError(f"unsupported activation dtype {x.dtype}")
    x = x.contiguous()
    if x.numel() % group_size:
        raise ValueError("numel must be a multiple of group_size")
    ng = x.numel() // group_size
    packed = torch.empty((ng, nwords // avg), dtype=torch.int32, device=x.device)
    scale = torch.empty((ng,), dtype=torch.float32, device=x.device)
    mn = torch.empty((ng,), dtype=torch.float32, device=x.device)
    if noise is not None:
        _require_cuda(noise, "noise")
        noise = noise.to(torch.float32).contiguous()
        if noise.numel() != x.numel():
            raise ValueError("noise must have as many elements as x")
    if seed is None:
        seed = _stream_seed()
    if offset is None:
        offset = _next_offset
        _next_offset += 1
    with _device_of(x):
        rc = _lib.load().act_quant_pack_avg(
            x.data_ptr(), _DTYPES[x.dtype], ng, group_size, bits, avg,
            noise.data_ptr() if noise is not None else None,
            seed & 0xFFFFFFFFFFFFFFFF, offset & 0xFFFFFFFFFFFFFFFF, flags, float(clamp_alpha),
            packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), _stream_ptr(x))
    _lib.check(rc, "act_quant_pack_avg")
    return packed, scale, mn


def dequant_unpack_avg(packed: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor, bits: int,
                       group_size: int, avg: int, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Inverse of quant_pack_avg: every code repeated `avg` times, [NG, group_size] of out_dtype."""
    _bits_consts(bits, group_size)
    _require_cuda(packed, "packed")
    packed = packed.contiguous()
    scale = scale.to(torch.float32).contiguous()
    mn = mn.to(torch.float32).contiguous()
    ng = scale.numel()
    y = torch.empty((ng, group_size), dtype=out_dtype, device=packed.device)
    with _device_of(packed):
        rc = _lib.load().act_dequant_unpack_avg(packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), ng,
                                                group_size, bits, avg, _DTYPES[out_dtype], y.data_ptr(),
                                                _stream_ptr(packed))
    _lib.check(rc, "act_dequant_unpack_avg")
    return y


def tiles_supported(x: torch.Tensor, group_size: int) -> bool:
    """4-D contiguous CUDA activations whose group is a square tile of 8, 16 or 32 that divides
    H and W: the shapes quant_pack_tiles / dequant_unpack_tiles take."""
    if x.dim() != 4 or not x.is_cuda or x.dtype not in _DTYPES or not x.is_contiguous():
        return False
    t = {64: 8, 256: 16, 1024: 32}.get(group_size)
    return t is not None and x.shape[2] % t == 0 and x.shape[3] % t == 0 and x.numel() > 0


def quant_pack_tiles(x: torch.Tensor, bits: int, tile: int, seed: Optional[int] = None,
                     offset: Optional[int] = None, flags: int = 0):
    """quant_pack of x [N, C, H, W] grouped into tile x tile spatial blocks, read in place:
    (packed [groups, tile*tile*bits/32], scale [groups], min [groups])."""
    global _next_offset
    gs = tile * tile
    _, nwords, _ = _bits_consts(bits, gs)
    N, C, H, W = x.shape
    groups = N * C * (H // tile) * (W // tile)
    packed = torch.empty((groups, nwords), dtype=torch.int32, device=x.device)
    scale = torch.empty((groups,), dtype=torch.float32, device=x.device)
    mn = torch.empty((groups,), dtype=torch.float32, device=x.device)
    if seed is None:
        seed = _stream_seed()
    if offset is None:
        offset = _next_offset
        _next_offset += 1
    with _device_of(x):
        rc = _lib.load().act_quant_pack_tiles(x.data_ptr(), _DTYPES[x.dtype], N * C, H, W, tile, bits,
                                              seed & 0xFFFFFFFFFFFFFFFF, offset & 0xFFFFFFFFFFFFFFFF, flags,
                                              packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), _stream_ptr(x))
    _lib.check(rc, "act_quant_pack_tiles")
    return packed, scale, mn


def dequant_unpack_tiles(packed: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor, bits: int, tile: int,
                         shape, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Inverse of quant_pack_tiles: the [N, C, H, W] tensor written in place (no permute back)."""
    N, C, H, W = shape
    y = torch.empty((N, C, H, W), dtype=out_dtype, device=packed.device)
    with _device_of(packed):
        rc = _lib.load().act_dequant_unpack_tiles(packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), N * C, H, W,
                                                  tile, bits, _DTYPES[out_dtype], y.data_ptr(), _stream_ptr(packed))
    _lib.check(rc, "act_dequant_unpack_tiles")
    return y


def pack_bits(x: torch.Tensor, bits: int, group_size: int) -> torch.Tensor:
    """int8 [NG*group_size] -> int32 words (mask / ready-made code packing)."""
    _, nwords, _ = _bits_consts(bits, group_size)
    _require_cuda(x, "x")
    x = x.to(torch.int8).contiguous()
    ng = x.numel() // group_size
    packed = torch.empty((ng, nwords), dtype=torch.int32, device=x.device)
    with _device_of(x):
        rc = _lib.load().act_pack_bits(x.data_ptr(), ng, group_size, bits, packed.data_ptr(),
                                       _stream_ptr(x))
    _lib.check(rc, "act_pack_bits")
    return packed


def unpack_bits(packed: torch.Tensor, bits: int, n_groups: int, group_size: int) -> torch.Tensor:
    _bits_consts(bits, group_size)
    _require_cuda(packed, "packed")
    packed = packed.contiguous()
    y = torch.empty((n_groups, group_size), dtype=torch.int8, device=packed.device)
    with _device_of(packed):
        rc = _lib.load().act_unpack_bits(packed.data_ptr(), n_groups, group_size, bits,
                                         y.data_ptr(), _stream_ptr(packed))
    _lib.check(rc, "act_unpack_bits")
    return y


def minmax(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row (min, max) over the last dimension of a 2-D or 3-D tensor
    (Activation_Compression/cpp_extension/src/min_max_kernel.cu:114-141)."""
    _require_cuda(x, "x")
    x = x.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols
    mn = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    mx = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    with _device_of(x):
        rc = _lib.load().act_minmax(x.data_ptr(), _DTYPES[x.dtype], rows, cols, mn.data_ptr(),
                                    mx.data_ptr(), _stream_ptr(x))
    _lib.check(rc, "act_minmax")
    return mn, mx


def calc_precision(b: torch.Tensor, C: torch.Tensor, w: torch.Tensor, target: float) -> torch.Tensor:
    """Greedy bit allocation on CPU int32 tensors, in place on b
    (Activation_Compression/cpp_extension/src/calc_precision.cc:10-53)."""
    for t, n in ((b, "b"), (C, "C"), (w, "w")):
        if t.device.type != "cpu" or not t.is_contiguous() or t.dtype != torch.int32:
            raise RuntimeError(f"{n} must be a contiguous CPU int32 tensor")
    rc = _lib.load().act_calc_precision(b.data_ptr(), C.data_ptr(), w.data_ptr(), b.numel(),
                                        float(target))
    _lib.check(rc, "act_calc_precision")
    return b


# ---------------------------------------------------------------- fused activation kernels

def relu_fwd_pack(x: torch.Tensor, relu6: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """y = relu(x) (or the ReLU6 window) and the 1-bit mask as int32 words, one pass."""
    _require_cuda(x, "x")
    # element-wise: a channels-last tensor is processed as it lies in memory (y and the mask
    # bits follow that order; relu_bwd_unpack must be given dy in the same memory format)
    x = x if is_channels_last(x) else x.contiguous()
    if x.numel() % 32:
        raise ValueError("numel must be a multiple of 32")
    y = torch.empty_like(x)
    bits = torch.empty((x.numel() // 32,), dtype=torch.int32, device=x.device)
    with _device_of(x):
        rc = _lib.load().act_relu_fwd_pack(x.data_ptr(), _DTYPES[x.dtype], x.numel(), int(relu6),
                                           y.data_ptr(), bits.data_ptr(), _stream_ptr(x))
    _lib.check(rc, "act_relu_fwd_pack")
    return y, bits


def relu_bwd_unpack(mask_bits: torch.Tensor, dy: torch.Tensor, channels_last: bool = False) -> torch.Tensor:
    """dx = mask ? dy : 0.  `channels_last`: the mask was taken from a channels-last tensor, so
    dy is walked (after a conversion if it arrives in another format) in that memory order."""
    _require_cuda(dy, "dy")
    if channels_last or is_channels_last(dy):
        dy = dy.contiguous(memory_format=torch.channels_last)
    else:
        dy = dy.contiguous()
    dx = torch.empty_like(dy)
    with _device_of(dy):
        rc = _lib.load().act_relu_bwd_unpack(mask_bits.data_ptr(), dy.data_ptr(), _DTYPES[dy.dtype],
                                             dy.numel(), dx.data_ptr(), _stream_ptr(dy))
    _lib.check(rc, "act_relu_bwd_unpack")
    return dx


def activation_fwd_quant_pack(x: torch.Tensor, kind: str, bits: int, group_size: int,
                              seed: Optional[int] = None, offset: Optional[int] = None, flags: int = 0):
    """y = act(x) and the packed derivative: (y, packed, scale, min).  kind: "gelu" (tanh
    approximation), "gelu_erf" (exact) or "silu"."""
    global _next_offset
    _, nwords, _ = _bits_consts(bits, group_size)
    _require_cuda(x, "x")
    x = x.contiguous()
    if x.numel() % group_size:
        raise ValueError("numel must be a multiple of group_size")
    ng = x.numel() // group_size
    y = torch.empty_like(x)
    packed = torch.empty((ng, nwords), dtype=torch.int32, device=x.device)
    scale = torch.empty((ng,), dtype=torch.float32, device=x.device)
    mn = torch.empty((ng,), dtype=torch.float32, device=x.device)
    if seed is None:
        seed = _stream_seed()
    if offset is None:
        offset = _next_offset
        _next_offset += 1
    k = {"gelu": _lib.ACT_KIND_GELU, "silu": _lib.ACT_KIND_SILU, "gelu_erf": _lib.ACT_KIND_GELU_ERF}[kind]
    with _device_of(x):
        rc = _lib.load().act_activation_fwd_quant_pack(
            x.data_ptr(), _DTYPES[x.dtype], k, ng, group_size, bits, seed & 0xFFFFFFFFFFFFFFFF,
            offset & 0xFFFFFFFFFFFFFFFF, flags, y.data_ptr(), packed.data_ptr(), scale.data_ptr(),
            mn.data_ptr(), _stream_ptr(x))
    _lib.check(rc, "act_activation_fwd_quant_pack")
    return y, packed, scale, mn


def mul_dequant_unpack(packed: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor, dy: torch.Tensor,
                       bits: int, group_size: int) -> torch.Tensor:
    """dx = dy * (code * scale + min): backward of an activation whose derivative was packed."""
    _bits_consts(bits, group_size)
    _require_cuda(dy, "dy")
    dy = dy.contiguous()
    dx = torch.empty_like(dy)
    with _device_of(dy):
        rc = _lib.load().act_mul_dequant_unpack(packed.data_ptr(), scale.data_ptr(), mn.data_ptr(),
                                                dy.data_ptr(), _DTYPES[dy.dtype], dy.numel() // group_size,
                                                group_size, bits, dx.data_ptr(), _stream_ptr(dy))
    _lib.check(rc, "act_mul_dequant_unpack")
    return dx


# ---------------------------------------------------------------- fused batch-norm kernels

def is_channels_last(x: torch.Tensor) -> bool:
    """True for a 4-D tensor stored channel-minor (NHWC memory) and not also NCHW-contiguous."""
    return (x.dim() == 4 and not x.is_contiguous()
            and x.is_contiguous(memory_format=torch.channels_last))


def _bn_layout(x: torch.Tensor):
    """(tensor whose storage the kernels walk, n_batch, C, hw) of a batch-norm operand.  A
    channels-last tensor is taken as it lies in memory, [N*H*W, C] with hw = 1 (the kernels'
    channel-minor layout); anything else as contiguous [N, C, HW]."""
    C = x.shape[1]
    if is_channels_last(x) and C % 8 == 0:
        return x, x.numel() // C, C, 1
    x = x.contiguous()
    return x, x.shape[0], C, x.numel() // (x.shape[0] * C)


def bn_fused_supported(x: torch.Tensor, group_size: int) -> bool:
    """Shapes the fused batch-norm kernels take: [N, C, ...] with HW a multiple of 4, or a
    channels-last [N, C, H, W] with C a multiple of 8 (groups then run over NHWC memory)."""
    if x.dim() < 3 or not x.is_cuda or x.dtype not in _DTYPES:
        return False
    C = x.shape[1]
    if is_channels_last(x) and C % 8 == 0:
        return C <= 4096 and x.numel() % group_size == 0
    hw = x.numel() // (x.shape[0] * C)
    return (hw % 4 == 0 and hw * (hw + 1024) < 2 ** 32 and C <= 4096
            and x.numel() % group_size == 0)


def bn_stats(x: torch.Tensor, eps: float, weight: Optional[torch.Tensor] = None,
             bias: Optional[torch.Tensor] = None, running_mean: Optional[torch.Tensor] = None,
             running_var: Optional[torch.Tensor] = None, momentum: float = 0.0) -> torch.Tensor:
    """Batch statistics of x [N, C, ...]: the fp32 [C, 4] table (mean, 1/sqrt(var+eps), weight,
    bias) that bn_fwd_norm_quant_pack reads; fp32 running statistics are updated in place."""
    x, N, C, hw = _bn_layout(x)

    def f32(t):
        if t is None:
            return None
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError("bn_stats takes contiguous fp32 parameters and running statistics")
        return t

    weight, bias, running_mean, running_var = f32(weight), f32(bias), f32(running_mean), f32(running_var)
    lib = _lib.load()
    params = torch.empty((C, 4), dtype=torch.float32, device=x.device)
    ws_bytes = int(lib.act_bn_stats_workspace(N, C))
    ws = torch.empty((max(ws_bytes, 4) // 4,), dtype=torch.float32, device=x.device)
    ptr = lambda t: None if t is None else t.data_ptr()
    with _device_of(x):
        rc = lib.act_bn_stats(x.data_ptr(), _DTYPES[x.dtype], N, C, hw, float(eps), ptr(weight), ptr(bias),
                              ptr(running_mean), ptr(running_var), float(momentum), params.data_ptr(),
                              ws.data_ptr(), ws_bytes, _stream_ptr(x))
    _lib.check(rc, "act_bn_stats")
    return params


def bn_fwd_norm_quant_pack(x: torch.Tensor, mean: Optional[torch.Tensor], invstd: Optional[torch.Tensor],
                           weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], bits: int,
                           group_size: int, seed: Optional[int] = None, offset: Optional[int] = None,
                           flags: int = 0, params: Optional[torch.Tensor] = None, relu: bool = False,
                           residual: Optional[torch.Tensor] = None):
    """y = (x - mean) * invstd * weight + bias and the packed x_hat: (y, packed, scale, min).
    `params` is bn_stats' table; without it the table is built from mean, invstd, weight, bias.
    relu=True also applies y = max(y, 0) and returns the 1-bit ReLU mask as a fifth value;
    with `residual` (x's shape, type and memory format) y = max(y + residual, 0)."""
    global _next_offset
    _, nwords, _ = _bits_consts(bits, group_size)
    x, N, C, hw = _bn_layout(x)
    if params is None:
        ones = torch.ones_like(mean) if weight is None else weight.float()
        zeros = torch.zeros_like(mean) if bias is None else bias.float()
        params = torch.stack([mean.float(), invstd.float(), ones, zeros], dim=1).contiguous()
    ng = x.numel() // group_size
    y = torch.empty_like(x)
    packed = torch.empty((ng, nwords), dtype=torch.int32, device=x.device)
    scale = torch.empty((ng,), dtype=torch.float32, device=x.device)
    mn = torch.empty((ng,), dtype=torch.float32, device=x.device)
    if seed is None:
        seed = _stream_seed()
    if offset is None:
        offset = _next_offset
        _next_offset += 1
    if residual is not None:
        if not relu:
            raise ValueError("the residual add is fused together with the ReLU only")
        if residual.shape != x.shape or residual.dtype != x.dtype:
            raise ValueError("residual must have x's shape and type")
        residual = residual.contiguous(memory_format=torch.channels_last) if hw == 1 and is_channels_last(x) \
            else residual.contiguous()
        mask = torch.empty((x.numel() // 8,), dtype=torch.uint8, device=x.device)
        with _device_of(x):
            rc = _lib.load().act_bn_add_relu_fwd_norm_quant_pack(
                x.data_ptr(), residual.data_ptr(), _DTYPES[x.dtype], N, C, hw, params.data_ptr(), group_size, bits,
                seed & 0xFFFFFFFFFFFFFFFF, offset & 0xFFFFFFFFFFFFFFFF, flags, y.data_ptr(), packed.data_ptr(),
                scale.data_ptr(), mn.data_ptr(), mask.data_ptr(), _stream_ptr(x))
        _lib.check(rc, "act_bn_add_relu_fwd_norm_quant_pack")
        return y, packed, scale, mn, mask
    if relu:
        mask = torch.empty((x.numel() // 8,), dtype=torch.uint8, device=x.device)
        with _device_of(x):
            rc = _lib.load().act_bn_relu_fwd_norm_quant_pack(
                x.data_ptr(), _DTYPES[x.dtype], N, C, hw, params.data_ptr(), group_size, bits,
                seed & 0xFFFFFFFFFFFFFFFF, offset & 0xFFFFFFFFFFFFFFFF, flags, y.data_ptr(), packed.data_ptr(),
                scale.data_ptr(), mn.data_ptr(), mask.data_ptr(), _stream_ptr(x))
        _lib.check(rc, "act_bn_relu_fwd_norm_quant_pack")
        return y, packed, scale, mn, mask
    with _device_of(x):
        rc = _lib.load().act_bn_fwd_norm_quant_pack(
            x.data_ptr(), _DTYPES[x.dtype], N, C, hw, params.data_ptr(), group_size, bits,
            seed & 0xFFFFFFFFFFFFFFFF, offset & 0xFFFFFFFFFFFFFFFF, flags, y.data_ptr(), packed.data_ptr(),
            scale.data_ptr(), mn.data_ptr(), _stream_ptr(x))
    _lib.check(rc, "act_bn_fwd_norm_quant_pack")
    return y, packed, scale, mn


def bn_bwd_reduce(packed: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor, dy: torch.Tensor, bits: int,
                  group_size: int, mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(sum dy * x_hat, sum dy) per channel, from the packed x_hat; with the fused ReLU's `mask`
    dy counts only where its bit is set."""
    dy, N, C, hw = _bn_layout(dy)
    sums = torch.zeros(2 * C, dtype=torch.float32, device=dy.device)
    lib = _lib.load()
    with _device_of(dy):
        if mask is None:
            rc = lib.act_bn_bwd_reduce(packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), dy.data_ptr(),
                                       _DTYPES[dy.dtype], N, C, hw, group_size, bits, sums.data_ptr(),
                                       _stream_ptr(dy))
        else:
            rc = lib.act_bn_relu_bwd_reduce(packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), dy.data_ptr(),
                                            mask.data_ptr(), _DTYPES[dy.dtype], N, C, hw, group_size, bits,
                                            sums.data_ptr(), _stream_ptr(dy))
    _lib.check(rc, "act_bn_bwd_reduce")
    return sums[:C], sums[C:]          # two views of one [2C] tensor (bn_bwd_coef takes it whole)


def bn_bwd_coef(sums: torch.Tensor, params: torch.Tensor, count: float) -> torch.Tensor:
    """The [C, 4] table (k1, k2, k3, 0) of bn_bwd_dx from bn_bwd_reduce's sums ([2C], or the
    pair it returns) and bn_stats' params."""
    if isinstance(sums, (tuple, list)):
        sums = torch.cat([sums[0], sums[1]])
    sums = sums.contiguous()
    C = params.shape[0]
    coef = torch.empty((C, 4), dtype=torch.float32, device=params.device)
    with _device_of(params):
        rc = _lib.load().act_bn_bwd_coef(sums.data_ptr(), params.data_ptr(), C, float(count), coef.data_ptr(),
                                         _stream_ptr(params))
    _lib.check(rc, "act_bn_bwd_coef")
    return coef


def bn_bwd_dx(packed: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor, dy: torch.Tensor,
              k1: Optional[torch.Tensor], k2: Optional[torch.Tensor], k3: Optional[torch.Tensor], bits: int,
              group_size: int, mask: Optional[torch.Tensor] = None,
              coef: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dx = k1[c] * dy - k2[c] - k3[c] * x_hat (dy zeroed where the fused ReLU's `mask` bit is
    clear); the constants come as three vectors or as bn_bwd_coef's table."""
    dy, N, C, hw = _bn_layout(dy)
    if coef is None:
        coef = torch.stack([k1.float(), k2.float(), k3.float(), torch.zeros_like(k1, dtype=torch.float32)], dim=1).contiguous()
    dx = torch.empty_like(dy)
    lib = _lib.load()
    with _device_of(dy):
        if mask is None:
            rc = lib.act_bn_bwd_dx(packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), dy.data_ptr(),
                                   _DTYPES[dy.dtype], N, C, hw, group_size, bits, coef.data_ptr(),
                                   dx.data_ptr(), _stream_ptr(dy))
        else:
            rc = lib.act_bn_relu_bwd_dx(packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), dy.data_ptr(),
                                        mask.data_ptr(), _DTYPES[dy.dtype], N, C, hw, group_size, bits,
                                        coef.data_ptr(), dx.data_ptr(), _stream_ptr(dy))
    _lib.check(rc, "act_bn_bwd_dx")
    return dx


# ---------------------------------------------------------------- one call per batch-norm layer

_bn_ws_bytes = {}


def bn_forward(x: torch.Tensor, eps: float, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
               running_mean: Optional[torch.Tensor], running_var: Optional[torch.Tensor], momentum: float,
               bits: int, group_size: int, flags: int = 0, relu: bool = False,
               residual: Optional[torch.Tensor] = None, seed: Optional[int] = None,
               offset: Optional[int] = None):
    """bn_stats followed by bn_fwd_norm_quant_pack in one library call (act_bn_forward).
    weight, bias and the running statistics are fp32 (or None).  Returns (y, packed, scale, min,
    params, mask) with mask None unless relu."""
    global _next_offset
    _, nwords, _ = _bits_consts(bits, group_size)
    x, N, C, hw = _bn_layout(x)
    for t in (weight, bias, running_mean, running_var):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise ValueError("bn_forward takes contiguous fp32 parameters and running statistics")
    if residual is not None:
        if not relu:
            raise ValueError("the residual add is fused together with the ReLU only")
        if residual.shape != x.shape or residual.dtype != x.dtype:
            raise ValueError("residual must have x's shape and type")
        residual = residual.contiguous(memory_format=torch.channels_last) if hw == 1 and is_channels_last(x) \
            else residual.contiguous()
    lib = _lib.load()
    key = (N, C)
    ws_bytes = _bn_ws_bytes.get(key)
    if ws_bytes is None:
        ws_bytes = _bn_ws_bytes[key] = int(lib.act_bn_stats_workspace(N, C))
    dev = x.device
    ng = x.numel() // group_size
    params = torch.empty((C, 4), dtype=torch.float32, device=dev)
    ws = torch.empty((max(ws_bytes, 4) // 4,), dtype=torch.float32, device=dev)
    y = torch.empty_like(x)
    packed = torch.empty((ng, nwords), dtype=torch.int32, device=dev)
    meta = torch.empty((2, ng), dtype=torch.float32, device=dev)
    mask = torch.empty((x.numel() // 8,), dtype=torch.uint8, device=dev) if relu else None
    if seed is None:
        seed = _stream_seed()
    if offset is None:
        offset = _next_offset
        _next_offset += 1
    ptr = lambda t: None if t is None else t.data_ptr()
    with _device_of(x):
        rc = lib.act_bn_forward(x.data_ptr(), ptr(residual), _DTYPES[x.dtype], N, C, hw, float(eps), ptr(weight),
                                ptr(bias), ptr(running_mean), ptr(running_var), float(momentum), params.data_ptr(),
                                ws.data_ptr(), ws_bytes, group_size, bits, seed & 0xFFFFFFFFFFFFFFFF,
                                offset & 0xFFFFFFFFFFFFFFFF, flags, y.data_ptr(), packed.data_ptr(),
                                meta[0].data_ptr(), meta[1].data_ptr(), ptr(mask), _stream_ptr(x))
    _lib.check(rc, "act_bn_forward")
    return y, packed, meta[0], meta[1], params, mask


def bn_backward(packed: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor, dy: torch.Tensor,
                mask: Optional[torch.Tensor], has_residual: bool, bits: int, group_size: int,
                params: torch.Tensor, count: float, dy2: Optional[torch.Tensor] = None):
    """bn_bwd_reduce, bn_bwd_coef and bn_bwd_dx in one library call (act_bn_backward_sum), dy being
    in the memory format of the forward input.  Returns (dx, dgamma, dbeta, dy_masked): with
    has_residual, dy under the ReLU mask (the residual's gradient), else None.  dy2 (residual form
    only; dy's shape, type and strides): a second gradient of the output, summed in the mask pass."""
    if dy2 is not None and (not has_residual or mask is None or dy2.shape != dy.shape or dy2.dtype != dy.dtype
                            or dy2.stride() != dy.stride()):
        raise ValueError("bn_backward: dy2 needs the residual form and dy's shape, type and strides")
    dy, N, C, hw = _bn_layout(dy)
    dev = dy.device
    work = torch.empty((6 * C,), dtype=torch.float32, device=dev)      # sums [2C] and coef [C][4]
    dx = torch.empty_like(dy)
    dym = torch.empty_like(dy) if has_residual else None
    with _device_of(dy):
        rc = _lib.load().act_bn_backward_sum(packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), dy.data_ptr(),
                                         None if dy2 is None else dy2.data_ptr(),
                                         None if mask is None else mask.data_ptr(), _DTYPES[dy.dtype], N, C, hw,
                                         group_size, bits, params.data_ptr(), float(count), work.data_ptr(),
                                         work[2 * C:].data_ptr(), None if dym is None else dym.data_ptr(),
                                         dx.data_ptr(), _stream_ptr(dy))
    _lib.check(rc, "act_bn_backward")
    return dx, work[:C], work[C:2 * C], dym


# ---------------------------------------------------------------- max pooling, channels-last

def maxpool_supported(x: torch.Tensor, k: int, s: int, pad: int) -> bool:
    """Channels-last 4-D CUDA activations with C a multiple of 8, window k <= 4, pad <= k/2."""
    return (x.dim() == 4 and x.is_cuda and x.dtype in _DTYPES and is_channels_last(x) and x.shape[1] % 8 == 0
            and 1 <= k <= 4 and s >= 1 and 0 <= 2 * pad <= k and x.shape[2] + 2 * pad >= k and x.shape[3] + 2 * pad >= k)


def maxpool_fwd(x: torch.Tensor, k: int, s: int, pad: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """max_pool2d of a channels-last x: (y channels-last, idx int32 [N*OH*OW*C/8] holding the
    4-bit window position of every maximum)."""
    if not maxpool_supported(x, k, s, pad):
        raise ValueError("maxpool_fwd takes a channels-last CUDA tensor with C % 8 == 0, k <= 4, pad <= k/2")
    N, C, H, W = x.shape
    OH, OW = (H + 2 * pad - k) // s + 1, (W + 2 * pad - k) // s + 1
    y = torch.empty((N, C, OH, OW), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
    idx = torch.empty((N * OH * OW * C // 8,), dtype=torch.int32, device=x.device)
    with _device_of(x):
        rc = _lib.load().act_maxpool_fwd_cl(x.data_ptr(), _DTYPES[x.dtype], N, H, W, C, k, s, pad, y.data_ptr(),
                                            idx.data_ptr(), _stream_ptr(x))
    _lib.check(rc, "act_maxpool_fwd_cl")
    return y, idx


def maxpool_bwd(idx: torch.Tensor, dy: torch.Tensor, input_shape, k: int, s: int, pad: int) -> torch.Tensor:
    """Gradient of maxpool_fwd's input (channels-last) from its idx and dy."""
    N, C, H, W = input_shape
    dy = dy.contiguous(memory_format=torch.channels_last)
    dx = torch.empty((N, C, H, W), dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
    with _device_of(dy):
        rc = _lib.load().act_maxpool_bwd_cl(idx.data_ptr(), dy.data_ptr(), _DTYPES[dy.dtype], N, H, W, C, k, s, pad,
                                            dx.data_ptr(), _stream_ptr(dy))
    _lib.check(rc, "act_maxpool_bwd_cl")
    return dx


# ---------------------------------------------------------------- column reductions

def col_sum_applies(t: torch.Tensor) -> bool:
    """act_col_sum / act_ln_bwd_params take a CUDA tensor of a codec dtype whose rows (last
    dimension, a multiple of 8) are contiguous and packed and whose base is 16-byte aligned."""
    return (t.is_cuda and t.dtype in _DTYPES and t.dim() >= 1 and t.shape[-1] % 8 == 0 and t.shape[-1] > 0
            and t.is_contiguous() and t.data_ptr() % 16 == 0)


def col_sum(a: torch.Tensor) -> torch.Tensor:
    """fp32 [C] = a.reshape(-1, C).sum(0): the bias gradient of a linear layer from its output
    gradient (Activation_Compression/modules/ops.py:496-526), one pass at HBM pace."""
    if not a.is_cuda:
        raise RuntimeError("col_sum needs a CUDA tensor: there is no CPU path")
    C = a.shape[-1]
    a2 = a.reshape(-1, C)
    if not col_sum_applies(a2):
        raise ValueError("col_sum: rows must be contiguous, a multiple of 8 long and 16-byte aligned")
    out = torch.empty(C, dtype=torch.float32, device=a.device)
    with _device_of(a):
        rc = _lib.load().act_col_sum(a2.data_ptr(), _DTYPES[a2.dtype], a2.shape[0], C, out.data_ptr(), _stream_ptr(a))
    _lib.check(rc, "act_col_sum")
    return out


def ln_bwd_params(dy: torch.Tensor, x: torch.Tensor, mean: torch.Tensor, rstd: torch.Tensor):
    """(dgamma, dbeta), fp32 [C]: sum over rows of dy * (x - mean) * rstd and of dy, for a
    LayerNorm over the last dimension; mean and rstd are the fp32 per-row statistics of the
    forward pass."""
    if not dy.is_cuda:
        raise RuntimeError("ln_bwd_params needs CUDA tensors: there is no CPU path")
    C = dy.shape[-1]
    dy2, x2 = dy.reshape(-1, C), x.reshape(-1, C)
    if dy2.dtype != x2.dtype or dy2.shape != x2.shape or not col_sum_applies(dy2) or not col_sum_applies(x2):
        raise ValueError("ln_bwd_params: dy and x must share type and shape, with contiguous aligned rows of a multiple of 8")
    mean = mean.reshape(-1).to(torch.float32).contiguous()
    rstd = rstd.reshape(-1).to(torch.float32).contiguous()
    if mean.numel() != dy2.shape[0] or rstd.numel() != dy2.shape[0]:
        raise ValueError("ln_bwd_params: one mean and one rstd per row")
    dgamma = torch.empty(C, dtype=torch.float32, device=dy.device)
    dbeta = torch.empty(C, dtype=torch.float32, device=dy.device)
    with _device_of(dy):
        rc = _lib.load().act_ln_bwd_params(dy2.data_ptr(), x2.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                           _DTYPES[dy2.dtype], dy2.shape[0], C, dgamma.data_ptr(), dbeta.data_ptr(),
                                           _stream_ptr(dy))
    _lib.check(rc, "act_ln_bwd_params")
    return dgamma, dbeta


# ---------------------------------------------------------------- LayerNorm fused with the codec

def ln_fused_applies(x: torch.Tensor, group_size: int, bits: int) -> bool:
    """act_ln_fwd_quant_pack / act_ln_bwd_from_packed take a contiguous CUDA tensor of a codec
    dtype whose last dimension is a multiple of group_size (32..256) and at most 1024."""
    C = x.shape[-1] if x.dim() else 0
    return (x.is_cuda and x.dtype in _DTYPES and x.dim() >= 2 and x.is_contiguous() and x.data_ptr() % 16 == 0
            and bits in (1, 2, 4, 8) and group_size in (32, 64, 128, 256) and 0 < C <= 1024 and C % group_size == 0)


def ln_residual_applies(x: torch.Tensor, residual: torch.Tensor) -> bool:
    """act_ln_add_fwd_quant_pack forms x + residual itself: both contiguous, one shape, one 16-bit type."""
    return (x.dtype in (torch.bfloat16, torch.float16) and residual.dtype == x.dtype and residual.shape == x.shape
            and residual.is_cuda and residual.device == x.device and residual.is_contiguous()
            and residual.data_ptr() % 16 == 0)


def ln_fwd_quant_pack(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float,
                      bits: int, group_size: int, seed: Optional[int] = None, offset: Optional[int] = None,
                      flags: int = 0, residual: Optional[torch.Tensor] = None):
    """(y, mean, rstd, packed, scale, min): LayerNorm over the last dimension and the packed input,
    the latter identical to quant_pack(x, bits, group_size, seed=seed, offset=offset, flags=flags).
    With `residual` (same shape and 16-bit type) the normalised and packed tensor is
    s = x + residual, rounded to that type, and s is returned first: (s, y, mean, ...)."""
    global _next_offset
    if not x.is_cuda:
        raise RuntimeError("ln_fwd_quant_pack needs a CUDA tensor: there is no CPU path")
    if not ln_fused_applies(x, group_size, bits):
        raise ValueError("ln_fwd_quant_pack: unsupported shape, type or group size")
    if residual is not None and not ln_residual_applies(x, residual):
        raise ValueError("ln_fwd_quant_pack: the residual must be a contiguous 16-bit tensor of x's shape and type")
    C = x.shape[-1]
    rows = x.numel() // C
    ng = x.numel() // group_size
    nwords = _packed_words(bits, group_size, False)
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    packed = torch.empty((ng, nwords), dtype=torch.int32, device=x.device)
    scale = torch.empty(ng, dtype=torch.float32, device=x.device)
    mn = torch.empty(ng, dtype=torch.float32, device=x.device)
    w = None if weight is None else weight.to(torch.float32).contiguous()
    b = None if bias is None else bias.to(torch.float32).contiguous()
    if seed is None:
        seed = _stream_seed()
    if offset is None:
        offset = _next_offset
        _next_offset += 1
    if residual is not None:
        total = torch.empty_like(x)
        with _device_of(x):
            rc = _lib.load().act_ln_add_fwd_quant_pack(
                x.data_ptr(), residual.data_ptr(), _DTYPES[x.dtype], rows, C, None if w is None else w.data_ptr(),
                None if b is None else b.data_ptr(), float(eps), group_size, bits, seed & 0xFFFFFFFFFFFFFFFF,
                offset & 0xFFFFFFFFFFFFFFFF, flags, total.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), _stream_ptr(x))
        _lib.check(rc, "act_ln_add_fwd_quant_pack")
        return total, y, mean, rstd, packed, scale, mn
    with _device_of(x):
        rc = _lib.load().act_ln_fwd_quant_pack(
            x.data_ptr(), _DTYPES[x.dtype], rows, C, None if w is None else w.data_ptr(),
            None if b is None else b.data_ptr(), float(eps), group_size, bits, seed & 0xFFFFFFFFFFFFFFFF,
            offset & 0xFFFFFFFFFFFFFFFF, flags, y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), packed.data_ptr(),
            scale.data_ptr(), mn.data_ptr(), _stream_ptr(x))
    _lib.check(rc, "act_ln_fwd_quant_pack")
    return y, mean, rstd, packed, scale, mn


def ln_bwd_from_packed(dy: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor, bits: int,
                       group_size: int, mean: torch.Tensor, rstd: torch.Tensor, weight: Optional[torch.Tensor],
                       dy2: Optional[torch.Tensor] = None):
    """(dx, dgamma, dbeta) of a LayerNorm over the last dimension whose input is given packed.
    `dy2` (dy's shape and type, contiguous): a second gradient of the input, added into dx."""
    if not dy.is_cuda:
        raise RuntimeError("ln_bwd_from_packed needs CUDA tensors: there is no CPU path")
    if not ln_fused_applies(dy, group_size, bits):
        raise ValueError("ln_bwd_from_packed: unsupported shape, type or group size")
    C = dy.shape[-1]
    rows = dy.numel() // C
    if scale.numel() * group_size != dy.numel() or mean.numel() != rows or rstd.numel() != rows:
        raise ValueError("ln_bwd_from_packed: packed input and statistics do not match dy")
    dx = torch.empty_like(dy)
    both = torch.empty((2, C), dtype=torch.float32, device=dy.device)    # adjacent: the library clears them in one pass
    dgamma, dbeta = both[0], both[1]
    w = None if weight is None else weight.to(torch.float32).contiguous()
    scale = scale.reshape(-1).contiguous()
    mn = mn.reshape(-1).contiguous()
    if dy2 is not None and (dy2.shape != dy.shape or dy2.dtype != dy.dtype or not dy2.is_contiguous()
                            or dy2.device != dy.device):
        raise ValueError("ln_bwd_from_packed: dy2 must be a contiguous tensor of dy's shape and type")
    with _device_of(dy):
        rc = _lib.load().act_ln_bwd_from_packed_sum(
            dy.data_ptr(), None if dy2 is None else dy2.data_ptr(), _DTYPES[dy.dtype], rows, C, packed.data_ptr(),
            scale.data_ptr(), mn.data_ptr(), group_size, bits, mean.data_ptr(), rstd.data_ptr(),
            None if w is None else w.data_ptr(), dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), _stream_ptr(dy))
    _lib.check(rc, "act_ln_bwd_from_packed_sum")
    return dx, dgamma, dbeta
