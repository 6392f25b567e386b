"""`torch.ops.act_lib.*` codec operators, backed by the sm_100a CUDA library.

The operator names, positional schemas and return orders are those of
Activation_Compression/act_triton_kernel.py:336-433 (there implemented in
Triton), so callers such as `modules/module_utils.py` work unchanged:

    quant_pack_triton(x[N,G,gs], bits, group_size, avg_alam, alam_bits, clamp, clamp_alpha)
        -> (packed int32 [N*G, gs*bits/32], scale [N,G], min [N,G])
    dequant_unpack_triton(packed, scale[N,G], xmin[N,G], bits, group_size, avg_alam, alam_bits)
        -> bf16 [N,G,gs]
    pack_triton(x int8 [N,G,gs], bits, group_size) -> int32 [N*G, gs*bits/32]
    unpack_triton(packed, bits, N, G, group_size)  -> int8 [N,G,gs]

Differences from the reference, on purpose:
  * scale and min are fp32 (the reference stores bf16); `set_mode("ref_compat")`
    switches to the live Triton arithmetic (clamp, tanh squash, round to nearest,
    bf16-rounded scale/min) for recipes that depend on it.
  * the default mode rounds stochastically with the in-kernel counter hash;
    `noise=` supplies the uniform tensor instead, `seed=` pins the stream.
  * the fake (meta) kernels have the real signatures, so FakeTensor tracing and
    torch.compile see correct shapes and dtypes.
The names keep their `_triton` suffix only because callers look them up by name.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib, codec
from .codec import _bits_consts

_MODE = "baseline"          # "baseline" | "nearest" | "ref_compat"


def set_mode(mode: str) -> None:
    """baseline: stochastic rounding, exact division (default).
    nearest: same arithmetic with the constant 0.5-1e-6 instead of noise.
    ref_compat: the reference's live arithmetic (clamp/tanh/truncate/bf16 meta)."""
    global _MODE
    if mode not in ("baseline", "nearest", "ref_compat"):
        raise ValueError(f"unknown codec mode {mode!r}")
    _MODE = mode


def get_mode() -> str:
    return _MODE


IMPL = {}


def _op(name):
    """Registers `fn` as torch.ops.act_lib.<name> and keeps the plain function in IMPL."""
    def deco(fn):
        IMPL[name] = fn
        return torch.library.custom_op(f"act_lib::{name}", fn, mutates_args=(), device_types="cuda")
    return deco


def op(name: str):
    """The callable behind `torch.ops.act_lib.<name>` for this package's own autograd Functions:
    the plain Python implementation in eager mode (a dispatcher round trip costs about 60 us
    of host time per call, more than most of these kernels run), the registered operator while
    torch.compile is tracing."""
    if torch.compiler.is_compiling():
        return getattr(torch.ops.act_lib, name)
    return IMPL[name]


@_op("quant_pack_triton")
def quant_pack_triton(x: torch.Tensor, bits: int, group_size: int, avg_alam: bool, alam_bits: int,
                      clamp: bool, clamp_alpha: float, noise: Optional[torch.Tensor] = None,
                      seed: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    N, G, gs = x.shape
    if gs != group_size:
        raise ValueError(f"last dimension {gs} != group_size {group_size}")
    flags, alpha = 0, 0.0
    if _MODE == "nearest":
        flags = _lib.ACT_FLAG_ROUND_NEAREST
    elif _MODE == "ref_compat":
        flags = _lib.ACT_FLAG_REF_COMPAT | _lib.ACT_FLAG_REF_TANH | _lib.ACT_FLAG_META_BF16
        if clamp:
            flags |= _lib.ACT_FLAG_REF_CLAMP
            alpha = clamp_alpha
    if avg_alam:
        # one code per alam_bits consecutive elements (act_triton_kernel.py:116-118, 344-347)
        packed, scale, mn = codec.quant_pack_avg(x, bits, group_size, alam_bits, noise=noise, seed=seed,
                                                 flags=flags, clamp_alpha=alpha)
    else:
        packed, scale, mn = codec.quant_pack(x, bits, group_size, noise=noise, seed=seed, flags=flags,
                                             clamp_alpha=alpha)
    return packed, scale.view(N, G), mn.view(N, G)


@quant_pack_triton.register_fake
def _(x, bits, group_size, avg_alam, alam_bits, clamp, clamp_alpha, noise=None, seed=None):
    N, G = x.shape[:2]
    _, nwords, _ = _bits_consts(bits, group_size)
    if avg_alam:
        nwords = -(-nwords // alam_bits)
    return (x.new_empty((N * G, nwords), dtype=torch.int32),
            x.new_empty((N, G), dtype=torch.float32), x.new_empty((N, G), dtype=torch.float32))


@_op("dequant_unpack_triton")
def dequant_unpack_triton(packed: torch.Tensor, scale: torch.Tensor, xmin: torch.Tensor, bits: int,
                          group_size: int, avg_alam: bool, alam_bits: int) -> torch.Tensor:
    N, G = scale.shape
    if avg_alam:
        y = codec.dequant_unpack_avg(packed, scale, xmin, bits, group_size, alam_bits, out_dtype=torch.bfloat16)
    else:
        y = codec.dequant_unpack(packed, scale, xmin, bits, group_size, out_dtype=torch.bfloat16)
    return y.view(N, G, group_size)


@dequant_unpack_triton.register_fake
def _(packed, scale, xmin, bits, group_size, avg_alam, alam_bits):
    N, G = scale.shape
    return packed.new_empty((N, G, group_size), dtype=torch.bfloat16)


@_op("pack_triton")
def pack_triton(x: torch.Tensor, bits: int, group_size: int) -> torch.Tensor:
    if x.shape[-1] != group_size:
        raise ValueError("last dimension must equal group_size")
    return codec.pack_bits(x, bits, group_size)


@pack_triton.register_fake
def _(x, bits, group_size):
    N, G, _ = x.shape
    _, nwords, _ = _bits_consts(bits, group_size)
    return x.new_empty((N * G, nwords), dtype=torch.int32)


@_op("unpack_triton")
def unpack_triton(packed: torch.Tensor, bits: int, N: int, G: int, group_size: int) -> torch.Tensor:
    return codec.unpack_bits(packed, bits, N * G, group_size).view(N, G, group_size)


@unpack_triton.register_fake
def _(packed, bits, N, G, group_size):
    return packed.new_empty((N, G, group_size), dtype=torch.int8)


# ---- fused activation operators (Activation_Compression/modules/activations/
# kernel_registration.py:43-94, 148-237, 262-319): same names, schemas and return orders ----

@_op("relu_fwd_fused_pack")
def relu_fwd_fused_pack(x: torch.Tensor, relu: bool, relu6: bool, bits: int,
                        group_size: int) -> Tuple[torch.Tensor, torch.Tensor, int, int]:
    if bits != 1:
        raise ValueError("the fused ReLU mask is 1 bit per element")
    N = x.shape[0]
    G = x.numel() // N // group_size
    y, packed = codec.relu_fwd_pack(x, relu6=(relu6 and not relu))
    return y, packed.view(N * G, group_size // 32), N, G


@relu_fwd_fused_pack.register_fake
def _(x, relu, relu6, bits, group_size):
    N = x.shape[0]
    G = x.numel() // N // group_size
    return torch.empty_like(x), x.new_empty((N * G, group_size // 32), dtype=torch.int32), N, G


@_op("relu_bwd_fused_unpack")
def relu_bwd_fused_unpack(packed: torch.Tensor, dy: torch.Tensor, bits: int, N: int, G: int,
                          group_size: int) -> torch.Tensor:
    return codec.relu_bwd_unpack(packed, dy)


@relu_bwd_fused_unpack.register_fake
def _(packed, dy, bits, N, G, group_size):
    return torch.empty_like(dy)


def _fused_act_fwd(x, kind, bits, group_size):
    N = x.shape[0]
    G = x.numel() // N // group_size
    flags = _lib.ACT_FLAG_ROUND_NEAREST if _MODE != "baseline" else 0
    y, packed, scale, mn = codec.activation_fwd_quant_pack(x, kind, bits, group_size, flags=flags)
    return y, packed, scale.view(N, G), mn.view(N, G), N, G


def _fused_act_fake(x, bits, group_size):
    N = x.shape[0]
    G = x.numel() // N // group_size
    _, nwords, _ = _bits_consts(bits, group_size)
    return (torch.empty_like(x), x.new_empty((N * G, nwords), dtype=torch.int32),
            x.new_empty((N, G), dtype=torch.float32), x.new_empty((N, G), dtype=torch.float32), N, G)


@_op("gelu_fwd_fused_quan_pack")
def gelu_fwd_fused_quan_pack(x: torch.Tensor, bits: int, group_size: int, exact: bool = False
                             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, int, int]:
    """`exact` (an addition to the reference's schema) selects x * Phi(x) instead of the tanh
    approximation, for modules built from nn.GELU(approximate="none")."""
    return _fused_act_fwd(x, "gelu_erf" if exact else "gelu", bits, group_size)


@gelu_fwd_fused_quan_pack.register_fake
def _(x, bits, group_size, exact=False):
    return _fused_act_fake(x, bits, group_size)


@_op("gelu_bwd_fused_dequan_unpack")
def gelu_bwd_fused_dequan_unpack(packed: torch.Tensor, dy: torch.Tensor, scale: torch.Tensor,
                                 min: torch.Tensor, bits: int, N: int, G: int, group_size: int) -> torch.Tensor:
    return codec.mul_dequant_unpack(packed, scale.reshape(-1), min.reshape(-1), dy, bits, group_size)


@gelu_bwd_fused_dequan_unpack.register_fake
def _(packed, dy, scale, min, bits, N, G, group_size):
    return torch.empty_like(dy)


def _no_alam(avg_alam: bool) -> None:
    if avg_alam:
        raise NotImplementedError("the fused activation operators do not average sub-groups; "
                                  "layers with AVG_ALAM take the unfused path (quant_pack_triton)")


@_op("silu_fwd_quan_pack")
def silu_fwd_quan_pack(input: torch.Tensor, bits: int, group_size: int, pack_only: bool, avg_alam: bool,
                       alam_bits: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, int,
                                                int, int, int, bool, bool]:
    _no_alam(avg_alam)
    y, packed, scale, mn, N, G = _fused_act_fwd(input, "silu", bits, group_size)
    return y, packed, scale, mn, N, G, 0, 0, False, False          # flat grouping


@silu_fwd_quan_pack.register_fake
def _(input, bits, group_size, pack_only, avg_alam, alam_bits):
    return _fused_act_fake(input, bits, group_size) + (0, 0, False, False)


@_op("silu_bwd_fused_dequan_unpack")
def silu_bwd_fused_dequan_unpack(act_packed: torch.Tensor, dy: torch.Tensor, scale: torch.Tensor,
                                 min: torch.Tensor, bits: int, N: int, G: int, group_size: int,
                                 pack_only: bool, new_H: int, new_W: int, spatical_padding_eligibility: bool,
                                 spatical_reshape_eligibility: bool, avg_alam: bool, alam_bits: int) -> torch.Tensor:
    _no_alam(avg_alam)
    return codec.mul_dequant_unpack(act_packed, scale.reshape(-1), min.reshape(-1), dy, bits, group_size)


@silu_bwd_fused_dequan_unpack.register_fake
def _(act_packed, dy, scale, min, bits, N, G, group_size, pack_only, new_H, new_W,
      spatical_padding_eligibility, spatical_reshape_eligibility, avg_alam, alam_bits):
    return torch.empty_like(dy)
