"""ctypes binding of libact_b200.so (the C ABI declared in include/act_b200.h).

The library is the only compute path of this package.  Loading fails loudly
when the shared object is missing; there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# ACT_B200_LIB points at another build of the same library (tuning experiments)
LIB_PATH = os.environ.get("ACT_B200_LIB") or os.path.join(HERE, "libact_b200.so")

ACT_DTYPE_F32, ACT_DTYPE_BF16, ACT_DTYPE_F16 = 0, 1, 2
ACT_FLAG_ROUND_NEAREST = 1
ACT_FLAG_REF_COMPAT = 2
ACT_FLAG_REF_CLAMP = 4
ACT_FLAG_REF_TANH = 8
ACT_FLAG_META_BF16 = 16
ACT_FLAG_BALLOT_REF_BIAS = 32
ACT_GEMM_B_IS_NK = 1
ACT_GEMM_SINGLE_CTA = 2
ACT_KIND_GELU, ACT_KIND_SILU, ACT_KIND_GELU_ERF = 1, 2, 3

# every symbol include/act_b200.h declares, with its ctypes signature
_vp, _i32, _i64, _u64, _f32 = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_uint64,
                               ctypes.c_float)
_f64, _sz = ctypes.c_double, ctypes.c_size_t
SIGNATURES = {
    "act_quant_pack": ([_vp, _i32, _i64, _i32, _i32, _vp, _u64, _u64, _i32, _f32, _vp, _vp, _vp, _vp], _i32),
    "act_dequant_unpack": ([_vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp], _i32),
    "act_quant_pack_tiles": ([_vp, _i32, _i64, _i32, _i32, _i32, _i32, _u64, _u64, _i32, _vp, _vp, _vp, _vp], _i32),
    "act_dequant_unpack_tiles": ([_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _vp], _i32),
    "act_pack_bits": ([_vp, _i64, _i32, _i32, _vp, _vp], _i32),
    "act_unpack_bits": ([_vp, _i64, _i32, _i32, _vp, _vp], _i32),
    "act_activation_fwd_quant_pack": ([_vp, _i32, _i32, _i64, _i32, _i32, _u64, _u64, _i32, _vp, _vp, _vp, _vp, _vp], _i32),
    "act_relu_fwd_pack": ([_vp, _i32, _i64, _i32, _vp, _vp, _vp], _i32),
    "act_relu_bwd_unpack": ([_vp, _vp, _i32, _i64, _vp, _vp], _i32),
    "act_relu_bwd_unpack_sum": ([_vp, _vp, _vp, _i32, _i64, _vp, _vp], _i32),
    "act_mul_dequant_unpack": ([_vp, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _vp, _vp], _i32),
    "act_bn_fwd_norm_quant_pack": ([_vp, _i32, _i64, _i32, _i64, _vp, _i32, _i32, _u64, _u64, _i32, _vp, _vp, _vp, _vp, _vp], _i32),
    "act_bn_stats_workspace": ([_i64, _i32], _sz),
    "act_bn_stats": ([_vp, _i32, _i64, _i32, _i64, _f64, _vp, _vp, _vp, _vp, _f64, _vp, _vp, _sz, _vp], _i32),
    "act_bn_bwd_reduce": ([_vp, _vp, _vp, _vp, _i32, _i64, _i32, _i64, _i32, _i32, _vp, _vp], _i32),
    "act_bn_bwd_coef": ([_vp, _vp, _i32, _f64, _vp, _vp], _i32),
    "act_bn_bwd_dx": ([_vp, _vp, _vp, _vp, _i32, _i64, _i32, _i64, _i32, _i32, _vp, _vp, _vp], _i32),
    "act_maxpool_fwd_cl": ([_vp, _i32, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp], _i32),
    "act_maxpool_bwd_cl": ([_vp, _vp, _i32, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp], _i32),
    "act_bn_forward": ([_vp, _vp, _i32, _i64, _i32, _i64, _f64, _vp, _vp, _vp, _vp, _f64, _vp, _vp, _sz, _i32, _i32,
                        _u64, _u64, _i32, _vp, _vp, _vp, _vp, _vp, _vp], _i32),
    "act_bn_backward": ([_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i64, _i32, _i32, _vp, _f64, _vp, _vp, _vp, _vp,
                         _vp], _i32),
    "act_bn_backward_sum": ([_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i64, _i32, _i32, _vp, _f64, _vp, _vp, _vp, _vp,
                         _vp], _i32),
    "act_bn_add_relu_bwd_reduce": ([_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i64, _i32, _i32, _vp, _vp, _vp], _i32),
    "act_bn_add_relu_bwd_reduce_sum": ([_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i64, _i32, _i32, _vp, _vp, _vp], _i32),
    "act_quant_pack_avg": ([_vp, _i32, _i64, _i32, _i32, _i32, _vp, _u64, _u64, _i32, _f32, _vp, _vp, _vp, _vp], _i32),
    "act_dequant_unpack_avg": ([_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _vp], _i32),
    "act_bn_relu_fwd_norm_quant_pack": ([_vp, _i32, _i64, _i32, _i64, _vp, _i32, _i32, _u64, _u64, _i32, _vp, _vp, _vp, _vp, _vp, _vp], _i32),
    "act_bn_add_relu_fwd_norm_quant_pack": ([_vp, _vp, _i32, _i64, _i32, _i64, _vp, _i32, _i32, _u64, _u64, _i32, _vp, _vp, _vp, _vp, _vp, _vp], _i32),
    "act_bn_relu_bwd_reduce": ([_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i64, _i32, _i32, _vp, _vp], _i32),
    "act_bn_relu_bwd_dx": ([_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i64, _i32, _i32, _vp, _vp, _vp], _i32),
    "act_minmax": ([_vp, _i32, _i64, _i64, _vp, _vp, _vp], _i32),
    "act_pack_ballot": ([_vp, _i32, _i64, _i32, _i32, _vp, _vp, _u64, _i32, _vp, _vp, _vp], _i32),
    "act_unpack_ballot": ([_vp, _vp, _vp, _i32, _i64, _i32, _i32, _vp, _vp], _i32),
    "act_copy": ([_vp, _vp, _sz, _sz, _sz, _vp], _i32),
    "act_fill_zero": ([_vp, _sz, _vp], _i32),
    "act_col_sum": ([_vp, _i32, _i64, _i32, _vp, _vp], _i32),
    "act_ln_bwd_params": ([_vp, _vp, _vp, _vp, _i32, _i64, _i32, _vp, _vp, _vp], _i32),
    "act_ln_fwd_quant_pack": ([_vp, _i32, _i64, _i32, _vp, _vp, ctypes.c_double, _i32, _i32, _u64, _u64,
                               _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp], _i32),
    "act_ln_bwd_from_packed": ([_vp, _i32, _i64, _i32, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp], _i32),
    "act_ln_add_fwd_quant_pack": ([_vp, _vp, _i32, _i64, _i32, _vp, _vp, ctypes.c_double, _i32, _i32, _u64, _u64,
                                   _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp], _i32),
    "act_ln_bwd_from_packed_sum": ([_vp, _vp, _i32, _i64, _i32, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp,
                                    _vp], _i32),
    "act_merge_heads": ([_vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp], _i32),
    "act_calc_precision": ([_vp, _vp, _vp, _i64, ctypes.c_double], _i32),
    "act_fp8_gemm_workspace": ([_i32, _i32, _i32, _i32], ctypes.c_size_t),
    "act_fp8_gemm": ([_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, ctypes.c_size_t, _vp], _i32),
    "act_fp8_gemm_status": ([_vp, _i32], _i32),
    "act_dw_from_packed": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _vp], _i32),
    "act_dw_from_packed_status": ([_vp, _i32], _i32),
    "act_fp8_gemm_static_limit": ([], ctypes.c_size_t),
    "act_fp8_gemm_static": ([_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp], _i32),
    "act_strerror": ([_i32], ctypes.c_char_p),
    "act_abi_version": ([], _i32),
}

_lib = None


class ActLibraryError(RuntimeError):
    """Raised when the C ABI returns a non-zero code."""


def load() -> ctypes.CDLL:
    """Load libact_b200.so; raises if it has not been built (python -m deep_optimization_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m deep_optimization_b200.build` "
                "(needs nvcc); this package has no fallback path")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if the symbol is not exported
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().act_strerror(code).decode()
        raise ActLibraryError(f"{what}: {msg} (code {code})")


_NO_SWITCH = None


def stream_ptr(t) -> int:
    """Raw handle of PyTorch's current stream on t's device (no Stream object is built)."""
    import torch
    return torch._C._cuda_getCurrentRawStream(t.device.index)


def device_of(t):
    """Context that makes t's device current for a launch; free when it already is."""
    import contextlib
    import torch
    global _NO_SWITCH
    if t.device.index == torch.cuda.current_device():
        if _NO_SWITCH is None:
            _NO_SWITCH = contextlib.nullcontext()
        return _NO_SWITCH
    return torch.cuda.device(t.device)
