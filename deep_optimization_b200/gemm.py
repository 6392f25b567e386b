"""FP8 e4m3 GEMM with per-row / per-column scales (tcgen05 kernel behind the C ABI).

`fp8_gemm(A8, B8, sa, sb)` computes bf16((A8 @ B8) * sa[:,None] * sb[None,:]) for
A8 [M,K] and B8 [K,N] (the operand layout of the reference's Triton_Linear,
Activation_Compression/triton_kernel/linear.py:43-95) or, with `b_is_nk=True`,
B8 given as [N,K] like an nn.Linear weight.  `quantize_e4m3` produces the
operands and scales the way the evaluation configuration describes (amax / 448).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

E4M3_MAX = 448.0


def quantize_e4m3(x: torch.Tensor, dim: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Scale each slice along `dim` to the e4m3 range; returns (fp8 tensor, fp32 scales)."""
    amax = x.abs().amax(dim=dim, keepdim=True).float().clamp_min(1e-12)
    scale = amax / E4M3_MAX
    q = (x.float() / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q, scale.squeeze(dim).contiguous()


def workspace_bytes(M: int, N: int, K: int, b_is_nk: bool) -> int:
    return int(_lib.load().act_fp8_gemm_workspace(M, N, K, _lib.ACT_GEMM_B_IS_NK if b_is_nk else 0))


def fp8_gemm(A8: torch.Tensor, B8: torch.Tensor, sa: torch.Tensor, sb: torch.Tensor,
             b_is_nk: bool = False, out: Optional[torch.Tensor] = None,
             workspace: Optional[torch.Tensor] = None, single_cta: bool = False) -> torch.Tensor:
    if not A8.is_cuda:
        raise RuntimeError("fp8_gemm needs CUDA tensors: there is no CPU path")
    if A8.dtype != torch.float8_e4m3fn or B8.dtype != torch.float8_e4m3fn:
        raise TypeError("operands must be torch.float8_e4m3fn")
    A8, B8 = A8.contiguous(), B8.contiguous()
    M, K = A8.shape
    N = B8.shape[0] if b_is_nk else B8.shape[1]
    if (B8.shape[1] if b_is_nk else B8.shape[0]) != K:
        raise ValueError("inner dimensions differ")
    sa = sa.to(torch.float32).contiguous()
    sb = sb.to(torch.float32).contiguous()
    if sa.numel() != M or sb.numel() != N:
        raise ValueError("sa must have M entries and sb N entries")
    C = out if out is not None else torch.empty((M, N), dtype=torch.bfloat16, device=A8.device)
    flags = (_lib.ACT_GEMM_B_IS_NK if b_is_nk else 0) | (_lib.ACT_GEMM_SINGLE_CTA if single_cta else 0)
    need = workspace_bytes(M, N, K, b_is_nk)
    ws_ptr, ws_len = None, 0
    if need:
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=A8.device)
        ws_ptr, ws_len = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    with _lib.device_of(A8):
        rc = _lib.load().act_fp8_gemm(A8.data_ptr(), B8.data_ptr(), sa.data_ptr(), sb.data_ptr(), C.data_ptr(),
                                      M, N, K, A8.stride(0), B8.stride(0), C.stride(0), flags, ws_ptr, ws_len,
                                      _lib.stream_ptr(A8))
    _lib.check(rc, "act_fp8_gemm")
    return C


def gemm_status(clear: bool = True) -> int:
    """Abort reason of the last GEMM (0 = none).  Synchronises the device."""
    import ctypes
    v = ctypes.c_uint(0)
    _lib.check(_lib.load().act_fp8_gemm_status(ctypes.byref(v), 1 if clear else 0), "act_fp8_gemm_status")
    return int(v.value)


def dw_from_packed(dy: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor, mn: torch.Tensor, bits: int,
                   group_size: int, K: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dW [N, K] (fp32) = dy[M, N]^T @ X~[M, K] with X~ decoded from `packed / scale / mn` (the
    output of codec.quant_pack on the row-major [M, K] layer input, flat groups) inside the
    GEMM: the step `dequant_unpack` + `dy.T.mm(x)` of a linear layer's backward
    (Activation_Compression/modules/ops.py:496-526) without the dequantised copy."""
    if not dy.is_cuda:
        raise RuntimeError("dw_from_packed needs CUDA tensors: there is no CPU path")
    if dy.dtype != torch.bfloat16:
        raise TypeError("dy must be bfloat16")
    dy = dy.reshape(-1, dy.shape[-1])
    if dy.stride(1) != 1:
        dy = dy.contiguous()
    M, N = dy.shape
    packed = packed.contiguous()
    scale = scale.reshape(-1).to(torch.float32).contiguous()
    mn = mn.reshape(-1).to(torch.float32).contiguous()
    if scale.numel() * group_size != M * K:
        raise ValueError("scale does not have one entry per group of the [M, K] input")
    dw = out if out is not None else torch.empty((N, K), dtype=torch.float32, device=dy.device)
    if dw.dtype != torch.float32 or dw.shape != (N, K) or dw.stride(1) != 1:
        raise ValueError("out must be a float32 [N, K] tensor with unit column stride")
    with _lib.device_of(dy):
        rc = _lib.load().act_dw_from_packed(dy.data_ptr(), packed.data_ptr(), scale.data_ptr(), mn.data_ptr(), bits,
                                            group_size, M, N, K, dy.stride(0), dw.data_ptr(), dw.stride(0),
                                            _lib.stream_ptr(dy))
    _lib.check(rc, "act_dw_from_packed")
    return dw


def dw_status(clear: bool = True) -> int:
    """Abort reason of the last dw_from_packed (0 = none).  Synchronises the device."""
    import ctypes
    v = ctypes.c_uint(0)
    _lib.check(_lib.load().act_dw_from_packed_status(ctypes.byref(v), 1 if clear else 0), "act_dw_from_packed_status")
    return int(v.value)
