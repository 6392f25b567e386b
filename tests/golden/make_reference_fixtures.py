"""Generates tests/golden/reference_triton_codec.npz by running the REFERENCE's own Triton
kernels (Activation_Compression/act_triton_kernel.py: quant_pack_kernel,
dequant_unpack_kernel, pack_kernel, unpack_kernel) under Triton's CPU interpreter, and
tests/golden/reference_triton_linear.npz by running its GEMM kernel
(Activation_Compression/triton_kernel/linear.py:43-95, Triton_Linear) the same way on
e4m3 operands.

Run where the reference checkout is available:

    TRITON_INTERPRET=1 python tests/golden/make_reference_fixtures.py /path/to/Deep_Optimization [codec|linear|all]

The kernels are called directly (their torch.library wrappers refuse interpreted
functions).  `libdevice.tanh`, which the interpreter cannot evaluate, is replaced for
the call either by the identity (then `tanh(x/0.5)*0.5` returns x exactly and the
kernel is the plain codec) or by numpy's tanh.  Nothing else of the reference is
modified.  The interpreter does not fuse multiply-add and truncates fp32 -> bf16 on
store; scale and min are therefore stored here from fp32 buffers (the kernel's `.to(bf16)`
on an fp32 pointer is then a value rounding done by the interpreter's numpy cast).
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")
import numpy as np
import torch

if len(sys.argv) < 2:
    raise SystemExit("usage: make_reference_fixtures.py /path/to/Deep_Optimization")
ref_root = sys.argv[1]
sys.path.insert(0, os.path.join(ref_root, "Activation_Compression"))
import act_triton_kernel as ref  # noqa: E402
from triton.language.extra import libdevice  # noqa: E402


def run_quant(x, bits, gs, clamp, alpha, tanh_mode):
    ng = x.shape[0]
    vpw, nwords, qmax = ref._bits_consts(bits, gs)
    packed = torch.zeros((ng, nwords), dtype=torch.int32)
    scale = torch.zeros(ng, dtype=torch.bfloat16)
    mn = torch.zeros(ng, dtype=torch.bfloat16)
    saved = libdevice.tanh
    import triton.language as tl
    if tanh_mode == "identity":
        libdevice.tanh = lambda v: v
    else:
        libdevice.tanh = lambda v: tl.core.tensor(
            type(v.handle)(np.tanh(v.handle.data.astype(np.float64)).astype(np.float32), v.handle.dtype), v.type)
    try:
        ref.quant_pack_kernel[(ng,)](x, packed, scale, mn, 42, x.stride(0), x.stride(1), packed.stride(0),
                                     packed.stride(1), BITS=bits, VPW=vpw, NWORDS=nwords, QMAX=qmax,
                                     AVG_ALAM=False, ALAM_BITS=0, ALAM_NWORDS=nwords, SUB_GROUP=0,
                                     CLAMP=clamp, CLAMP_ALPHA=alpha)
    finally:
        libdevice.tanh = saved
    return packed, scale, mn


def run_dequant(packed, scale, mn, bits, gs):
    ng = packed.shape[0]
    vpw, nwords, _ = ref._bits_consts(bits, gs)
    y = torch.zeros((ng, gs), dtype=torch.bfloat16)
    ref.dequant_unpack_kernel[(ng,)](packed, scale, mn, y, 42, packed.stride(0), packed.stride(1), y.stride(0),
                                     y.stride(1), BITS=bits, VPW=vpw, NWORDS=nwords, AVG_ALAM=False,
                                     ALAM_BITS=0, ALAM_NWORDS=nwords, SUB_GROUP=0)
    return y


def bits16(t):
    return t.view(torch.int16).numpy().view(np.uint16)


def main():
    out = {}
    g = torch.Generator().manual_seed(0)
    for bits in (1, 2, 4, 8):
        for gs in (64, 256):
            ng = 6
            x = torch.relu(torch.randn(ng, gs, generator=g)).to(torch.bfloat16)
            x[1] = 0.0                     # constant group: the degenerate-range rule
            x[2, ::2] *= -1.0              # signed values
            key = f"b{bits}_g{gs}"
            out[key + "_x"] = bits16(x)
            for mode, clamp, alpha in (("identity", False, 0.0), ("identity", True, 1.0), ("tanh", True, 3.0)):
                p, s, m = run_quant(x, bits, gs, clamp, alpha, mode)
                tag = f"{key}_{mode}_{'c' if clamp else 'n'}"
                out[tag + "_packed"] = p.numpy().view(np.uint32)
                out[tag + "_scale"] = bits16(s)
                out[tag + "_min"] = bits16(m)
                if mode == "identity" and not clamp:
                    out[tag + "_deq"] = bits16(run_dequant(p, s, m, bits, gs))
            # mask pack / unpack
            # int8 inputs: values above 127 would be sign-extended by the reference's kernel
            # (a quirk no caller meets: masks are 0/1), so the fixture stays below 128
            mask = (torch.rand(ng, gs, generator=g) * min(1 << bits, 128)).to(torch.int8)
            vpw, nwords, _ = ref._bits_consts(bits, gs)
            pk = torch.zeros((ng, nwords), dtype=torch.int32)
            ref.pack_kernel[(ng,)](mask, pk, mask.stride(0), mask.stride(1), pk.stride(0), pk.stride(1),
                                   BITS=bits, VPW=vpw, NWORDS=nwords)
            un = torch.zeros((ng, gs), dtype=torch.int8)
            ref.unpack_kernel[(ng,)](pk, un, pk.stride(0), pk.stride(1), un.stride(0), un.stride(1),
                                     BITS=bits, VPW=vpw, NWORDS=nwords)
            out[key + "_mask"] = mask.numpy()
            out[key + "_mask_packed"] = pk.numpy().view(np.uint32)
            out[key + "_mask_unpacked"] = un.numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_triton_codec.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, len(out), "arrays")


def run_linear(A8, B8, block):
    """C = A8 @ B8 by the reference's Triton_Linear (the jitted function under its autotuner,
    one of its own tile shapes given explicitly), fp32 accumulator stored as fp32."""
    import triton
    import triton.language as tl
    sys.path.insert(0, os.path.join(ref_root, "Activation_Compression", "triton_kernel"))
    import linear as ref_linear
    M, K = A8.shape
    N = B8.shape[1]
    bm, bn, bk = block
    C = torch.zeros((M, N), dtype=torch.float32)
    grid = (triton.cdiv(M, bm) * triton.cdiv(N, bn),)
    ref_linear.Triton_Linear.fn[grid](A8, B8, C, M, N, K, A8.stride(0), A8.stride(1), B8.stride(0), B8.stride(1),
                                      C.stride(0), C.stride(1), BLOCK_SIZE_M=bm, BLOCK_SIZE_N=bn,
                                      BLOCK_SIZE_K=bk, GROUP_SIZE_M=8, OUT_DTYPE=tl.float32)
    return C


def main_linear():
    """Two kinds of case.  `int`: small-integer operands (every product and partial sum is exact in
    fp32, so any correct GEMM returns the same bits whatever its summation order).  `rand`: N(0,1)
    operands scaled to the e4m3 range as the evaluation configuration describes; the fp32 sums then
    depend on the order, which the test bounds."""
    out = {}
    g = torch.Generator().manual_seed(0)
    cases = (("int", 96, 136, 160, (32, 64, 32)), ("int", 130, 72, 272, (64, 32, 32)),
             ("rand", 64, 128, 256, (32, 64, 32)), ("rand", 100, 264, 144, (64, 128, 64)))
    for i, (kind, M, N, K, block) in enumerate(cases):
        if kind == "int":
            A = torch.randint(-8, 9, (M, K), generator=g).float()
            B = torch.randint(-8, 9, (K, N), generator=g).float()
        else:
            A = torch.randn(M, K, generator=g)
            B = torch.randn(K, N, generator=g)
            A = A / (A.abs().amax(1, keepdim=True) / 448.0)
            B = B / (B.abs().amax(0, keepdim=True) / 448.0)
        A8, B8 = A.to(torch.float8_e4m3fn), B.to(torch.float8_e4m3fn)
        C = run_linear(A8, B8, block)
        out[f"case{i}_kind"] = np.array(kind)
        out[f"case{i}_A8"] = A8.view(torch.uint8).numpy()
        out[f"case{i}_B8"] = B8.view(torch.uint8).numpy()
        out[f"case{i}_C"] = C.numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_triton_linear.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, len(out), "arrays")


if __name__ == "__main__":
    what = sys.argv[2] if len(sys.argv) > 2 else "all"
    if what in ("codec", "all"):
        main()
    if what in ("linear", "all"):
        main_linear()
