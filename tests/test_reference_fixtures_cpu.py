"""Pins the oracle against outputs of the REFERENCE's own Triton kernels, produced by
tests/golden/make_reference_fixtures.py under Triton's CPU interpreter and committed as
tests/golden/reference_triton_codec.npz.

What is pinned bit-for-bit: the word layout, the clamp to [0,qmax], the degenerate-range
rule (scale 1 for a constant group), the rounding rule of the live kernel
(a*(1/s) + (0.5-1e-6), truncation), the group minimum, mask pack/unpack.  The interpreter
stores fp32 -> bf16 by truncation where GPUs round to nearest even, so the stored scale is
accepted in either form.  With the tanh squash on, libm's tanhf and numpy's tanh differ in
the last bit on a few inputs; the test allows 0.5 % of codes to differ by one step.
"""
import os

import numpy as np
import pytest

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_triton_codec.npz")


@pytest.fixture(scope="module")
def fix():
    return np.load(FIX)


def _bf16_trunc(f32):
    return (np.ascontiguousarray(f32, np.float32).view(np.uint32) >> 16).astype(np.uint16)


@pytest.mark.parametrize("bits", (1, 2, 4, 8))
@pytest.mark.parametrize("gs", (64, 256))
def test_live_kernel_arithmetic(oracle, fix, bits, gs):
    key = f"b{bits}_g{gs}"
    x = fix[key + "_x"]
    F = oracle
    for tag, flags, alpha in (("identity_n", F.FLAG_REF_COMPAT | F.FLAG_META_BF16, 0.0),
                              ("identity_c", F.FLAG_REF_COMPAT | F.FLAG_META_BF16 | F.FLAG_REF_CLAMP, 1.0)):
        packed, scale, mn = oracle.quant_pack(x, gs, bits, dtype="bf16", flags=flags, clamp_alpha=alpha)
        assert np.array_equal(packed, fix[f"{key}_{tag}_packed"]), tag
        assert np.array_equal(oracle.f32_to_bf16_bits(mn), fix[f"{key}_{tag}_min"]), tag
        # scale: unrounded fp32 value truncated (interpreter) or rounded to nearest even (GPU)
        p2, s_full, _ = oracle.quant_pack(x, gs, bits, dtype="bf16", flags=flags & ~F.FLAG_META_BF16, clamp_alpha=alpha)
        want = fix[f"{key}_{tag}_scale"]
        ok = (want == _bf16_trunc(s_full)) | (want == oracle.f32_to_bf16_bits(s_full))
        assert ok.all(), tag
        assert scale[1] == 1.0                       # constant group


@pytest.mark.parametrize("bits", (1, 2, 4, 8))
@pytest.mark.parametrize("gs", (64, 256))
def test_live_kernel_with_tanh(oracle, fix, bits, gs):
    key = f"b{bits}_g{gs}"
    F = oracle
    flags = F.FLAG_REF_COMPAT | F.FLAG_META_BF16 | F.FLAG_REF_CLAMP | F.FLAG_REF_TANH
    packed, _, _ = oracle.quant_pack(fix[key + "_x"], gs, bits, dtype="bf16", flags=flags, clamp_alpha=3.0)
    _, _, mn_full = oracle.quant_pack(fix[key + "_x"], gs, bits, dtype="bf16", flags=flags & ~F.FLAG_META_BF16,
                                      clamp_alpha=3.0)
    got = oracle.np_unpack_codes(packed, gs, bits).astype(np.int64)
    want = oracle.np_unpack_codes(fix[f"{key}_tanh_c_packed"], gs, bits).astype(np.int64)
    diff = np.abs(got - want)
    assert diff.max() <= 1 and (diff != 0).mean() <= 0.005
    want_mn = fix[f"{key}_tanh_c_min"]           # truncated by the interpreter, rounded on a GPU
    near = np.abs(oracle.bf16_bits_to_f32(want_mn) - mn_full) <= np.abs(mn_full) * 2.0 ** -7 + 1e-30
    assert near.all()


@pytest.mark.parametrize("bits", (1, 2, 4, 8))
@pytest.mark.parametrize("gs", (64, 256))
def test_dequant_and_masks(oracle, fix, bits, gs):
    key = f"b{bits}_g{gs}"
    tag = f"{key}_identity_n"
    scale = oracle.bf16_bits_to_f32(fix[tag + "_scale"])
    mn = oracle.bf16_bits_to_f32(fix[tag + "_min"])
    y = oracle.dequant_unpack(fix[tag + "_packed"], scale, mn, gs, bits, out="bf16")
    want = fix[tag + "_deq"]
    # the interpreter rounds q*scale and +min separately and truncates to bf16; the oracle
    # fuses and rounds to nearest: equal up to one bf16 step
    d = np.abs(oracle.bf16_bits_to_f32(y).astype(np.float64) - oracle.bf16_bits_to_f32(want).astype(np.float64))
    step = np.maximum(np.abs(oracle.bf16_bits_to_f32(want)), 1e-30).astype(np.float64) * 2.0 ** -7
    assert (d <= step).all()
    assert np.array_equal(oracle.np_unpack_codes(fix[tag + "_packed"], gs, bits).max() <= (1 << bits) - 1, True)
    # mask pack / unpack: exact
    mask = fix[key + "_mask"]
    assert np.array_equal(oracle.pack_bits(mask, gs, bits), fix[key + "_mask_packed"])
    assert np.array_equal(oracle.unpack_bits(fix[key + "_mask_packed"], gs, bits), fix[key + "_mask_unpacked"])


# ---------------------------------------------------------------- FP8 GEMM
# tests/golden/reference_triton_linear.npz: outputs of the reference's own GEMM kernel
# (Activation_Compression/triton_kernel/linear.py:43-95) run under Triton's CPU interpreter on
# e4m3 operands, fp32 accumulator stored as fp32.  With scales of one the oracle's product must
# reproduce them: exactly where every partial sum is exact (small-integer operands), and within
# the fp32 summation-order bound K * 2^-24 * sum|a*b| otherwise (the oracle sums in double).
LIN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_triton_linear.npz")


@pytest.mark.parametrize("case", range(4))
def test_gemm_oracle_against_reference_kernel(oracle, case):
    fx = np.load(LIN)
    A8, B8, want = fx[f"case{case}_A8"], fx[f"case{case}_B8"], fx[f"case{case}_C"]
    M, K = A8.shape
    N = B8.shape[1]
    _, got = oracle.fp8_gemm(A8, B8, np.ones(M, np.float32), np.ones(N, np.float32))
    if str(fx[f"case{case}_kind"]) == "int":
        assert np.array_equal(got, want)
    else:
        a = np.abs(oracle.e4m3_decode(A8).astype(np.float64))
        b = np.abs(oracle.e4m3_decode(B8).astype(np.float64))
        bound = (a @ b) * K * 2.0 ** -24 + 1e-30
        assert (np.abs(got.astype(np.float64) - want.astype(np.float64)) <= bound).all()
        # and the double-accumulated value is the closer one to the exact product
        exact = oracle.e4m3_decode(A8).astype(np.float64) @ oracle.e4m3_decode(B8).astype(np.float64)
        assert np.abs(got - exact).max() <= np.abs(exact).max() * 2.0 ** -23
