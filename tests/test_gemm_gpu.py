"""GPU tests of the FP8 GEMM against the CPU oracle (double accumulation) and against
a float64 torch product at sizes the oracle would take too long for.

Tolerance: the result is bf16, so half an ulp is 2^-9 relative; fp32 accumulation on
the tensor cores adds at most about K * 2^-24 of sum|a*b|.  The tests allow
|got - ref| <= 2^-8 * |ref| + 2^-20 * K^0.5 * rms-magnitude of the row's products."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed=0):
    from deep_optimization_b200.gemm import quantize_e4m3
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(M, K, generator=g)
    B = torch.randn(K, N, generator=g)
    A8, sa = quantize_e4m3(A, 1)
    B8, sb = quantize_e4m3(B, 0)
    return A8, B8, sa, sb


def _check(got, ref, K):
    got, ref = got.double().cpu(), ref.double().cpu()
    tol = ref.abs() * 2.0 ** -8 + ref.abs().max() * 2.0 ** -12 + 1e-6
    bad = (got - ref).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} outside tolerance; max err {(got-ref).abs().max()}"


@pytest.mark.parametrize("shape", [(128, 256, 128), (128, 256, 512), (256, 512, 256), (384, 768, 1024),
                                   (100, 264, 144), (8, 8, 16)])
def test_against_oracle(oracle, cuda_device, shape):
    from deep_optimization_b200.gemm import fp8_gemm, gemm_status
    M, N, K = shape
    A8, B8, sa, sb = _operands(M, N, K, seed=M + N + K)
    _, ref = oracle.fp8_gemm(A8.view(torch.uint8).numpy(), B8.view(torch.uint8).numpy(), sa.numpy(), sb.numpy())
    d = cuda_device
    got = fp8_gemm(A8.to(d), B8.to(d), sa.to(d), sb.to(d))
    assert gemm_status() == 0
    _check(got, torch.from_numpy(ref), K)
    got2 = fp8_gemm(A8.to(d), B8.t().contiguous().to(d), sa.to(d), sb.to(d), b_is_nk=True)
    assert torch.equal(got, got2)          # same kernel, same operands: identical bits


@pytest.mark.parametrize("shape", [(2048, 1024, 768), (1280, 3072, 768), (1024, 768, 3072)])
def test_against_float64_product(cuda_device, shape):
    from deep_optimization_b200.gemm import fp8_gemm, gemm_status
    M, N, K = shape
    A8, B8, sa, sb = _operands(M, N, K, seed=1)
    d = cuda_device
    got = fp8_gemm(A8.to(d), B8.to(d), sa.to(d), sb.to(d))
    assert gemm_status() == 0
    ref = (A8.to(d).double() @ B8.to(d).double()) * sa.to(d).double()[:, None] * sb.to(d).double()[None, :]
    _check(got, ref, K)


def _full_check(cuda_device, oracle, M, N, K, seed, layouts=(False, True), oracle_rows=48):
    """Whole output against the float64 product on the GPU, a row sample against the C oracle
    (double accumulation, bf16 bits compared as values), abort word clear, both B layouts."""
    from deep_optimization_b200.gemm import fp8_gemm, gemm_status
    d = cuda_device
    g = torch.Generator(device=d).manual_seed(seed)
    from deep_optimization_b200.gemm import quantize_e4m3
    A8, sa = quantize_e4m3(torch.randn(M, K, device=d, generator=g), 1)
    B8, sb = quantize_e4m3(torch.randn(K, N, device=d, generator=g), 0)
    ref = (A8.double() @ B8.double()) * sa.double()[:, None] * sb.double()[None, :]
    rows = torch.linspace(0, M - 1, min(M, oracle_rows), device=d).long().unique()
    _, want_rows = oracle.fp8_gemm(A8[rows].cpu().view(torch.uint8).numpy(), B8.cpu().view(torch.uint8).numpy(),
                                   sa[rows].cpu().numpy(), sb.cpu().numpy())
    first = None
    for b_is_nk in layouts:
        Bop = B8.t().contiguous() if b_is_nk else B8
        C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=d)
        fp8_gemm(A8, Bop, sa, sb, b_is_nk=b_is_nk, out=C)
        assert gemm_status() == 0
        assert not torch.isnan(C).any(), "part of C was never written"
        _check(C, ref, K)
        _check(C[rows], torch.from_numpy(want_rows), K)
        if first is None:
            first = C
        else:
            assert torch.equal(first, C)       # same kernel and operands: the layouts agree bit for bit
    del ref


# More tiles than the 148 CTAs of the persistent grid, odd and uneven tile counts per CTA, ragged
# edges: the second accumulator buffer, every mbarrier phase flip and the ring carried from one
# tile to the next all run here.  (M, N, K): tiles = ceil(M/128) * ceil(N/256).
@pytest.mark.parametrize("shape", [(5000, 1024, 256),        # 40 x 4 = 160 tiles: 12 CTAs take two
                                   (128 * 151, 768, 384),    # 453 tiles: 3 per CTA and 9 take a fourth
                                   (4096, 4096, 256),        # 512 tiles, two k-blocks each
                                   (4096, 2304, 384),        # 288 tiles, three k-blocks: the ring phase drifts
                                   (4100, 2312, 400),        # ragged M, N and K (K % 128 != 0)
                                   (19000, 520, 144),        # 447 tiles with a 8-column last tile, 2 k-blocks
                                   (12800, 256, 2048)])      # 100 tiles of 16 k-blocks on 100 CTAs, then ...
def test_persistent_multi_tile(oracle, cuda_device, shape):
    M, N, K = shape
    _full_check(cuda_device, oracle, M, N, K, seed=M + N + K)


# The three shapes of the evaluation configuration (M, K, N) = (8192,4096,4096), (50432,768,3072),
# (50432,3072,768): 1024 / 4728 / 1182 tiles.
@pytest.mark.parametrize("shape", [(8192, 4096, 4096), (50432, 3072, 768), (50432, 768, 3072)])
def test_evaluation_shapes(oracle, cuda_device, shape):
    M, N, K = shape
    _full_check(cuda_device, oracle, M, N, K, seed=5)
    torch.cuda.empty_cache()


def test_two_calls_back_to_back_keep_their_results(cuda_device):
    """Two GEMMs in flight on one stream with different operands and outputs: the second must not
    disturb the first (nothing but the abort word is shared between launches)."""
    from deep_optimization_b200.gemm import fp8_gemm, gemm_status, quantize_e4m3
    d = cuda_device
    g = torch.Generator(device=d).manual_seed(3)
    ops = []
    for (M, N, K) in ((6000, 1536, 512), (3000, 2048, 640)):
        A8, sa = quantize_e4m3(torch.randn(M, K, device=d, generator=g), 1)
        B8, sb = quantize_e4m3(torch.randn(N, K, device=d, generator=g), 1)
        ops.append((A8, B8, sa, sb))
    outs = [fp8_gemm(A8, B8, sa, sb, b_is_nk=True) for (A8, B8, sa, sb) in ops]
    assert gemm_status() == 0
    for (A8, B8, sa, sb), C in zip(ops, outs):
        ref = (A8.double() @ B8.double().t()) * sa.double()[:, None] * sb.double()[None, :]
        _check(C, ref, A8.shape[1])


def test_linearity_and_identity(cuda_device):
    """Size-independent properties: an identity B returns A scaled, and doubling sa doubles C."""
    from deep_optimization_b200.gemm import fp8_gemm
    d = cuda_device
    K = 256
    A = (torch.randint(-8, 9, (512, K)).float()).to(torch.float8_e4m3fn).to(d)
    eye = torch.eye(K).to(torch.float8_e4m3fn).to(d)
    ones_m, ones_n = torch.ones(512, device=d), torch.ones(K, device=d)
    C = fp8_gemm(A, eye, ones_m, ones_n)
    assert torch.equal(C.float(), A.float())
    C2 = fp8_gemm(A, eye, 2 * ones_m, ones_n)
    assert torch.equal(C2.float(), 2 * A.float())


def test_argument_errors(cuda_device):
    from deep_optimization_b200 import _lib
    from deep_optimization_b200.gemm import fp8_gemm
    d = cuda_device
    A = torch.zeros(16, 24, device=d).to(torch.float8_e4m3fn)       # K not a multiple of 16
    B = torch.zeros(24, 16, device=d).to(torch.float8_e4m3fn)
    with pytest.raises(_lib.ActLibraryError):
        fp8_gemm(A, B, torch.ones(16, device=d), torch.ones(16, device=d))


@pytest.mark.parametrize("case", range(4))
def test_against_reference_kernel_fixture(cuda_device, case):
    """The CUDA kernel against outputs of the reference's own Triton GEMM kernel
    (tests/golden/reference_triton_linear.npz, made by tests/golden/make_reference_fixtures.py):
    scales of one.  Integer-operand cases: every product and partial sum is exact in fp32, so the
    only rounding is the final one to bf16 and the comparison is exact.  Random cases: within the
    GEMM tolerance."""
    import os
    from deep_optimization_b200.gemm import fp8_gemm, gemm_status
    fx = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_triton_linear.npz"))
    A8 = torch.from_numpy(fx[f"case{case}_A8"]).view(torch.float8_e4m3fn)
    B8 = torch.from_numpy(fx[f"case{case}_B8"]).view(torch.float8_e4m3fn)
    want = torch.from_numpy(fx[f"case{case}_C"])
    M, K = A8.shape
    N = B8.shape[1]
    d = cuda_device
    got = fp8_gemm(A8.to(d), B8.to(d), torch.ones(M, device=d), torch.ones(N, device=d))
    assert gemm_status() == 0
    if str(fx[f"case{case}_kind"]) == "int":
        assert torch.equal(got.cpu(), want.to(torch.bfloat16))       # exact sums, one rounding to bf16
    else:
        _check(got, want, K)


# ------------------------------------------------- weight gradient from the packed input
def _dw_case(cuda_device, M, N, K, bits, gs, seed=0):
    """dW from the packed input against (a) the float64 product of dy with the dequantised input
    and (b) the unfused path, dequant_unpack + matmul in bf16 with fp32 accumulation."""
    from deep_optimization_b200 import codec
    from deep_optimization_b200.gemm import dw_from_packed, dw_status
    g = torch.Generator(device=cuda_device).manual_seed(seed)
    x = torch.nn.functional.gelu(torch.randn(M, K, device=cuda_device, generator=g)).to(torch.bfloat16)
    dy = (torch.randn(M, N, device=cuda_device, generator=g) * 0.1).to(torch.bfloat16)
    packed, scale, mn = codec.quant_pack(x, bits, gs, seed=3, offset=1)
    xq = codec.dequant_unpack(packed, scale, mn, bits, gs, out_dtype=torch.bfloat16).view(M, K)
    dw = torch.full((N, K), float("nan"), device=cuda_device)
    dw_from_packed(dy, packed, scale, mn, bits, gs, K, out=dw)
    assert dw_status() == 0
    assert not torch.isnan(dw).any()
    ref = dy.double().t() @ xq.double()
    # fp32 accumulation of M products of bf16 values, summed in slices: well inside 2^-10 of the
    # row's scale; the decoded operand is bit-identical to the unfused path's
    tol = ref.abs() * 2.0 ** -10 + ref.abs().max() * 2.0 ** -13 + 1e-6
    err = (dw.double() - ref).abs()
    assert (err <= tol).all(), f"max err {err.max().item()} vs tol {tol.min().item()}"
    return dw, ref


# (M, N, K, group): one stage; a single 8-row tile; ragged M, N and K with 32-element groups (K = 160);
# several slices of M; more tiles than SMs would need N*K > 148 tiles, covered by (3000, 2048, 5120)
@pytest.mark.parametrize("shape", [(64, 256, 256, 128), (128, 8, 128, 128), (1000, 264, 160, 32), (4096, 768, 256, 256),
                                   (50432 // 8, 512, 768, 128), (3000, 2048, 5120, 512)])
def test_dw_from_packed_two_bits(cuda_device, shape):
    M, N, K, gs = shape
    _dw_case(cuda_device, M, N, K, 2, gs)


@pytest.mark.parametrize("bits", (1, 4, 8))
@pytest.mark.parametrize("gs", (32, 256))
def test_dw_from_packed_other_widths(cuda_device, bits, gs):
    _dw_case(cuda_device, 1500, 384, 512, bits, gs, seed=bits)


@pytest.mark.parametrize("shape", [(50432, 3072, 768), (50432, 768, 3072)])
def test_dw_from_packed_vit_shapes(cuda_device, shape):
    """The two MLP weight gradients of ViT-B/16 at batch 256 (M = 256 * 197)."""
    M, N, K = shape
    _dw_case(cuda_device, M, N, K, 2, 128)
