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
