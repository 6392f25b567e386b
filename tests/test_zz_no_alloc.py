"""The allocation-free GEMM entry point, called through the C ABI.

`act_fp8_gemm_static` serves callers that cannot obtain device memory when they
call (a plugin inside another framework's memory plan, a loop that bans allocator
calls): its staging buffer is an array inside the library.  The test runs it twice
in a row on different operands and checks each result against the ordinary entry
point, which takes a caller-owned workspace.  It sits in a file that sorts last so
that a run stopping at the first failure has already been through everything else;
it also passes when run alone in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed, dev):
    from deep_optimization_b200.gemm import quantize_e4m3
    g = torch.Generator().manual_seed(seed)
    A8, sa = quantize_e4m3(torch.randn(M, K, generator=g), 1)
    B8, sb = quantize_e4m3(torch.randn(K, N, generator=g), 0)
    return A8.to(dev), B8.to(dev), sa.to(dev), sb.to(dev)


def _static_gemm(lib, A8, B8, sa, sb):
    M, K = A8.shape
    N = B8.shape[1]
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=A8.device)
    rc = lib.act_fp8_gemm_static(A8.data_ptr(), B8.data_ptr(), sa.data_ptr(), sb.data_ptr(), C.data_ptr(),
                                 M, N, K, A8.stride(0), B8.stride(0), C.stride(0),
                                 torch.cuda.current_stream().cuda_stream)
    return rc, C


def test_static_scratch_gemm_matches_workspace_gemm(cuda_device):
    from deep_optimization_b200 import _lib
    from deep_optimization_b200.gemm import fp8_gemm, gemm_status
    lib = _lib.load()
    assert lib.act_fp8_gemm_static_limit() == 4 << 20
    # two calls in a row, different shapes and data: the second must not see the first's scratch
    for seed, (M, N, K) in enumerate([(384, 768, 1024), (256, 1024, 512)]):
        A8, B8, sa, sb = _operands(M, N, K, seed, cuda_device)
        rc, got = _static_gemm(lib, A8, B8, sa, sb)
        assert rc == 0, lib.act_strerror(rc)
        want = fp8_gemm(A8, B8, sa, sb)                  # existing entry point, caller-owned workspace
        assert gemm_status() == 0
        g, w = got.double(), want.double()
        tol = w.abs() * 2.0 ** -8 + w.abs().max() * 2.0 ** -12 + 1e-6       # the GEMM tests' tolerance
        assert not torch.isnan(g).any()
        assert ((g - w).abs() <= tol).all()


def test_static_scratch_gemm_rejects_large_problems(cuda_device):
    from deep_optimization_b200 import _lib
    lib = _lib.load()
    p = ctypes.c_void_p(256)                              # never dereferenced: the size check comes first
    rc = lib.act_fp8_gemm_static(p, p, p, p, p, 128, 4096, 4096, 4096, 4096, 4096, None)
    assert rc == 12 and b"built-in scratch" in lib.act_strerror(rc)
