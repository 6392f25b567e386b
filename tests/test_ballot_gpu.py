"""GPU parity of the legacy ballot-plane codec (cpp_extension.pack_mixed_precision_cuda /
unpack_mixed_precision_cuda) and of the bounds-checked copy against the CPU oracle, plus guard
bands around every output of the main entry points: a kernel that writes one byte past the end of
a buffer passes an oracle comparison of the buffer's contents, so each output here is a slice of a
larger allocation whose margins must keep their fill pattern."""
import numpy as np
import pytest
import torch

from tests.inputs import relu_normal, to_numpy

pytestmark = pytest.mark.gpu

DTYPES = (torch.float32, torch.bfloat16, torch.float16)
_NP = {torch.float32: np.float32, torch.float16: np.float16, torch.bfloat16: np.uint16}


def _bits_of(t):
    if t.dtype == torch.bfloat16:
        return t.cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.cpu().numpy()


@pytest.mark.parametrize("dtype", DTYPES, ids=("f32", "bf16", "f16"))
@pytest.mark.parametrize("bits", (1, 2, 3, 4, 8))
@pytest.mark.parametrize("gs", (32, 256))
def test_mixed_precision_pack_unpack_bit_exact(oracle, cuda_device, dtype, bits, gs):
    from deep_optimization_b200 import cpp_extension as cx
    N, G = 5, 7                                            # 35 groups: not a multiple of anything
    x = (relu_normal((N, G, gs), seed=bits + gs, dtype=torch.float32) * 3 - 0.5).to(dtype)
    mn, mx = x.float().amin(-1).to(dtype), x.float().amax(-1).to(dtype)
    arr, tag = to_numpy(x)
    a_mn, _ = to_numpy(mn)
    a_mx, _ = to_numpy(mx)
    for ref_bias in (False, True):
        packed, scale = cx.pack_mixed_precision_cuda(x.to(cuda_device), mn.to(cuda_device), mx.to(cuda_device), bits,
                                                     True, seed=99, ref_bias=ref_bias)
        want_p, want_s = oracle.pack_ballot(arr.reshape(-1, gs), a_mn.reshape(-1), a_mx.reshape(-1), gs, bits, seed=99,
                                            flags=oracle.FLAG_BALLOT_REF_BIAS if ref_bias else 0, dtype=tag)
        assert scale.shape == (N, G, 1) and packed.numel() == N * G * (gs // 32) * bits
        assert np.array_equal(_bits_of(scale).reshape(-1).view(want_s.dtype), want_s), "scale differs"
        assert np.array_equal(packed.cpu().numpy().view(np.uint32), want_p), "packed words differ"
        y = cx.unpack_mixed_precision_cuda(packed, bits, scale, mn.to(cuda_device), N, G, gs)
        want_y = oracle.unpack_ballot(want_p, want_s, a_mn.reshape(-1), gs, bits, dtype=tag)
        assert y.shape == (N, G, gs) and y.dtype == dtype
        assert np.array_equal(_bits_of(y).reshape(-1, gs).view(want_y.dtype), want_y), "decoded values differ"
    # the unbiased form stays within one step of the input
    step = 1.0 / scale.float()
    tol = step * 1.01 + x.to(cuda_device).float().abs() * (2.0 ** -7 if dtype != torch.float32 else 1e-6)
    packed, scale = cx.pack_mixed_precision_cuda(x.to(cuda_device), mn.to(cuda_device), mx.to(cuda_device), bits, True, seed=5)
    y = cx.unpack_mixed_precision_cuda(packed, bits, scale, mn.to(cuda_device), N, G, gs)
    assert ((y.float() - x.to(cuda_device).float()).abs() <= tol).all()


def test_copy_launch_is_bounds_checked(cuda_device):
    from deep_optimization_b200 import _lib, cpp_extension as cx
    for dtype in (torch.float32, torch.bfloat16, torch.float8_e4m3fn):
        src = torch.randn(3, 4, 256, device=cuda_device).to(dtype)
        dst = torch.zeros_like(src)
        cx.copy_launch(src, dst, 3, 4)
        assert torch.equal(src.view(torch.uint8), dst.view(torch.uint8))
    small = torch.zeros(3, 3, 256, device=cuda_device)
    with pytest.raises(_lib.ActLibraryError):             # the reference's kernel would write past the end here
        cx.copy_launch(torch.randn(3, 4, 256, device=cuda_device), small, 3, 4)
    assert float(small.abs().sum()) == 0.0


# ------------------------------------------------------------------ guard bands
GUARD = 256
PATTERN = 0xA5


class Guarded:
    """Outputs carved out of pattern-filled allocations with 256-byte margins on both sides."""

    def __init__(self, device):
        self.device, self.blocks = device, []

    def empty(self, shape, dtype):
        numel = 1
        for d in shape:
            numel *= d
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        pad = (-nbytes) % 16                                   # keep the tail margin 16-byte aligned
        raw = torch.full((GUARD + nbytes + pad + GUARD,), PATTERN, dtype=torch.uint8, device=self.device)
        self.blocks.append((raw, nbytes))
        return raw[GUARD:GUARD + nbytes].view(dtype).view(shape)

    def check(self, what):
        torch.cuda.synchronize()
        for raw, nbytes in self.blocks:
            assert bool((raw[:GUARD] == PATTERN).all()), f"{what}: bytes before an output were overwritten"
            assert bool((raw[GUARD + nbytes:] == PATTERN).all()), f"{what}: bytes after an output were overwritten"
        self.blocks = []


@pytest.mark.parametrize("dtype", DTYPES, ids=("f32", "bf16", "f16"))
@pytest.mark.parametrize("bits", (1, 2, 4, 8))
def test_guard_bands_codec(cuda_device, dtype, bits):
    from deep_optimization_b200 import _lib, codec
    gd = Guarded(cuda_device)
    for gs, ng in ((32, 37), (128, 75), (1024, 3), (256, 1)):          # odd group counts: partial tiles
        x = relu_normal((ng, gs), seed=gs, dtype=dtype).to(cuda_device)
        nwords = gs * bits // 32
        for flags, noise in ((0, None), (0, torch.rand((ng, gs), device=cuda_device)), (_lib.ACT_FLAG_ROUND_NEAREST, None),
                             (_lib.ACT_FLAG_REF_COMPAT | _lib.ACT_FLAG_META_BF16, None)):
            out = (gd.empty((ng, nwords), torch.int32), gd.empty((ng,), torch.float32), gd.empty((ng,), torch.float32))
            codec.quant_pack(x, bits, gs, noise=noise, flags=flags, out=out)
            gd.check(f"quant_pack g{gs} flags{flags}")
            y = gd.empty((ng, gs), dtype)
            codec.dequant_unpack(*out, bits, gs, out_dtype=dtype, out=y)
            gd.check(f"dequant_unpack g{gs}")


def test_guard_bands_other_entries(cuda_device):
    """The entries that allocate their own outputs are called through the C ABI with guarded
    buffers: mask pack / unpack, 3-bit planes, sub-group averaging, tiles, ReLU, the fused
    activation and batch-norm kernels (both layouts), ballot codec, GEMM."""
    from deep_optimization_b200 import _lib, codec
    lib = _lib.load()
    gd = Guarded(cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    BF = _lib.ACT_DTYPE_BF16
    chk = lambda rc, what: (_lib.check(rc, what), gd.check(what))
    # mask pack / unpack: 37 groups of 64 int8
    m = (torch.rand(37, 64, device=cuda_device) > 0.5).to(torch.int8)
    pk = gd.empty((37, 2), torch.int32)
    chk(lib.act_pack_bits(m.data_ptr(), 37, 64, 1, pk.data_ptr(), st), "act_pack_bits")
    un = gd.empty((37, 64), torch.int8)
    chk(lib.act_unpack_bits(pk.data_ptr(), 37, 64, 1, un.data_ptr(), st), "act_unpack_bits")
    assert torch.equal(un, m)
    # relu forward (y + mask) and backward on 75 * 128 elements
    x = torch.randn(75 * 128, device=cuda_device).to(torch.bfloat16)
    y, mask = gd.empty((75 * 128,), torch.bfloat16), gd.empty((75 * 128 // 8,), torch.uint8)
    chk(lib.act_relu_fwd_pack(x.data_ptr(), BF, 75 * 128, 0, y.data_ptr(), mask.data_ptr(), st), "act_relu_fwd_pack")
    dx = gd.empty((75 * 128,), torch.bfloat16)
    chk(lib.act_relu_bwd_unpack(mask.data_ptr(), x.data_ptr(), BF, 75 * 128, dx.data_ptr(), st), "act_relu_bwd_unpack")
    # fused activation forward / backward, 75 groups of 128
    for kind in (_lib.ACT_KIND_GELU, _lib.ACT_KIND_SILU, _lib.ACT_KIND_GELU_ERF):
        y = gd.empty((75, 128), torch.bfloat16)
        pk, sc, mn = gd.empty((75, 8), torch.int32), gd.empty((75,), torch.float32), gd.empty((75,), torch.float32)
        chk(lib.act_activation_fwd_quant_pack(x.data_ptr(), BF, kind, 75, 128, 2, 1, 2, 0, y.data_ptr(), pk.data_ptr(),
                                              sc.data_ptr(), mn.data_ptr(), st), "act_activation_fwd_quant_pack")
        dx = gd.empty((75, 128), torch.bfloat16)
        chk(lib.act_mul_dequant_unpack(pk.data_ptr(), sc.data_ptr(), mn.data_ptr(), x.data_ptr(), BF, 75, 128, 2,
                                       dx.data_ptr(), st), "act_mul_dequant_unpack")
    # 3-bit planes and sub-group averaging through the Python wrappers' out= buffers
    x3 = relu_normal((35, 256), 3, torch.bfloat16).to(cuda_device)
    out = (gd.empty((35, 24), torch.int32), gd.empty((35,), torch.float32), gd.empty((35,), torch.float32))
    codec.quant_pack(x3, 3, 256, out=out, planes3=True)
    gd.check("quant_pack 3-bit")
    y = gd.empty((35, 256), torch.bfloat16)
    codec.dequant_unpack(*out, 3, 256, out_dtype=torch.bfloat16, out=y, planes3=True)
    gd.check("dequant_unpack 3-bit")
    # ballot codec: 35 groups of 96 (three chunks), 3 bits
    xb = torch.rand(35, 96, device=cuda_device)
    mnb, mxb = xb.amin(1).contiguous(), xb.amax(1).contiguous()
    pk, sc = gd.empty((35 * 3 * 3,), torch.int32), gd.empty((35,), torch.float32)
    chk(lib.act_pack_ballot(xb.data_ptr(), _lib.ACT_DTYPE_F32, 35, 96, 3, mnb.data_ptr(), mxb.data_ptr(), 7, 0,
                            pk.data_ptr(), sc.data_ptr(), st), "act_pack_ballot")
    yb = gd.empty((35, 96), torch.float32)
    chk(lib.act_unpack_ballot(pk.data_ptr(), sc.data_ptr(), mnb.data_ptr(), _lib.ACT_DTYPE_F32, 35, 96, 3, yb.data_ptr(), st),
        "act_unpack_ballot")
    # copy: 1000 bytes (not a multiple of 16)
    src = torch.randint(0, 255, (1008,), dtype=torch.uint8, device=cuda_device)
    dst = gd.empty((1000,), torch.uint8)
    chk(lib.act_copy(src.data_ptr(), dst.data_ptr(), 1000, 1008, 1000, st), "act_copy")
    assert torch.equal(dst, src[:1000])
    # GEMM with ragged M and N: the bulk tensor stores are clipped at the edges of C
    from deep_optimization_b200.gemm import gemm_status, quantize_e4m3
    for (M, N, K) in ((300, 264, 144), (100, 72, 64)):                 # CTA pairs / single CTA
        A8, sa = quantize_e4m3(torch.randn(M, K, device=cuda_device), 1)
        B8, sb = quantize_e4m3(torch.randn(N, K, device=cuda_device), 1)
        C = gd.empty((M, N), torch.bfloat16)
        chk(lib.act_fp8_gemm(A8.data_ptr(), B8.data_ptr(), sa.data_ptr(), sb.data_ptr(), C.data_ptr(), M, N, K, K, K, N,
                             _lib.ACT_GEMM_B_IS_NK, None, 0, st), f"act_fp8_gemm {M}x{N}x{K}")
        assert gemm_status() == 0
        ref = (A8.double() @ B8.double().t()) * sa.double()[:, None] * sb.double()[None, :]
        assert ((C.double() - ref).abs() <= ref.abs() * 2.0 ** -8 + ref.abs().max() * 2.0 ** -12 + 1e-6).all()


@pytest.mark.parametrize("channels_last", (False, True))
def test_guard_bands_batch_norm(cuda_device, channels_last):
    """The fused batch-norm entries with guarded outputs, HW = 36 (a multiple of 4 but not of 8)
    in NCHW and C = 24 channel-minor."""
    from deep_optimization_b200 import _lib
    lib = _lib.load()
    gd = Guarded(cuda_device)
    st = torch.cuda.current_stream().cuda_stream
    N, C, H, W = 8, 24, 6, 6
    n = N * C * H * W
    gs, bits = 64, 2
    fmt = torch.channels_last if channels_last else torch.contiguous_format
    x = torch.randn(N, C, H, W, device=cuda_device).to(torch.bfloat16).contiguous(memory_format=fmt)
    dy = torch.randn(N, C, H, W, device=cuda_device).to(torch.bfloat16).contiguous(memory_format=fmt)
    nb, hw = (N * H * W, 1) if channels_last else (N, H * W)
    w, b = torch.ones(C, device=cuda_device), torch.zeros(C, device=cuda_device)
    ws_bytes = lib.act_bn_stats_workspace(nb * C * hw, C)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=cuda_device)
    params = gd.empty((C, 4), torch.float32)
    _lib.check(lib.act_bn_stats(x.data_ptr(), _lib.ACT_DTYPE_BF16, nb, C, hw, 1e-5, w.data_ptr(), b.data_ptr(), None, None,
                                0.0, params.data_ptr(), ws.data_ptr(), ws_bytes, st), "act_bn_stats")
    gd.check("act_bn_stats")
    params = params.clone()
    y = gd.empty((n,), torch.bfloat16)
    pk, sc, mn = gd.empty((n // gs, gs * bits // 32), torch.int32), gd.empty((n // gs,), torch.float32), gd.empty((n // gs,), torch.float32)
    mask = gd.empty((n // 8,), torch.uint8)
    _lib.check(lib.act_bn_relu_fwd_norm_quant_pack(x.data_ptr(), _lib.ACT_DTYPE_BF16, nb, C, hw, params.data_ptr(), gs, bits,
                                                   3, 4, 0, y.data_ptr(), pk.data_ptr(), sc.data_ptr(), mn.data_ptr(),
                                                   mask.data_ptr(), st), "act_bn_relu_fwd_norm_quant_pack")
    gd.check("act_bn_relu_fwd_norm_quant_pack")
    pk, sc, mn, mask = pk.clone(), sc.clone(), mn.clone(), mask.clone()
    sums = gd.empty((2, C), torch.float32)
    sums.zero_()
    _lib.check(lib.act_bn_relu_bwd_reduce(pk.data_ptr(), sc.data_ptr(), mn.data_ptr(), mask.data_ptr(), dy.data_ptr(),
                                          _lib.ACT_DTYPE_BF16, nb, C, hw, gs, bits, sums.data_ptr(), st), "act_bn_relu_bwd_reduce")
    gd.check("act_bn_relu_bwd_reduce")
