"""GPU tests of the producer/consumer-fused kernels against their unfused compositions."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = (torch.float32, torch.bfloat16, torch.float16)


@pytest.mark.parametrize("dtype", DTYPES, ids=("f32", "bf16", "f16"))
@pytest.mark.parametrize("relu6", (False, True))
def test_relu_fused_bit_exact(oracle, cuda_device, dtype, relu6):
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(37 * 1024 + 96, generator=g) * 4).to(dtype)
    x[5], x[6], x[7] = 0.0, -0.0, float("nan")
    xd = x.to(cuda_device)
    y, bits = codec.relu_fwd_pack(xd, relu6=relu6)
    keep = (x > 0) & (x < 6) if relu6 else (x > 0)
    want_y = torch.where(keep, x, torch.zeros((), dtype=dtype))
    assert torch.equal(y.cpu(), want_y)
    want_bits = oracle.pack_bits(keep.to(torch.int8).numpy(), 32, 1).reshape(-1)
    assert np.array_equal(bits.cpu().numpy().view(np.uint32), want_bits)
    dy = torch.randn(x.shape, generator=g).to(dtype)
    dx = codec.relu_bwd_unpack(bits, dy.to(cuda_device))
    assert torch.equal(dx.cpu(), torch.where(keep, dy, torch.zeros((), dtype=dtype)))


@pytest.mark.parametrize("kind", ("gelu", "silu"))
@pytest.mark.parametrize("bits", (2, 8))
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16), ids=("f32", "bf16"))
def test_activation_fused_forward(oracle, cuda_device, kind, bits, dtype):
    """y within the output type's rounding of the exact activation; the packed derivative
    decodes to within one quantisation step (+ the hardware tanh/exp error, 2^-10) of the
    exact derivative; scale/min equal those of the derivative tensor up to that error."""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(64, 2048, generator=g) * 2).to(dtype)
    xd = x.to(cuda_device)
    gs = 256
    y, packed, scale, mn = codec.activation_fwd_quant_pack(xd, kind, bits, gs, seed=5, offset=1)
    xr = xd.double().requires_grad_()
    yr = torch.nn.functional.gelu(xr, approximate="tanh") if kind == "gelu" else torch.nn.functional.silu(xr)
    (dr,) = torch.autograd.grad(yr.sum(), xr)
    ytol = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -10
    assert (y.double() - yr).abs().max() <= ytol * (1 + yr.abs().max())
    d = codec.dequant_unpack(packed, scale, mn, bits, gs, out_dtype=torch.float32).view_as(xd)
    step = scale.view(-1, 1).expand(-1, gs).reshape(xd.shape)
    assert ((d.double() - dr).abs() <= step.double() * 1.001 + 2e-3).all()
    dmin = dr.view(-1, gs).amin(1)
    assert (mn.double() - dmin).abs().max() <= 2e-3
    # backward: dy * decoded derivative, exactly what the separate kernels compute
    dy = torch.randn(x.shape, generator=g).to(dtype).to(cuda_device)
    dx = codec.mul_dequant_unpack(packed, scale, mn, dy, bits, gs)
    want = (dy.float() * d).to(dtype)
    assert torch.equal(dx, want)


def test_fused_paths_in_layers(cuda_device):
    """The modules take the fused kernels when no padding is needed and give the same
    gradients as PyTorch's own activations (ReLU exactly, GELU within the 8-bit step)."""
    from deep_optimization_b200.modules.activations.act_layers import DOGELU, DOReLU_Variance
    meta = {"r": {"bits": 1, "pack_only": True, "group_size": 256, "act_padding": False, "N": 8,
                  "AVG_ALAM": False, "ALAM_BITS": 0, "DIVISION": None},
            "g": {"bits": 8, "pack_only": False, "group_size": 256, "act_padding": False, "N": 8,
                  "AVG_ALAM": False, "ALAM_BITS": 0, "DIVISION": None}}
    x = torch.randn(8, 4, 16, 16, device=cuda_device, requires_grad=True)
    xr = x.detach().clone().requires_grad_()
    g = torch.randn_like(x)
    relu = DOReLU_Variance(target_name="r", meta=meta).to(cuda_device).train()
    y = relu(x); y.backward(g); torch.relu(xr).backward(g)
    assert torch.equal(y, torch.relu(xr)) and torch.equal(x.grad, xr.grad)
    x.grad = None; xr.grad = None
    gelu = DOGELU(target_name="g", meta=meta).to(cuda_device).train()
    y = gelu(x); y.backward(g)
    yr = torch.nn.functional.gelu(xr, approximate="tanh"); yr.backward(g)
    assert torch.allclose(y, yr, atol=2e-3)
    assert (x.grad - xr.grad).abs().max() < 0.02 * g.abs().max()


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16), ids=("f32", "bf16"))
@pytest.mark.parametrize("shape", [(8, 16, 32, 32), (6, 24, 14, 14), (8, 5, 2, 2), (16, 64, 56, 56)])
def test_bn_fused_forward(oracle, cuda_device, dtype, shape):
    """x_hat = (x - mean) * invstd with both steps rounded to fp32: the packed codes, scale and
    min must be bit-exact with the oracle applied to that fp32 tensor; y within the output
    type's rounding of x_hat * w + b."""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(shape, generator=g) * 2 + 0.5).to(dtype).to(cuda_device)
    C = shape[1]
    mean = torch.randn(C, generator=g).to(cuda_device)
    invstd = (torch.rand(C, generator=g) + 0.5).to(cuda_device)
    w = torch.randn(C, generator=g).to(cuda_device)
    b = torch.randn(C, generator=g).to(cuda_device)
    gs = 64 if x.numel() % 256 else 256
    if x.numel() % gs:
        gs = 32
    assert codec.bn_fused_supported(x, gs)
    y, packed, scale, mn = codec.bn_fwd_norm_quant_pack(x, mean, invstd, w, b, 2, gs, seed=3, offset=2)
    view = [1, C, 1, 1]
    x_hat = (x.float() - mean.view(view)) * invstd.view(view)           # fp32, two roundings
    want = oracle.quant_pack(x_hat.cpu().numpy(), gs, 2, seed=3, offset=2)
    assert np.array_equal(packed.cpu().numpy().view(np.uint32), want[0])
    assert np.array_equal(scale.cpu().numpy().view(np.uint32), want[1].view(np.uint32))
    assert np.array_equal(mn.cpu().numpy().view(np.uint32), want[2].view(np.uint32))
    y_ref = x_hat * w.view(view) + b.view(view)
    assert torch.equal(y, y_ref.to(dtype))


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16), ids=("f32", "bf16"))
@pytest.mark.parametrize("shape", [(8, 16, 32, 32), (6, 24, 14, 14), (8, 5, 2, 2)])
@pytest.mark.parametrize("bits", (2, 8))
def test_bn_fused_backward(cuda_device, dtype, shape, bits):
    """Sums and dx from the packed x_hat equal the same formulas on the decoded tensor
    (sums: fp32 accumulation in another order, relative 1e-4; dx: one output rounding)."""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(6)
    xh = torch.randn(shape, generator=g).to(cuda_device)
    dy = torch.randn(shape, generator=g).to(dtype).to(cuda_device)
    C = shape[1]
    gs = 32
    packed, scale, mn = codec.quant_pack(xh, bits, gs, seed=1, offset=0)
    dec = codec.dequant_unpack(packed, scale, mn, bits, gs, out_dtype=torch.float32).view(shape)
    s1, s2 = codec.bn_bwd_reduce(packed, scale, mn, dy, bits, gs)
    dims = [0, 2, 3]
    r1, r2 = (dy.float() * dec).sum(dims), dy.float().sum(dims)
    assert torch.allclose(s1, r1, rtol=1e-4, atol=1e-3 * r1.abs().max().item())
    assert torch.allclose(s2, r2, rtol=1e-4, atol=1e-3 * r2.abs().max().item() + 1e-3)
    k1, k2, k3 = (torch.randn(C, generator=g).to(cuda_device) for _ in range(3))
    dx = codec.bn_bwd_dx(packed, scale, mn, dy, k1, k2, k3, bits, gs)
    view = [1, C, 1, 1]
    want = k1.view(view) * dy.float() - k2.view(view) - k3.view(view) * dec
    tol = 2.0 ** -7 if dtype == torch.bfloat16 else 1e-5
    assert ((dx.float() - want).abs() <= tol * (1 + want.abs())).all()


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16, torch.float16), ids=("f32", "bf16", "f16"))
@pytest.mark.parametrize("shape", [(8, 16, 32, 32), (6, 24, 14, 14), (8, 5, 2, 2), (64, 64, 56, 56), (3, 130, 4, 4)])
def test_bn_stats(cuda_device, dtype, shape):
    """Mean and inverse deviation against float64 statistics of the same tensor (the kernel
    sums in fp32 per block around a pivot and combines in double: relative 2e-5), a large
    offset included; identical from run to run; running statistics as nn.BatchNorm2d updates them."""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(8)
    C = shape[1]
    offset = torch.linspace(-50, 50, C).view(1, C, 1, 1)
    x = (torch.randn(shape, generator=g) * 1.5 + offset).to(dtype).to(cuda_device)
    w = torch.randn(C, generator=g).to(cuda_device)
    b = torch.randn(C, generator=g).to(cuda_device)
    rm = torch.randn(C, generator=g).to(cuda_device)
    rv = (torch.rand(C, generator=g) + 0.5).to(cuda_device)
    rm0, rv0 = rm.clone(), rv.clone()
    eps, mom = 1e-5, 0.1
    params = codec.bn_stats(x, eps, w, b, rm, rv, mom)
    xd = x.double()
    mean = xd.mean((0, 2, 3))
    var = xd.var((0, 2, 3), unbiased=False)
    M = x.numel() // C
    assert torch.allclose(params[:, 0].double(), mean, rtol=2e-5, atol=2e-5)
    assert torch.allclose(params[:, 1].double(), 1.0 / torch.sqrt(var + eps), rtol=2e-5)
    assert torch.equal(params[:, 2], w) and torch.equal(params[:, 3], b)
    assert torch.allclose(rm.double(), 0.9 * rm0.double() + 0.1 * mean, rtol=1e-5, atol=1e-5)
    assert torch.allclose(rv.double(), 0.9 * rv0.double() + 0.1 * var * M / max(M - 1, 1), rtol=1e-4)
    again = codec.bn_stats(x, eps)
    assert torch.equal(again[:, :2], codec.bn_stats(x, eps)[:, :2])
    assert torch.equal(again[:, 0], params[:, 0]) and torch.equal(again[:, 1], params[:, 1])
    assert (again[:, 2] == 1).all() and (again[:, 3] == 0).all()


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16), ids=("f32", "bf16"))
@pytest.mark.parametrize("shape", [(8, 16, 32, 32), (6, 24, 14, 14), (8, 5, 2, 2)])
def test_bn_relu_fused(oracle, cuda_device, dtype, shape):
    """Forward: the packed x_hat is the one of the kernel without ReLU (bit-exact), y is its y
    clamped at zero and the mask is y > 0.  Backward: sums and dx equal those of the unfused
    kernels fed with dy * mask."""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(15)
    x = (torch.randn(shape, generator=g) * 2 + 0.5).to(dtype).to(cuda_device)
    C = shape[1]
    mean = torch.randn(C, generator=g).to(cuda_device)
    invstd = (torch.rand(C, generator=g) + 0.5).to(cuda_device)
    w = torch.randn(C, generator=g).to(cuda_device)
    b = torch.randn(C, generator=g).to(cuda_device)
    gs = 64 if x.numel() % 256 else 256
    if x.numel() % gs:
        gs = 32
    y0, p0, s0, m0 = codec.bn_fwd_norm_quant_pack(x, mean, invstd, w, b, 2, gs, seed=3, offset=2)
    y1, p1, s1, m1, mask = codec.bn_fwd_norm_quant_pack(x, mean, invstd, w, b, 2, gs, seed=3, offset=2, relu=True)
    assert torch.equal(p0, p1) and torch.equal(s0, s1) and torch.equal(m0, m1)
    assert torch.equal(y1, torch.relu(y0))
    keep = (y0 > 0)
    bits = np.unpackbits(mask.cpu().numpy(), bitorder="little")[: x.numel()].reshape(shape)
    assert np.array_equal(bits.astype(bool), keep.cpu().numpy())
    dy = torch.randn(shape, generator=g).to(dtype).to(cuda_device)
    dym = torch.where(keep, dy, torch.zeros_like(dy))
    a1, b1 = codec.bn_bwd_reduce(p1, s1, m1, dy, 2, gs, mask=mask)
    a0, b0 = codec.bn_bwd_reduce(p1, s1, m1, dym, 2, gs)
    assert torch.allclose(a1, a0, rtol=1e-5, atol=1e-4) and torch.allclose(b1, b0, rtol=1e-5, atol=1e-4)
    k1, k2, k3 = (torch.randn(C, generator=g).to(cuda_device) for _ in range(3))
    d1 = codec.bn_bwd_dx(p1, s1, m1, dy, k1, k2, k3, 2, gs, mask=mask)
    d0 = codec.bn_bwd_dx(p1, s1, m1, dym, k1, k2, k3, 2, gs)
    assert torch.equal(d1, d0)


def test_bn_relu_module_matches_pytorch(cuda_device):
    """DOBatchNorm2d with fuse_relu against BatchNorm2d + ReLU: output exact to rounding,
    gradients within the 8-bit codec's error."""
    from deep_optimization_b200.modules.normalization.normalization_layers import DOBatchNorm2d
    torch.manual_seed(2)
    meta = {"b": {"bits": 8, "pack_only": False, "group_size": 256, "act_padding": False, "N": 8,
                  "AVG_ALAM": False, "ALAM_BITS": 0, "DIVISION": None}}
    bn = DOBatchNorm2d(4, target_name="b", meta=meta).to(cuda_device).train()
    bn.fuse_relu = True
    rb = torch.nn.BatchNorm2d(4).to(cuda_device).train()
    with torch.no_grad():
        bn.weight.copy_(torch.randn(4)); bn.bias.copy_(torch.randn(4))
        rb.weight.copy_(bn.weight); rb.bias.copy_(bn.bias)
    x = torch.randn(8, 4, 16, 16, device=cuda_device, requires_grad=True)
    xr = x.detach().clone().requires_grad_()
    g = torch.randn_like(x)
    y, yr = bn(x), torch.relu(rb(xr))
    assert torch.allclose(y, yr, atol=1e-4)
    y.backward(g); yr.backward(g)
    assert (x.grad - xr.grad).abs().max() < 0.05
    assert (bn.weight.grad - rb.weight.grad).norm() / rb.weight.grad.norm() < 0.03
    assert torch.allclose(bn.bias.grad, rb.bias.grad, rtol=1e-4, atol=1e-3)


def test_bn_bwd_coef(cuda_device):
    """k1 = w * invstd, k2 = k1 * sum(dy) / M, k3 = k1 * sum(dy * x_hat) / M, each product rounded to fp32."""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(21)
    C, M = 37, 5000.0
    sums = torch.randn(2 * C, generator=g).to(cuda_device)
    params = torch.rand(C, 4, generator=g).to(cuda_device) + 0.5
    coef = codec.bn_bwd_coef(sums, params, M)
    k1 = params[:, 2] * params[:, 1]
    inv = torch.tensor(1.0 / M, dtype=torch.float32, device=cuda_device)
    assert torch.equal(coef[:, 0], k1)
    assert torch.equal(coef[:, 1], k1 * sums[C:] * inv)
    assert torch.equal(coef[:, 2], k1 * sums[:C] * inv)
    assert (coef[:, 3] == 0).all()


# ------------------------------------------------------------------ channels-last (channel-minor) batch norm

_CL_SHAPES = [(8, 16, 32, 32), (6, 24, 14, 14), (4, 64, 56, 56), (3, 136, 4, 4), (2, 2048, 7, 7), (5, 8, 3, 5)]


def _cl_group(numel):
    for gs in (256, 128, 64, 32):
        if numel % gs == 0:
            return gs
    return None


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16), ids=("f32", "bf16"))
@pytest.mark.parametrize("shape", _CL_SHAPES)
@pytest.mark.parametrize("relu", (False, True))
def test_bn_fused_forward_channels_last(oracle, cuda_device, dtype, shape, relu):
    """A channels-last activation is normalised and grouped as it lies in memory ([N*H*W, C]):
    codes, scale and min bit-exact with the oracle applied to the fp32 x_hat in NHWC order, y
    exact, y channels-last, mask = y > 0 in memory order."""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(31)
    gs = _cl_group(int(np.prod(shape)))
    if gs is None:
        pytest.skip("no group size divides this shape")
    x = (torch.randn(shape, generator=g) * 2 + 0.5).to(dtype).to(cuda_device).contiguous(memory_format=torch.channels_last)
    C = shape[1]
    mean = torch.randn(C, generator=g).to(cuda_device)
    invstd = (torch.rand(C, generator=g) + 0.5).to(cuda_device)
    w = torch.randn(C, generator=g).to(cuda_device)
    b = torch.randn(C, generator=g).to(cuda_device)
    assert codec.bn_fused_supported(x, gs)
    out = codec.bn_fwd_norm_quant_pack(x, mean, invstd, w, b, 2, gs, seed=3, offset=2, relu=relu)
    y, packed, scale, mn = out[:4]
    assert y.is_contiguous(memory_format=torch.channels_last) and y.shape == x.shape
    view = [1, C, 1, 1]
    x_hat = (x.float() - mean.view(view)) * invstd.view(view)
    nhwc = x_hat.permute(0, 2, 3, 1).contiguous()
    want = oracle.quant_pack(nhwc.cpu().numpy().reshape(-1), gs, 2, seed=3, offset=2)
    assert np.array_equal(packed.cpu().numpy().view(np.uint32).reshape(-1), np.asarray(want[0]).reshape(-1))
    assert np.array_equal(scale.cpu().numpy().view(np.uint32), want[1].view(np.uint32).reshape(-1))
    assert np.array_equal(mn.cpu().numpy().view(np.uint32), want[2].view(np.uint32).reshape(-1))
    y_ref = (x_hat * w.view(view) + b.view(view))
    if relu:
        keep = y_ref > 0
        y_ref = torch.where(keep, y_ref, torch.zeros_like(y_ref))
        bits = np.unpackbits(out[4].cpu().numpy(), bitorder="little")[: x.numel()]
        assert np.array_equal(bits.astype(bool), keep.permute(0, 2, 3, 1).reshape(-1).cpu().numpy())
    assert torch.equal(y, y_ref.to(dtype))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16, torch.float16), ids=("f32", "bf16", "f16"))
@pytest.mark.parametrize("shape", _CL_SHAPES + [(64, 64, 56, 56)])
def test_bn_stats_channels_last(cuda_device, dtype, shape):
    """Statistics of a channels-last tensor equal those of the same values stored NCHW (to the
    tolerance of test_bn_stats against float64), run-to-run identical."""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(8)
    C = shape[1]
    offset = torch.linspace(-50, 50, C).view(1, C, 1, 1)
    x = (torch.randn(shape, generator=g) * 1.5 + offset).to(dtype).to(cuda_device).contiguous(memory_format=torch.channels_last)
    rm = torch.zeros(C, device=cuda_device)
    rv = torch.ones(C, device=cuda_device)
    eps = 1e-5
    params = codec.bn_stats(x, eps, None, None, rm, rv, 0.1)
    xd = x.double()
    mean = xd.mean((0, 2, 3))
    var = xd.var((0, 2, 3), unbiased=False)
    M = x.numel() // C
    assert torch.allclose(params[:, 0].double(), mean, rtol=2e-5, atol=2e-5)
    assert torch.allclose(params[:, 1].double(), 1.0 / torch.sqrt(var + eps), rtol=2e-5)
    assert torch.allclose(rm.double(), 0.1 * mean, rtol=1e-5, atol=1e-5)
    assert torch.allclose(rv.double(), 0.9 + 0.1 * var * M / max(M - 1, 1), rtol=1e-4)
    assert torch.equal(params, codec.bn_stats(x, eps))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16), ids=("f32", "bf16"))
@pytest.mark.parametrize("shape", _CL_SHAPES)
@pytest.mark.parametrize("bits", (2, 8))
@pytest.mark.parametrize("masked", (False, True))
def test_bn_fused_backward_channels_last(cuda_device, dtype, shape, bits, masked):
    """Channel-minor sums and dx against the formulas on the decoded tensor (tolerances of
    test_bn_fused_backward)."""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(6)
    gs = 32
    if int(np.prod(shape)) % gs:
        pytest.skip("numel not a multiple of 32")
    N, C, H, W = shape
    xh_nhwc = torch.randn((N, H, W, C), generator=g).to(cuda_device)
    dy = torch.randn(shape, generator=g).to(dtype).to(cuda_device).contiguous(memory_format=torch.channels_last)
    packed, scale, mn = codec.quant_pack(xh_nhwc, bits, gs, seed=1, offset=0)
    dec = codec.dequant_unpack(packed, scale, mn, bits, gs, out_dtype=torch.float32).view(N, H, W, C).permute(0, 3, 1, 2)
    mask = keep = None
    dyf = dy.float()
    if masked:
        keep = torch.rand(shape, generator=g).to(cuda_device) > 0.4
        flat = keep.permute(0, 2, 3, 1).reshape(-1).cpu().numpy()
        mask = torch.from_numpy(np.packbits(flat, bitorder="little")).to(cuda_device)
        dyf = torch.where(keep, dyf, torch.zeros_like(dyf))
    s1, s2 = codec.bn_bwd_reduce(packed, scale, mn, dy, bits, gs, mask=mask)
    dims = [0, 2, 3]
    r1, r2 = (dyf * dec).sum(dims), dyf.sum(dims)
    assert torch.allclose(s1, r1, rtol=1e-4, atol=1e-3 * r1.abs().max().item())
    assert torch.allclose(s2, r2, rtol=1e-4, atol=1e-3 * r2.abs().max().item() + 1e-3)
    k1, k2, k3 = (torch.randn(C, generator=g).to(cuda_device) for _ in range(3))
    dx = codec.bn_bwd_dx(packed, scale, mn, dy, k1, k2, k3, bits, gs, mask=mask)
    assert dx.is_contiguous(memory_format=torch.channels_last)
    view = [1, C, 1, 1]
    want = k1.view(view) * dyf - k2.view(view) - k3.view(view) * dec
    tol = 2.0 ** -7 if dtype == torch.bfloat16 else 1e-5
    assert ((dx.float() - want).abs() <= tol * (1 + want.abs())).all()


@pytest.mark.gpu
def test_channels_last_modules_match_pytorch(cuda_device):
    """conv -> BN(+ReLU) -> ReLU on a channels-last input through the DO* modules: outputs stay
    channels-last, the forward equals PyTorch's to rounding, gradients agree within the 8-bit
    codec's error, and the saved conv input is rebuilt channels-last."""
    from deep_optimization_b200.layers import DOConv2d
    from deep_optimization_b200.modules.activations.act_layers import DOReLU_Variance
    from deep_optimization_b200.modules.module_utils import unified_dequantize, unified_quantize
    from deep_optimization_b200.modules.normalization.normalization_layers import DOBatchNorm2d
    torch.manual_seed(4)
    entry = {"bits": 8, "pack_only": False, "group_size": 256, "act_padding": False, "N": 8,
             "AVG_ALAM": False, "ALAM_BITS": 0, "DIVISION": None}
    meta = {"c": dict(entry), "b": dict(entry), "r": dict(entry, bits=1, pack_only=True)}
    x = torch.randn(8, 16, 16, 16, device=cuda_device).contiguous(memory_format=torch.channels_last)
    q, q_meta, _ = unified_quantize(x, None, "c", meta, clamp=False, clamp_alpha=0.0)
    back = unified_dequantize(q, q_meta, None)
    assert back.shape == x.shape and back.is_contiguous(memory_format=torch.channels_last)
    assert (back.float() - x).abs().max() < 0.05
    bn = DOBatchNorm2d(16, target_name="b", meta=meta).to(cuda_device).train()
    rb = torch.nn.BatchNorm2d(16).to(cuda_device).train()
    relu = DOReLU_Variance(target_name="r", meta=meta).train()
    conv = DOConv2d(16, 16, 3, padding=1, target_name="c", meta=meta).to(cuda_device).train()
    rc = torch.nn.Conv2d(16, 16, 3, padding=1, bias=False).to(cuda_device)
    conv = conv.to(memory_format=torch.channels_last)
    rc = rc.to(memory_format=torch.channels_last)
    with torch.no_grad():
        rc.weight.copy_(conv.weight)
    xr = x.detach().clone().requires_grad_()
    xq = x.detach().clone().requires_grad_()
    y = relu(bn(conv(xq)))
    yr = torch.relu(rb(rc(xr)))
    assert y.is_contiguous(memory_format=torch.channels_last)
    assert torch.allclose(y, yr, atol=2e-3)
    gy = torch.randn_like(y)
    y.backward(gy); yr.backward(gy)
    assert xq.grad.is_contiguous(memory_format=torch.channels_last)
    assert (xq.grad - xr.grad).abs().max() < 0.05
    assert torch.allclose(bn.bias.grad, rb.bias.grad, rtol=1e-4, atol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16), ids=("f32", "bf16"))
@pytest.mark.parametrize("shape", [(8, 16, 32, 32), (6, 24, 14, 14), (4, 64, 56, 56)])
@pytest.mark.parametrize("channels_last", (False, True))
def test_bn_add_relu_fused_forward(cuda_device, dtype, shape, channels_last):
    """y = max(x_hat * w + b + residual, 0): the packed x_hat is the one of the kernel without
    the add (bit-exact), y equals the fp32 chain rounded once to the output type, the mask is
    that of the sum, in both layouts."""
    from deep_optimization_b200 import codec
    fmt = torch.channels_last if channels_last else torch.contiguous_format
    g = torch.Generator().manual_seed(41)
    x = (torch.randn(shape, generator=g) * 2 + 0.5).to(dtype).to(cuda_device).contiguous(memory_format=fmt)
    r = torch.randn(shape, generator=g).to(dtype).to(cuda_device).contiguous(memory_format=fmt)
    C = shape[1]
    mean = torch.randn(C, generator=g).to(cuda_device)
    invstd = (torch.rand(C, generator=g) + 0.5).to(cuda_device)
    w = torch.randn(C, generator=g).to(cuda_device)
    b = torch.randn(C, generator=g).to(cuda_device)
    gs = _cl_group(x.numel())
    y0, p0, s0, m0 = codec.bn_fwd_norm_quant_pack(x, mean, invstd, w, b, 2, gs, seed=3, offset=2)
    y1, p1, s1, m1, mask = codec.bn_fwd_norm_quant_pack(x, mean, invstd, w, b, 2, gs, seed=3, offset=2,
                                                        relu=True, residual=r)
    assert torch.equal(p0, p1) and torch.equal(s0, s1) and torch.equal(m0, m1)
    view = [1, C, 1, 1]
    x_hat = (x.float() - mean.view(view)) * invstd.view(view)
    total = (x_hat * w.view(view) + b.view(view)) + r.float()
    keep = total > 0
    assert torch.equal(y1, torch.where(keep, total, torch.zeros_like(total)).to(dtype))
    assert y1.is_contiguous(memory_format=fmt)
    order = keep.permute(0, 2, 3, 1) if channels_last else keep
    bits = np.unpackbits(mask.cpu().numpy(), bitorder="little")[: x.numel()]
    assert np.array_equal(bits.astype(bool), order.reshape(-1).cpu().numpy())


@pytest.mark.gpu
@pytest.mark.parametrize("channels_last", (False, True))
def test_bn_add_relu_module_matches_pytorch(cuda_device, channels_last):
    """DOBatchNorm2d(x, residual) with fuse_relu against relu(BatchNorm2d(x) + residual): output
    exact to rounding, gradients of x, the residual and the affine parameters within the 8-bit
    codec's error."""
    from deep_optimization_b200.modules.normalization.normalization_layers import DOBatchNorm2d
    torch.manual_seed(3)
    fmt = torch.channels_last if channels_last else torch.contiguous_format
    meta = {"b": {"bits": 8, "pack_only": False, "group_size": 256, "act_padding": False, "N": 8,
                  "AVG_ALAM": False, "ALAM_BITS": 0, "DIVISION": None}}
    bn = DOBatchNorm2d(16, target_name="b", meta=meta).to(cuda_device).train()
    bn.fuse_relu = True
    rb = torch.nn.BatchNorm2d(16).to(cuda_device).train()
    with torch.no_grad():
        bn.weight.copy_(torch.randn(16)); bn.bias.copy_(torch.randn(16))
        rb.weight.copy_(bn.weight); rb.bias.copy_(bn.bias)
    x = torch.randn(8, 16, 16, 16, device=cuda_device).contiguous(memory_format=fmt).requires_grad_()
    s = torch.randn(8, 16, 16, 16, device=cuda_device).contiguous(memory_format=fmt).requires_grad_()
    xr, sr = x.detach().clone().requires_grad_(), s.detach().clone().requires_grad_()
    g = torch.randn_like(x)
    y, yr = bn(x, s), torch.relu(rb(xr) + sr)
    assert torch.allclose(y, yr, atol=1e-4)
    y.backward(g); yr.backward(g)
    assert torch.equal(s.grad, sr.grad)
    assert (x.grad - xr.grad).abs().max() < 0.05
    assert (bn.weight.grad - rb.weight.grad).norm() / rb.weight.grad.norm() < 0.03
    assert torch.allclose(bn.bias.grad, rb.bias.grad, rtol=1e-4, atol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16), ids=("f32", "bf16"))
@pytest.mark.parametrize("geom", [(3, 2, 1), (2, 2, 0), (3, 1, 1), (4, 2, 2), (3, 2, 0)])
@pytest.mark.parametrize("shape", [(4, 64, 112, 112), (3, 8, 7, 9), (2, 16, 4, 4)])
def test_maxpool_channels_last(cuda_device, dtype, geom, shape):
    """Forward equals F.max_pool2d exactly (ties and repeated values included); backward equals
    PyTorch's on fp32 exactly and on bf16 to one rounding of the sum; the saved state is 4 bits
    per output."""
    from deep_optimization_b200 import codec
    k, s, p = geom
    g = torch.Generator().manual_seed(51)
    # few distinct values: many ties inside a window
    x = torch.randint(-3, 4, shape, generator=g).to(dtype).to(cuda_device).contiguous(memory_format=torch.channels_last)
    assert codec.maxpool_supported(x, k, s, p)
    y, idx = codec.maxpool_fwd(x, k, s, p)
    xr = x.detach().clone().requires_grad_()
    yr = torch.nn.functional.max_pool2d(xr, k, s, p)
    assert torch.equal(y, yr) and y.is_contiguous(memory_format=torch.channels_last)
    assert idx.numel() * 32 == y.numel() * 4
    dy = torch.randn(yr.shape, generator=g).to(dtype).to(cuda_device).contiguous(memory_format=torch.channels_last)
    yr.backward(dy)
    dx = codec.maxpool_bwd(idx, dy, x.shape, k, s, p)
    if dtype == torch.float32:
        assert torch.allclose(dx, xr.grad, rtol=1e-6, atol=1e-6)
    else:
        assert ((dx.float() - xr.grad.float()).abs() <= 2.0 ** -6 * (1 + xr.grad.float().abs())).all()


@pytest.mark.gpu
def test_maxpool_module_and_nan(cuda_device):
    """DOMaxPool2d: channels-last training input takes the 4-bit path, an NCHW input or eval mode
    the stock operator; a NaN in a window is that window's maximum."""
    from deep_optimization_b200.modules.activations.act_layers import DOMaxPool2d
    pool = DOMaxPool2d(3, 2, 1).train()
    x = torch.randn(2, 16, 12, 12, device=cuda_device)
    x[0, 3, 5, 5] = float("nan")
    xc = x.contiguous(memory_format=torch.channels_last).requires_grad_()
    xn = x.clone().requires_grad_()
    yc, yn = pool(xc), pool(xn)
    assert type(yc.grad_fn).__name__ == "_DOMaxPool2dBackward" and type(yn.grad_fn).__name__ != "_DOMaxPool2dBackward"
    assert torch.equal(torch.nan_to_num(yc, nan=7.0), torch.nan_to_num(yn, nan=7.0)) and torch.isnan(yc).sum() == 4
    g = torch.randn_like(yn)
    yc.backward(g); yn.backward(g)
    assert torch.allclose(xc.grad, xn.grad, rtol=1e-6, atol=1e-6)
    assert pool.eval()(xc).grad_fn is None or type(pool(xc).grad_fn).__name__ != "_DOMaxPool2dBackward"


@pytest.mark.gpu
@pytest.mark.parametrize("channels_last", (False, True))
@pytest.mark.parametrize("mode", ("plain", "relu", "residual"))
def test_bn_backward_one_call(cuda_device, channels_last, mode):
    """act_bn_backward (sums zeroed inside, reduction, constants, dx, and for a residual block
    dy under the mask as a by-product of the reduction) against the separate entry points."""
    from deep_optimization_b200 import codec
    fmt = torch.channels_last if channels_last else torch.contiguous_format
    g = torch.Generator().manual_seed(61)
    shape, gs, bits = (6, 32, 14, 14), 64, 2
    x = torch.randn(shape, generator=g).to(torch.bfloat16).to(cuda_device).contiguous(memory_format=fmt)
    dy = torch.randn(shape, generator=g).to(torch.bfloat16).to(cuda_device).contiguous(memory_format=fmt)
    C = shape[1]
    w = torch.randn(C, generator=g).to(cuda_device)
    b = torch.randn(C, generator=g).to(cuda_device)
    y, packed, scale, mn, params, mask = codec.bn_forward(x, 1e-5, w, b, None, None, 0.0, bits, gs,
                                                          relu=(mode != "plain"), seed=5, offset=1)
    count = x.numel() // C
    dx, dg, db, dym = codec.bn_backward(packed, scale, mn, dy, mask, mode == "residual", bits, gs, params, count)
    if mode == "residual":
        want_dym = codec.relu_bwd_unpack(mask, dy, channels_last=channels_last)
        assert torch.equal(dym, want_dym)
        s1, s2 = codec.bn_bwd_reduce(packed, scale, mn, want_dym, bits, gs)
        coef = codec.bn_bwd_coef((s1, s2), params, count)
        want_dx = codec.bn_bwd_dx(packed, scale, mn, want_dym, None, None, None, bits, gs, coef=coef)
    else:
        assert dym is None
        s1, s2 = codec.bn_bwd_reduce(packed, scale, mn, dy, bits, gs, mask=mask)
        coef = codec.bn_bwd_coef((s1, s2), params, count)
        want_dx = codec.bn_bwd_dx(packed, scale, mn, dy, None, None, None, bits, gs, mask=mask, coef=coef)
    assert torch.allclose(dg, s1, rtol=1e-4, atol=1e-3) and torch.allclose(db, s2, rtol=1e-4, atol=1e-3)
    assert ((dx.float() - want_dx.float()).abs() <= 2.0 ** -6 * (1 + want_dx.float().abs())).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(50432, 768), (1000, 3072), (197, 8), (3, 2056), (1, 64)])
def test_column_reductions(cuda_device, dtype, shape):
    """act_col_sum and act_ln_bwd_params against float64 sums of the same (rounded) inputs."""
    from deep_optimization_b200 import codec
    torch.manual_seed(shape[0] + shape[1])
    R, C = shape
    dy = torch.randn(R, C, device=cuda_device).to(dtype)
    x = (torch.randn(R, C, device=cuda_device) * 2 + 0.5).to(dtype)
    s = codec.col_sum(dy)
    ref = dy.double().sum(0)
    tol = dy.double().abs().sum(0) * 2e-6 + 1e-6
    assert s.dtype == torch.float32 and ((s.double() - ref).abs() <= tol).all()
    y, mean, rstd = torch.ops.aten.native_layer_norm(x, [C], None, None, 1e-5)
    dg, db = codec.ln_bwd_params(dy, x, mean, rstd)
    xh = (x.double() - mean.double().view(-1, 1)) * rstd.double().view(-1, 1)
    ref_g = (dy.double() * xh).sum(0)
    tol_g = (dy.double() * xh).abs().sum(0) * 4e-6 + 1e-5
    assert ((dg.double() - ref_g).abs() <= tol_g).all() and ((db.double() - ref).abs() <= tol).all()
    # and what ATen computes for the same call
    if dtype != torch.float16:
        _, tg, tb = torch.ops.aten.native_layer_norm_backward(dy, x, [C], mean, rstd, torch.ones(C, device=cuda_device, dtype=dtype),
                                                              torch.zeros(C, device=cuda_device, dtype=dtype), [False, True, True])
        assert ((dg.double() - tg.double()).abs() <= tol_g + tg.double().abs() * 2.0 ** -7).all()


def test_column_reductions_reject_bad_layouts(cuda_device):
    from deep_optimization_b200 import codec
    with pytest.raises(ValueError):
        codec.col_sum(torch.randn(16, 12, device=cuda_device))          # 12 columns: not a multiple of 8
    with pytest.raises(ValueError):
        codec.col_sum(torch.randn(16, 32, device=cuda_device)[:, ::2])  # rows not contiguous
    assert codec.col_sum(torch.empty(0, 16, device=cuda_device)).abs().sum() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("shape,gs", [((64, 197, 768), 128), ((3, 5, 256), 256), ((7, 960), 64), ((2, 9, 32), 32),
                                      ((5, 1024), 128)])
def test_layer_norm_fused_with_codec(cuda_device, dtype, bits, shape, gs):
    """act_ln_fwd_quant_pack: the packed input equals act_quant_pack's bit for bit (same seed and
    offset, stochastic and round-to-nearest), y and the statistics equal ATen's within rounding;
    act_ln_bwd_from_packed equals ATen's backward on the dequantised input within rounding."""
    from deep_optimization_b200 import _lib, codec
    torch.manual_seed(bits * 1000 + shape[-1])
    C = shape[-1]
    x = (torch.randn(shape, device=cuda_device) * 1.5 + 0.3).to(dtype)
    w = (torch.rand(C, device=cuda_device) + 0.5)
    b = torch.randn(C, device=cuda_device) * 0.1
    for flags in (0, _lib.ACT_FLAG_ROUND_NEAREST):
        y, mean, rstd, packed, scale, mn = codec.ln_fwd_quant_pack(x, w, b, 1e-6, bits, gs, seed=77, offset=5, flags=flags)
        p2, s2, m2 = codec.quant_pack(x, bits, gs, seed=77, offset=5, flags=flags)
        assert torch.equal(packed, p2) and torch.equal(scale, s2) and torch.equal(mn, m2)
    yr, mr, rr = torch.ops.aten.native_layer_norm(x.float(), [C], w, b, 1e-6)
    assert torch.allclose(mean, mr.reshape(-1), atol=1e-5, rtol=1e-5) and torch.allclose(rstd, rr.reshape(-1), rtol=1e-4)
    tol = {torch.float32: 1e-5, torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}[dtype]
    assert ((y.float() - yr).abs() <= tol * (yr.abs() + 1)).all()
    # backward
    dy = torch.randn(shape, device=cuda_device).to(dtype)
    dx, dg, db = codec.ln_bwd_from_packed(dy, packed, scale, mn, bits, gs, mean, rstd, w)
    xq = codec.dequant_unpack(packed, scale, mn, bits, gs, out_dtype=torch.bfloat16).reshape(shape)
    dxr, dgr, dbr = torch.ops.aten.native_layer_norm_backward(dy.double(), xq.double(), [C], mean.double().view(*shape[:-1], 1),
                                                              rstd.double().view(*shape[:-1], 1), w.double(), b.double(),
                                                              [True, True, True])
    assert ((dx.double() - dxr).abs() <= tol * (dxr.abs() + dxr.abs().max())).all()
    rows = x.numel() // C
    assert ((dg.double() - dgr).abs() <= 1e-5 * rows ** 0.5 * (dgr.abs() + 1) + 1e-4).all()
    assert ((db.double() - dbr).abs() <= 1e-5 * rows ** 0.5 * (dbr.abs() + 1) + 1e-4).all()


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16), ids=("bf16", "f16"))
@pytest.mark.parametrize("bits", (1, 2, 4, 8))
@pytest.mark.parametrize("shape,gs", [((64, 197, 768), 128), ((37, 960), 64), ((5, 7, 256), 256), ((300, 64), 32),
                                      ((129, 1024), 128)])
def test_layer_norm_with_residual_addition(cuda_device, dtype, bits, shape, gs):
    """act_ln_add_fwd_quant_pack: the sum it writes equals the separate addition bit for bit, and
    y, the statistics and the packed sum equal act_ln_fwd_quant_pack's on that sum bit for bit;
    act_ln_bwd_from_packed_sum equals act_ln_bwd_from_packed's dx plus the second gradient to
    within one rounding of the element type, with the parameter gradients unchanged."""
    from deep_optimization_b200 import _lib, codec
    torch.manual_seed(bits * 100 + shape[-1])
    C = shape[-1]
    a = (torch.randn(shape, device=cuda_device) * 1.5 + 0.3).to(dtype)
    r = (torch.randn(shape, device=cuda_device) * 0.7).to(dtype)
    w = (torch.rand(C, device=cuda_device) + 0.5)
    b = torch.randn(C, device=cuda_device) * 0.1
    for flags in (0, _lib.ACT_FLAG_ROUND_NEAREST):
        got = codec.ln_fwd_quant_pack(a, w, b, 1e-6, bits, gs, seed=9, offset=3, flags=flags, residual=r)
        total = a + r
        assert torch.equal(got[0], total)
        want = codec.ln_fwd_quant_pack(total, w, b, 1e-6, bits, gs, seed=9, offset=3, flags=flags)
        for g, t in zip(got[1:], want):
            assert torch.equal(g.view(torch.uint8), t.view(torch.uint8))
    _, y, mean, rstd, packed, scale, mn = got
    dy = torch.randn(shape, device=cuda_device).to(dtype)
    dy2 = torch.randn(shape, device=cuda_device).to(dtype)
    dx, dg, db = codec.ln_bwd_from_packed(dy, packed, scale, mn, bits, gs, mean, rstd, w)
    dx2, dg2, db2 = codec.ln_bwd_from_packed(dy, packed, scale, mn, bits, gs, mean, rstd, w, dy2=dy2)
    ulp = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}[dtype]
    want = dx.double() + dy2.double()                    # dx carries one rounding of its own
    assert ((dx2.double() - want).abs() <= ulp * (want.abs() + dx.double().abs()) + 1e-6).all()
    assert torch.allclose(dg2, dg, rtol=1e-4, atol=1e-3) and torch.allclose(db2, db, rtol=1e-4, atol=1e-3)
    with pytest.raises(ValueError):
        codec.ln_fwd_quant_pack(a, w, b, 1e-6, bits, gs, residual=r.float())
    with pytest.raises(ValueError):
        codec.ln_bwd_from_packed(dy, packed, scale, mn, bits, gs, mean, rstd, w, dy2=dy2[..., : C // 2])


def test_layer_norm_fused_irregular_groups(cuda_device):
    """Groups with a zero, a denormal, a huge or a non-finite range take the general encoder; the
    packed bytes still equal act_quant_pack's."""
    from deep_optimization_b200 import codec
    x = torch.randn(16, 768, device=cuda_device)
    x[0, :128] = 3.0
    x[1, 128:256] *= 1e-42
    x[2, 0] = 3e38; x[2, 1] = -3e38
    x[3, 300] = float("inf")
    x[4, 500] = float("nan")
    for dtype in (torch.float32, torch.bfloat16):
        xd = x.to(dtype)
        _, _, _, packed, scale, mn = codec.ln_fwd_quant_pack(xd, None, None, 1e-5, 2, 128, seed=1, offset=2)
        p2, s2, m2 = codec.quant_pack(xd, 2, 128, seed=1, offset=2)
        assert torch.equal(packed, p2)
        assert torch.equal(scale.view(torch.int32), s2.view(torch.int32)) and torch.equal(mn.view(torch.int32), m2.view(torch.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16), ids=("bf16", "f16"))
def test_maxpool_packed_pairs_nan_and_infinities(cuda_device, dtype):
    """The 16-bit forward kernel compares packed pairs: NaN, -inf and +inf inside windows and ties
    give what F.max_pool2d gives, values and gradient routing.  (A window that holds nothing but
    -inf is left out: there PyTorch's channels-last kernel sends the gradient to position 0 of the
    plane and its NCHW kernel to the window's first position, which is what this one does.)"""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(77)
    x = torch.randint(-2, 3, (3, 16, 13, 11), generator=g).to(dtype)
    x[0, 1, 4, 4] = float("nan"); x[0, 1, 4, 5] = float("nan")          # two NaN in one window
    x[1, 2, 6, 6] = float("inf"); x[1, 3, 2, 2] = float("-inf")
    x[2, 6, 0, 0] = float("nan")                                         # NaN at the border
    x = x.to(cuda_device).contiguous(memory_format=torch.channels_last)
    for k, s, p in ((3, 2, 1), (2, 2, 0), (3, 1, 1)):
        y, idx = codec.maxpool_fwd(x, k, s, p)
        xr = x.detach().clone().requires_grad_()
        yr = torch.nn.functional.max_pool2d(xr, k, s, p)
        assert torch.equal(torch.isnan(y), torch.isnan(yr))
        assert torch.equal(torch.nan_to_num(y.float(), nan=9.0), torch.nan_to_num(yr.float(), nan=9.0))
        dy = torch.randint(-4, 5, yr.shape, generator=g).to(dtype).to(cuda_device).contiguous(memory_format=torch.channels_last)
        yr.backward(dy)
        dx = codec.maxpool_bwd(idx, dy, x.shape, k, s, p)
        assert torch.equal(dx.float(), xr.grad.float())                  # small integers: sums are exact
