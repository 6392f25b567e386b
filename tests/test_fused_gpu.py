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
