"""GPU tests of the drop-in layers: forward equals the stock module, gradients equal
those computed from the dequantised activation, and stay close to the exact ones."""
import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


def _meta(target, bits, gs, N, pack_only=False, pad=False):
    return {target: {"bits": bits, "pack_only": pack_only, "group_size": gs, "act_padding": pad, "N": N,
                     "AVG_ALAM": False, "ALAM_BITS": 0, "DIVISION": None}}


def test_module_utils_round_trip(cuda_device):
    from deep_optimization_b200.modules.module_utils import unified_dequantize, unified_quantize
    x = torch.relu(torch.randn(8, 16, 32, 32, device=cuda_device)).to(torch.bfloat16)
    for gs, pad in ((256, False), (128, False), (256, True)):
        meta = _meta("t", 4, gs, 8, pad=pad)
        (p, s, m), q_meta, _ = unified_quantize(x, None, "t", meta, True, 3.0)
        assert len(q_meta) == 14 and q_meta[0] == 4 and tuple(q_meta[-1]) == tuple(x.shape)
        y = unified_dequantize((p, s, m), q_meta, None)
        assert y.shape == x.shape and y.dtype == torch.bfloat16
        assert (y.float() - x.float()).abs().max() <= s.max() * 1.01 + 0.02
    mask = (x > 0).to(torch.int8)
    (p, s, m), q_meta, _ = unified_quantize(mask, None, "t", _meta("t", 1, 256, 8, pack_only=True), False, 0.0)
    assert s is None and torch.equal(unified_dequantize((p, None, None), q_meta, None), mask)


def test_conv2d_layer(cuda_device):
    from deep_optimization_b200.layers import DOConv2d
    torch.manual_seed(0)
    meta = _meta("c", 8, 256, 4)
    conv = DOConv2d(16, 32, 3, padding=1, target_name="c", meta=meta).to(cuda_device).train()
    ref = nn.Conv2d(16, 32, 3, padding=1, bias=False).to(cuda_device)
    ref.weight.data.copy_(conv.weight.data)
    x = torch.relu(torch.randn(4, 16, 32, 32, device=cuda_device)).requires_grad_()
    xr = x.detach().clone().requires_grad_()
    y = conv(x); yr = ref(xr)
    assert torch.allclose(y, yr, atol=1e-5)
    g = torch.randn_like(y)
    y.backward(g); yr.backward(g)
    assert torch.allclose(x.grad.float(), xr.grad, atol=1e-3, rtol=1e-2)       # dx does not use the saved input
    rel = (conv.weight.grad - ref.weight.grad).norm() / ref.weight.grad.norm()
    assert rel < 0.02                                                            # 8-bit codes: ~1/255 of the range
    conv.eval()
    assert torch.allclose(conv(x), ref(x), atol=1e-5)


def test_linear_bn_relu_gelu_layers(cuda_device):
    from deep_optimization_b200.layers import DOLinear
    from deep_optimization_b200.modules.activations.act_layers import DOGELU, DOReLU_Variance, DOSiLU
    from deep_optimization_b200.modules.normalization.normalization_layers import DOBatchNorm2d
    torch.manual_seed(1)
    # linear
    meta = _meta("l", 8, 256, 8)
    lin = DOLinear(256, 64, target_name="l", meta=meta).to(cuda_device).train()
    ref = nn.Linear(256, 64).to(cuda_device); ref.load_state_dict(lin.state_dict())
    x = torch.randn(8, 50, 256, device=cuda_device, requires_grad=True); xr = x.detach().clone().requires_grad_()
    y, yr = lin(x), ref(xr)
    assert torch.allclose(y, yr, atol=1e-4)
    y.sum().backward(); yr.sum().backward()
    assert torch.allclose(x.grad, xr.grad, atol=1e-3)
    assert (lin.weight.grad - ref.weight.grad).norm() / ref.weight.grad.norm() < 0.02
    # relu: 1-bit mask is lossless
    relu = DOReLU_Variance(target_name="r", meta=_meta("r", 1, 256, 8, pack_only=True)).to(cuda_device).train()
    x = torch.randn(8, 4, 16, 16, device=cuda_device, requires_grad=True); xr = x.detach().clone().requires_grad_()
    g = torch.randn_like(x)
    relu(x).backward(g); torch.relu(xr).backward(g)
    assert torch.equal(x.grad, xr.grad)
    # gelu / silu: derivative is quantised to 8 bits
    for mod, fn in ((DOGELU(target_name="g", meta=_meta("g", 8, 256, 8)), lambda t: nn.functional.gelu(t, approximate="tanh")),
                    (DOSiLU(target_name="g", meta=_meta("g", 8, 256, 8)), nn.functional.silu)):
        mod = mod.to(cuda_device).train()
        x = torch.randn(8, 4, 16, 16, device=cuda_device, requires_grad=True); xr = x.detach().clone().requires_grad_()
        y, yr = mod(x), fn(xr)
        assert torch.allclose(y, yr, atol=1e-5)
        y.backward(g); yr.backward(g)
        assert (x.grad - xr.grad).abs().max() < 0.02 * g.abs().max()
    # batch norm
    bn = DOBatchNorm2d(4, target_name="b", meta=_meta("b", 8, 256, 8)).to(cuda_device).train()
    rb = nn.BatchNorm2d(4).to(cuda_device).train()
    x = torch.randn(8, 4, 16, 16, device=cuda_device, requires_grad=True); xr = x.detach().clone().requires_grad_()
    y, yr = bn(x), rb(xr)
    assert torch.allclose(y, yr, atol=1e-4)
    assert torch.allclose(bn.running_var, rb.running_var, atol=1e-5)
    y.backward(g); yr.backward(g)
    assert (x.grad - xr.grad).abs().max() < 0.05
    # x_hat is kept as bf16 + 8-bit stochastic codes: compare the gradient vectors as a whole
    assert (bn.weight.grad - rb.weight.grad).norm() / rb.weight.grad.norm() < 0.03


def test_controller_end_to_end_step(cuda_device):
    from deep_optimization_b200.controller import Controller
    torch.manual_seed(0)
    model = nn.Sequential(nn.Conv2d(3, 32, 3, padding=1, bias=False), nn.BatchNorm2d(32), nn.ReLU(),
                          nn.Conv2d(32, 32, 3, padding=1, bias=False), nn.AdaptiveAvgPool2d(1), nn.Flatten(),
                          nn.Linear(32, 10))
    cfg = dict(default_bits=2, auto_precision=None, batch_size=32, min_activation_mib=0.5)
    c = Controller(model, cfg, input_shape=(3, 32, 32), test=False)
    net = c.traced_model
    opt = torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9)
    x = torch.randn(32, 3, 32, 32, device=cuda_device); y = torch.randint(0, 10, (32,), device=cuda_device)
    losses = []
    for _ in range(30):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = nn.functional.cross_entropy(net(x), y)
        opt.zero_grad(); loss.backward(); opt.step()
        losses.append(loss.item())
    assert all(l == l for l in losses) and min(losses[-3:]) < losses[0] - 0.05   # 2-bit activations still train


def test_cpp_extension_mirror(cuda_device):
    from deep_optimization_b200 import cpp_extension as cx
    x = torch.relu(torch.randn(4, 6, 256, device=cuda_device)).to(torch.bfloat16)
    for bits, pack, unpack in ((2, cx.pack2, cx.unpack2), (3, cx.pack3, cx.unpack3), (8, cx.pack8, cx.unpack8)):
        out = torch.zeros(4 * 6 * 8 * bits, dtype=torch.int32, device=cuda_device)
        scaler = torch.empty(4, 6, dtype=torch.bfloat16, device=cuda_device)
        mn = torch.empty(24, dtype=torch.bfloat16, device=cuda_device)
        pack(x, out, scaler, mn, 0.9)
        y = torch.empty(4, 6, 256, dtype=torch.bfloat16, device=cuda_device)
        unpack(out, y, scaler, mn, 4, 6, 4)
        step = scaler.float().view(4, 6, 1)
        assert ((y.float() - x.float()).abs() <= step * 1.05 + 0.02).all()
    lo, hi = cx.min_max_kernel(x)
    assert torch.equal(lo, x.float().amin(-1)) and torch.equal(hi, x.float().amax(-1))
