"""CPU tests of the host-side mirror of the reference interface: grouping helpers,
operator registration (fake kernels), controller planning, bit-allocation policy."""
import pytest
import copy

import torch
from torch import nn


def test_reshape_round_trips():
    from deep_optimization_b200.modules.tensor_act_reshape_utils import (
        spatical_aware_act_tensor_reshape as fwd, spatical_aware_act_tensor_reshape_back as back)
    cases = [((4, 6, 32, 48), 256, False), ((4, 6, 32, 48), 64, False), ((4, 6, 32, 48), 128, False),
             ((4, 6, 30, 30), 256, True), ((3, 197, 7), 256, True), ((5, 1000), 256, True),
             ((2, 8, 16, 48), 256, False)]           # H != W with spatial tiles
    for shape, gs, pad in cases:
        x = torch.randn(shape)
        g, N, G, nh, nw, shp, pe, re_, cm = fwd(x, gs, pad, False)
        assert g.shape == (N, G, gs) and g.is_contiguous()
        y = back(g, shp, gs, nh, nw, pad, pe, re_, cm)
        assert torch.equal(x, y), (shape, gs, pad)


def test_spatial_tiles_are_tiles():
    from deep_optimization_b200.modules.tensor_act_reshape_utils import spatical_aware_act_tensor_reshape
    x = torch.arange(2 * 3 * 32 * 32, dtype=torch.float32).view(2, 3, 32, 32)
    g, *_ = spatical_aware_act_tensor_reshape(x, 256, False, False)
    assert torch.equal(g[0, 0].view(16, 16), x[0, 0, :16, :16])
    assert torch.equal(g[0, 1].view(16, 16), x[0, 0, :16, 16:32])


def test_ops_are_registered_with_real_schemas():
    import deep_optimization_b200.act_kernels  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(4, 8, 128, dtype=torch.bfloat16, device="cuda")
        p, s, m = torch.ops.act_lib.quant_pack_triton(x, 2, 128, False, 0, True, 3.0)
        assert p.shape == (32, 8) and p.dtype == torch.int32 and s.shape == (4, 8) and m.dtype == torch.float32
        y = torch.ops.act_lib.dequant_unpack_triton(p, s, m, 2, 128, False, 0)
        assert y.shape == (4, 8, 128) and y.dtype == torch.bfloat16
        mask = torch.empty(4, 8, 128, dtype=torch.int8, device="cuda")
        pk = torch.ops.act_lib.pack_triton(mask, 1, 128)
        assert pk.shape == (32, 4)
        assert torch.ops.act_lib.unpack_triton(pk, 1, 4, 8, 128).shape == (4, 8, 128)
        with pytest.raises(ValueError):
            torch.ops.act_lib.quant_pack_triton(x, 3, 128, False, 0, True, 3.0)


def test_find_group_size():
    from deep_optimization_b200.controller import find_group_size
    assert find_group_size(64 * 56 * 56, 2) == (512, False)
    assert find_group_size(197 * 768, 2) == (256, False)
    assert find_group_size(1000, 2) == (256, True)
    assert find_group_size(1024 * 3, 2, special=True) == (1024, False)


def test_controller_plans_and_swaps():
    from deep_optimization_b200.controller import Controller
    from deep_optimization_b200.layers import DOConv2d, DOLinear
    from deep_optimization_b200.modules.activations.act_layers import DOReLU_Variance
    from deep_optimization_b200.modules.normalization.normalization_layers import DOBatchNorm2d
    model = nn.Sequential(nn.Conv2d(3, 64, 3, padding=1, bias=False), nn.BatchNorm2d(64), nn.ReLU(),
                          nn.Conv2d(64, 64, 3, padding=1, bias=False), nn.Flatten(), nn.Linear(64 * 32 * 32, 10))
    cfg = dict(default_bits=2, auto_precision=None, batch_size=64, min_activation_mib=1)
    w0 = model[0].weight.detach().clone()
    c = Controller(model, dict(cfg, fuse_bn_relu=False), input_shape=(3, 32, 32), test=False, device="cpu")
    net = c.traced_model
    t = [net.get_submodule(str(i)) for i in range(6)]
    assert isinstance(t[0], DOConv2d) and isinstance(t[1], DOBatchNorm2d)
    assert not t[1].fuse_relu and c.fused_bn_relu == []
    assert isinstance(t[2], DOReLU_Variance) and isinstance(t[3], DOConv2d)
    assert isinstance(t[5], nn.Linear) and not isinstance(t[5], DOLinear)      # output too small
    assert torch.equal(t[0].weight, w0)
    m = c.meta["3"]
    assert (m["bits"], m["group_size"], m["act_padding"], m["N"], m["pack_only"]) == (2, 512, False, 64, False)
    assert c.meta["2"]["pack_only"] and c.meta["2"]["bits"] == 1
    assert set(("AVG_ALAM", "ALAM_BITS", "DIVISION", "NG")) <= set(m)
    # eval mode is the stock module path and runs on CPU
    net.eval()
    with torch.no_grad():
        assert net(torch.randn(2, 3, 32, 32)).shape == (2, 10)


def test_controller_fuses_bn_add_relu():
    """relu(bn(x) + skip), the end of a residual block, becomes one BatchNorm call taking the
    skip as its second argument, also when the skip is computed after the BatchNorm; the
    eval-mode output is unchanged."""
    from deep_optimization_b200.controller import Controller
    from deep_optimization_b200.payload.resnet import Bottleneck

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.stem = nn.Conv2d(3, 64, 3, padding=1, bias=False)
            self.a = Bottleneck(64, 16, project=False)
            self.b = Bottleneck(64, 32, project=True)

        def forward(self, x):
            return self.b(self.a(self.stem(x)))

    torch.manual_seed(0)
    model = Net()
    ref = copy.deepcopy(model).eval()
    cfg = dict(default_bits=2, auto_precision=None, batch_size=64, min_activation_mib=0.1)
    c = Controller(model, cfg, input_shape=(3, 32, 32), test=False, device="cpu")
    net = c.traced_model
    assert sorted(c.fused_bn_add_relu) == ["a.bn3", "b.bn3"]
    targets = [n.target for n in net.graph.nodes if n.op == "call_module"]
    assert "a.relu3" not in targets and "b.relu3" not in targets
    assert net.a.bn3.fuse_relu and net.b.bn3.fuse_relu and not net.get_submodule("b.shortcut.1").fuse_relu
    for n in net.graph.nodes:
        if n.op == "call_module" and n.target in ("a.bn3", "b.bn3"):
            assert len(n.args) == 2
    net.eval()
    x = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        assert torch.allclose(net(x), ref(x), atol=1e-6)
    off = Controller(copy.deepcopy(ref).train(), dict(cfg, fuse_bn_add_relu=False), input_shape=(3, 32, 32),
                     test=False, device="cpu")
    assert off.fused_bn_add_relu == []


def test_controller_fuses_add_layer_norm():
    """s = a + b; y = norm(s) in a pre-norm transformer block becomes one LayerNorm call on (a, b)
    returning (y, s); an addition with a broadcast operand is rewritten too and added by the
    module the ordinary way; the eval-mode output is unchanged."""
    from deep_optimization_b200.controller import Controller
    from deep_optimization_b200.payload.vit import VisionTransformer

    torch.manual_seed(0)
    model = VisionTransformer(image=32, patch=8, dim=64, depth=2, heads=2, mlp_dim=128, num_classes=10)
    ref = copy.deepcopy(model).eval()
    cfg = dict(default_bits=2, auto_precision=None, batch_size=8, min_activation_mib=0.0)
    c = Controller(model, cfg, input_shape=(3, 32, 32), test=False, device="cpu")
    net = c.traced_model
    # every LayerNorm follows an addition: the position embedding (broadcast), the blocks' two
    assert sorted(c.fused_add_layer_norm) == ["blocks.0.norm1", "blocks.0.norm2", "blocks.1.norm1", "blocks.1.norm2", "norm"]
    for n in net.graph.nodes:
        if n.op == "call_module" and n.target in c.fused_add_layer_norm:
            assert len(n.args) == 2
    net.eval()
    x = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        assert torch.allclose(net(x), ref(x), atol=1e-5)
    off = Controller(copy.deepcopy(ref).train(), dict(cfg, fuse_add_layer_norm=False), input_shape=(3, 32, 32),
                     test=False, device="cpu")
    assert off.fused_add_layer_norm == []


def test_add_layer_norm_rewrite_keeps_order_and_skips_scaled_additions():
    """The LayerNorm call moves to the addition's place, so a consumer of the sum that the trace
    lists before the LayerNorm still finds it; torch.add is rewritten like `+`; an addition with
    `alpha` is left alone."""
    from deep_optimization_b200.controller import Controller

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.inp = nn.Linear(64, 64)
            self.n1, self.n2, self.n3 = nn.LayerNorm(64), nn.LayerNorm(64), nn.LayerNorm(64)
            self.f1, self.f2, self.f3 = nn.Linear(64, 64), nn.Linear(64, 64), nn.Linear(64, 10)

        def forward(self, x):
            h = self.inp(x)
            s = torch.add(h, self.f1(h))
            early = s * 2.0                       # a consumer of the sum ahead of its LayerNorm
            y = self.n1(s)
            t = torch.add(y, early, alpha=0.5)    # scaled: not the pattern
            z = self.n2(t)
            u = z + self.f2(z)
            return self.f3(self.n3(u))

    torch.manual_seed(0)
    model = Net()
    ref = copy.deepcopy(model).eval()
    cfg = dict(default_bits=2, auto_precision=None, batch_size=8, min_activation_mib=0.0)
    c = Controller(model, cfg, input_shape=(16, 64), test=False, device="cpu")
    assert sorted(c.fused_add_layer_norm) == ["n1", "n3"]
    net = c.traced_model.eval()
    x = torch.randn(8, 16, 64)
    with torch.no_grad():
        assert torch.allclose(net(x), ref(x), atol=1e-5)


def test_controller_fuses_bn_relu():
    """A BatchNorm whose only consumer is a ReLU takes the ReLU over (the default); one with a
    second consumer, or followed by ReLU6, keeps its ReLU node."""
    from deep_optimization_b200.controller import Controller

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.c1, self.b1, self.r1 = nn.Conv2d(3, 64, 3, padding=1, bias=False), nn.BatchNorm2d(64), nn.ReLU()
            self.c2, self.b2, self.r2 = nn.Conv2d(64, 64, 3, padding=1, bias=False), nn.BatchNorm2d(64), nn.ReLU()
            self.c3, self.b3, self.r3 = nn.Conv2d(64, 64, 3, padding=1, bias=False), nn.BatchNorm2d(64), nn.ReLU6()

        def forward(self, x):
            x = self.r1(self.b1(self.c1(x)))
            y = self.b2(self.c2(x))
            x = self.r2(y) + y                      # b2 has two consumers
            return self.r3(self.b3(self.c3(x)))

    cfg = dict(default_bits=2, auto_precision=None, batch_size=64, min_activation_mib=1)
    c = Controller(Net(), cfg, input_shape=(3, 32, 32), test=False, device="cpu")
    net = c.traced_model
    assert c.fused_bn_relu == ["b1"]
    assert net.b1.fuse_relu and not net.b2.fuse_relu and not net.b3.fuse_relu
    targets = [n.target for n in net.graph.nodes if n.op == "call_module"]
    assert "r1" not in targets and "r2" in targets and "r3" in targets
    # eval mode: the fused module still applies the ReLU
    net.eval()
    ref = Net().eval()
    ref.load_state_dict({k: v for k, v in net.state_dict().items()})
    x = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        assert torch.allclose(net(x), ref(x), atol=1e-6)


def test_quantizer_policy():
    from deep_optimization_b200.quantizer import Quantizer
    q = Quantizer(dict(default_bits=4, auto_precision=None), {"a": None, "b": None})
    q.iterate()
    assert q.bits == {"a": 4, "b": 4}
    assert [q.hessian2bit_lookup_table(v) for v in (10, 60, 300, 600, 2000)] == [1, 2, 3, 4, 8]
    p = nn.Parameter(torch.zeros(3, 3))
    q.filter_tensors([("p", p)])
    assert not q.check_quantize(p)
    assert q.check_quantize(torch.zeros(2, 3, requires_grad=True))
    assert not q.check_quantize(torch.zeros(2, 3))
