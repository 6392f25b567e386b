"""GPU parity: the CUDA codec, called through the C ABI, against the CPU oracle.
Integer outputs (packed words) and fp32 scale/min must be bit-exact."""
import numpy as np
import pytest
import torch

from tests.inputs import adversarial_groups, gelu_normal, relu_normal, to_numpy, uniform_noise

pytestmark = pytest.mark.gpu

BITS = (1, 2, 4, 8)
GROUPS = (32, 64, 128, 256, 512, 1024)
DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _codec():
    from deep_optimization_b200 import codec
    return codec


def _same_bits(a: np.ndarray, b: np.ndarray) -> bool:
    return np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))


def _cmp_pack(oracle, got, want, what):
    packed, scale, mn = (t.cpu().numpy() for t in got)
    assert np.array_equal(packed.view(np.uint32), want[0]), f"packed words differ: {what}"
    nan = np.isnan(want[2])
    assert np.array_equal(np.isnan(mn), nan), what
    assert _same_bits(scale, want[1]), f"scale differs: {what}"
    assert _same_bits(mn[~nan], want[2][~nan]), f"min differs: {what}"


@pytest.mark.parametrize("dtype", DTYPES, ids=("f32", "bf16", "f16"))
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("gs", GROUPS)
def test_pack_all_modes(oracle, cuda_device, dtype, bits, gs):
    # 75 groups: odd count -> partial last tile for every group size but 1024
    x = relu_normal((75, gs), seed=bits + gs, dtype=dtype)
    u = uniform_noise(x.shape, seed=2)
    arr, tag = to_numpy(x)
    xd, ud = x.to(cuda_device), u.to(cuda_device)
    c = _codec()
    F = oracle
    cases = [
        ("noise tensor", dict(noise=ud), dict(noise=u.numpy())),
        ("hash noise", dict(seed=1234, offset=77), dict(seed=1234, offset=77)),
        ("round nearest", dict(flags=F.FLAG_ROUND_NEAREST), dict(flags=F.FLAG_ROUND_NEAREST)),
        ("ref compat", dict(flags=F.FLAG_REF_COMPAT | F.FLAG_META_BF16 | F.FLAG_REF_CLAMP, clamp_alpha=1.5),
         dict(flags=F.FLAG_REF_COMPAT | F.FLAG_META_BF16 | F.FLAG_REF_CLAMP, clamp_alpha=1.5)),
    ]
    for name, gkw, okw in cases:
        got = c.quant_pack(xd, bits, gs, **gkw)
        want = oracle.quant_pack(arr, gs, bits, dtype=tag, **okw)
        _cmp_pack(oracle, got, want, f"{name} {tag} b{bits} g{gs}")


@pytest.mark.parametrize("dtype", DTYPES, ids=("f32", "bf16", "f16"))
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("gs", (32, 128, 1024))
def test_unpack_bit_exact(oracle, cuda_device, dtype, bits, gs):
    rng = np.random.default_rng(bits * gs)
    ng = 77
    packed = rng.integers(0, 2**32, (ng, gs * bits // 32), dtype=np.uint64).astype(np.uint32)
    scale = rng.random(ng).astype(np.float32) + 1e-3
    mn = rng.standard_normal(ng).astype(np.float32)
    tag = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}[dtype]
    want = oracle.dequant_unpack(packed, scale, mn, gs, bits, out=tag)
    got = _codec().dequant_unpack(torch.from_numpy(packed.view(np.int32)).to(cuda_device),
                                  torch.from_numpy(scale).to(cuda_device),
                                  torch.from_numpy(mn).to(cuda_device), bits, gs, out_dtype=dtype)
    g, _ = to_numpy(got)
    assert np.array_equal(g.view(np.uint8), want.view(np.uint8))


@pytest.mark.parametrize("gs", (32, 64, 256))
@pytest.mark.parametrize("bits", BITS)
def test_adversarial_groups(oracle, cuda_device, bits, gs):
    """Constant groups, signed zeros, denormal / huge / overflowing ranges, inf, NaN."""
    x = adversarial_groups(gs)
    u = uniform_noise(x.shape, seed=5)
    c = _codec()
    for kw_g, kw_o in ((dict(noise=u.to(cuda_device)), dict(noise=u.numpy())),
                       (dict(seed=3, offset=0), dict(seed=3, offset=0)),
                       (dict(flags=oracle.FLAG_ROUND_NEAREST), dict(flags=oracle.FLAG_ROUND_NEAREST))):
        got = c.quant_pack(x.to(cuda_device), bits, gs, **kw_g)
        want = oracle.quant_pack(x.numpy(), gs, bits, **kw_o)
        _cmp_pack(oracle, got, want, f"adversarial b{bits} g{gs} {list(kw_o)}")


def test_negative_and_large_noise(oracle, cuda_device):
    """Noise outside [0,1) must hit the clamp exactly as the oracle does."""
    x = relu_normal((40, 128), seed=1)
    u = (uniform_noise(x.shape) * 6 - 3)
    for bits in BITS:
        got = _codec().quant_pack(x.to(cuda_device), bits, 128, noise=u.to(cuda_device))
        want = oracle.quant_pack(x.numpy(), 128, bits, noise=u.numpy())
        _cmp_pack(oracle, got, want, f"wide noise b{bits}")


def test_ref_compat_tanh_close(oracle, cuda_device):
    """The tanh squash uses the device's tanhf; codes may differ from libm's by a
    rounding step on a vanishing fraction of elements (tolerance: < 0.1 % of codes)."""
    x = relu_normal((64, 256), seed=8, dtype=torch.bfloat16)
    arr, tag = to_numpy(x)
    flags = oracle.FLAG_REF_COMPAT | oracle.FLAG_REF_CLAMP | oracle.FLAG_REF_TANH | oracle.FLAG_META_BF16
    got = _codec().quant_pack(x.to(cuda_device), 2, 256, flags=flags, clamp_alpha=3.0)
    want = oracle.quant_pack(arr, 256, 2, dtype=tag, flags=flags, clamp_alpha=3.0)
    gc = oracle.np_unpack_codes(got[0].cpu().numpy().view(np.uint32), 256, 2)
    wc = oracle.np_unpack_codes(want[0], 256, 2)
    assert (gc != wc).mean() < 1e-3
    assert np.allclose(got[1].cpu().numpy(), want[1], rtol=1e-2)


@pytest.mark.parametrize("bits", BITS)
def test_mask_pack_unpack(oracle, cuda_device, bits):
    rng = np.random.default_rng(bits)
    x = rng.integers(0, 1 << bits, (33, 128)).astype(np.int8)
    c = _codec()
    p = c.pack_bits(torch.from_numpy(x).to(cuda_device), bits, 128)
    assert np.array_equal(p.cpu().numpy().view(np.uint32), oracle.pack_bits(x, 128, bits))
    y = c.unpack_bits(p, bits, 33, 128)
    assert np.array_equal(y.cpu().numpy(), oracle.unpack_bits(oracle.pack_bits(x, 128, bits), 128, bits))


@pytest.mark.parametrize("dtype", DTYPES, ids=("f32", "bf16", "f16"))
def test_minmax(oracle, cuda_device, dtype):
    x = (relu_normal((37, 301), seed=6) - 0.3).to(dtype)
    arr, tag = to_numpy(x)
    mn, mx = _codec().minmax(x.to(cuda_device))
    wmn, wmx = oracle.minmax(arr, dtype=tag)
    assert _same_bits(mn.cpu().numpy(), wmn) and _same_bits(mx.cpu().numpy(), wmx)


def test_config1_full_size_round_trip(oracle, cuda_device):
    """fp32 [128,64,56,56], group 256, 2 bits: full-size properties plus an oracle
    comparison on a slice (the whole tensor takes the oracle a few seconds)."""
    x = relu_normal((128, 64, 56, 56), seed=0)
    u = uniform_noise(x.shape, seed=1)
    c = _codec()
    xd = x.to(cuda_device)
    packed, scale, mn = c.quant_pack(xd, 2, 256, noise=u.to(cuda_device))
    assert packed.shape == (100352, 16)
    want = oracle.quant_pack(x.numpy(), 256, 2, noise=u.numpy())
    _cmp_pack(oracle, (packed, scale, mn), want, "config 1")
    y = c.dequant_unpack(packed, scale, mn, 2, 256, out_dtype=torch.float32).view_as(xd)
    assert ((y - xd).abs().view(-1, 256) <= scale[:, None] * 1.0001 + 1e-6).all()
    # idempotence: values already on the code points re-quantise to themselves (u = 0)
    p2, s2, m2 = c.quant_pack(y, 2, 256, noise=torch.zeros_like(xd))
    y2 = c.dequant_unpack(p2, s2, m2, 2, 256, out_dtype=torch.float32).view_as(xd)
    assert (y2 - y).abs().max() <= 1e-6 * 8


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("kind", ("conv", "vit"))
def test_config2_sweep(oracle, cuda_device, bits, kind):
    """bf16 conv [256,256,28,28] / ViT [256,197,768], group 128: packed words, scale and minimum
    of ALL 401 408 / 302 592 groups against the C oracle (hash mode), the dequantised tensor too,
    plus size-independent properties on the whole tensor."""
    x = (relu_normal((256, 256, 28, 28), 0, torch.bfloat16) if kind == "conv"
         else gelu_normal((256, 197, 768), 0, torch.bfloat16))
    c = _codec()
    xd = x.to(cuda_device)
    packed, scale, mn = c.quant_pack(xd, bits, 128, seed=42, offset=0)
    arr, tag = to_numpy(x.reshape(-1, 128))
    want = oracle.quant_pack(arr, 128, bits, dtype=tag, seed=42, offset=0)
    _cmp_pack(oracle, (packed, scale, mn), want, f"config 2 {kind} b{bits}")
    want_y = oracle.dequant_unpack(want[0], want[1], want[2], 128, bits, out="bf16")
    got_y = c.dequant_unpack(packed, scale, mn, bits, 128, out_dtype=torch.bfloat16)
    assert np.array_equal(got_y.cpu().view(torch.int16).numpy().view(np.uint16), want_y)
    y = c.dequant_unpack(packed, scale, mn, bits, 128, out_dtype=torch.float32)
    err = (y - xd.float().view(-1, 128)).abs()
    assert (err <= scale[:, None] * 1.0001 + 1e-6).all()
    # checksum of checksums: group minima and maxima survive the codec exactly
    xg = xd.float().view(-1, 128)
    assert torch.equal(mn, xg.amin(1))
    yb = c.dequant_unpack(packed, scale, mn, bits, 128, out_dtype=torch.bfloat16)
    assert yb.dtype == torch.bfloat16 and yb.shape == (xd.numel() // 128, 128)


def test_empty_input(cuda_device):
    c = _codec()
    p, s, m = c.quant_pack(torch.empty((0, 128), device=cuda_device), 2, 128)
    assert p.shape == (0, 8) and s.numel() == 0
    assert c.dequant_unpack(p, s, m, 2, 128).shape == (0, 128)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("gs", (64, 256))
def test_cuda_against_reference_fixtures(oracle, cuda_device, bits, gs):
    """The CUDA kernels in reference-compatible mode against outputs of the reference's own
    Triton kernels (tests/golden/reference_triton_codec.npz, made under the CPU interpreter)."""
    import os
    fix = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_triton_codec.npz"))
    key = f"b{bits}_g{gs}"
    x = torch.from_numpy(fix[key + "_x"].view(np.int16)).view(torch.bfloat16).to(cuda_device)
    F = oracle
    c = _codec()
    for tag, flags, alpha in (("identity_n", F.FLAG_REF_COMPAT | F.FLAG_META_BF16, 0.0),
                              ("identity_c", F.FLAG_REF_COMPAT | F.FLAG_META_BF16 | F.FLAG_REF_CLAMP, 1.0)):
        packed, scale, mn = c.quant_pack(x, bits, gs, flags=flags, clamp_alpha=alpha)
        assert np.array_equal(packed.cpu().numpy().view(np.uint32), fix[f"{key}_{tag}_packed"]), tag
        assert np.array_equal(oracle.f32_to_bf16_bits(mn.cpu().numpy()), fix[f"{key}_{tag}_min"]), tag
    mask = torch.from_numpy(fix[key + "_mask"]).to(cuda_device)
    pk = c.pack_bits(mask, bits, gs)
    assert np.array_equal(pk.cpu().numpy().view(np.uint32), fix[key + "_mask_packed"])
    assert np.array_equal(c.unpack_bits(pk, bits, mask.shape[0], gs).cpu().numpy(), fix[key + "_mask_unpacked"])


def test_cuda_graph_capture_and_replay(oracle, cuda_device):
    """The entry points neither synchronise nor allocate, so a captured pack + unpack pair
    replays on new data (the reference drives its training step from CUDA graphs,
    Train/utils_train.py:92-180).  Noise stream and offset are frozen at capture time."""
    c = _codec()
    x = relu_normal((64, 4096), seed=3, dtype=torch.bfloat16).to(cuda_device)
    static_x = x.clone()
    ng = x.numel() // 128
    outs = (torch.empty((ng, 8), dtype=torch.int32, device=cuda_device),
            torch.empty(ng, device=cuda_device), torch.empty(ng, device=cuda_device))
    y = torch.empty((ng, 128), dtype=torch.bfloat16, device=cuda_device)
    c.quant_pack(static_x, 2, 128, seed=5, offset=9, out=outs)              # warm-up outside capture
    c.dequant_unpack(*outs, 2, 128, out_dtype=torch.bfloat16, out=y)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        c.quant_pack(static_x, 2, 128, seed=5, offset=9, out=outs)
        c.dequant_unpack(*outs, 2, 128, out_dtype=torch.bfloat16, out=y)
    x2 = relu_normal((64, 4096), seed=4, dtype=torch.bfloat16).to(cuda_device)
    static_x.copy_(x2)
    g.replay()
    torch.cuda.synchronize()
    arr, tag = to_numpy(x2)
    want = oracle.quant_pack(arr, 128, 2, dtype=tag, seed=5, offset=9)
    _cmp_pack(oracle, outs, want, "graph replay")
    wy = oracle.dequant_unpack(*want, 128, 2, out="bf16")
    assert np.array_equal(to_numpy(y)[0], wy)


def test_beyond_32bit_indices(oracle, cuda_device):
    """Maximum sizes: 2^34 + 2^20 bf16 elements (34 GB), so element indices pass 2^32 and the
    hash counters pass 2^32 as well.  Checked against the oracle on the first and on the last
    2^20 elements (the oracle is told where the slice sits), plus group minima everywhere."""
    free, _ = torch.cuda.mem_get_info(cuda_device)
    n_tail = 1 << 20
    n = (1 << 34) + n_tail
    if free < n * 2 * 1.4:
        pytest.skip("not enough free device memory for the 34 GB case")
    base = relu_normal((n_tail,), seed=9, dtype=torch.bfloat16).to(cuda_device)
    x = base.repeat(n // n_tail)
    assert x.numel() == n
    x[-n_tail:] = x[-n_tail:] * 0.5 + 0.25             # make the tail differ from the head
    c = _codec()
    gs, bits = 128, 2
    packed, scale, mn = c.quant_pack(x, bits, gs, seed=77, offset=5)
    ng_tail = n_tail // gs
    for first in (0, (n - n_tail) // gs):
        sl = x[first * gs: first * gs + n_tail]
        arr, tag = to_numpy(sl)
        want = oracle.quant_pack(arr, gs, bits, dtype=tag, seed=77, offset=5, first_group=first)
        got = (packed[first: first + ng_tail], scale[first: first + ng_tail], mn[first: first + ng_tail])
        _cmp_pack(oracle, got, want, f"slice at group {first}")
    # size-independent property on the whole tensor, in slabs to bound temporary memory
    slab = 1 << 28
    for s0 in range(0, n, slab * 8):
        xs = x[s0: s0 + slab].float().view(-1, gs)
        assert torch.equal(mn[s0 // gs: s0 // gs + xs.shape[0]], xs.amin(1))
    y = c.dequant_unpack(packed[-ng_tail:], scale[-ng_tail:], mn[-ng_tail:], bits, gs, out_dtype=torch.float32)
    err = (y - x[-n_tail:].float().view(-1, gs)).abs()
    assert (err <= scale[-ng_tail:, None] * 1.0001 + 1e-6).all()


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16, torch.float16), ids=("f32", "bf16", "f16"))
@pytest.mark.parametrize("tile", (8, 16, 32))
@pytest.mark.parametrize("bits", (1, 2, 4, 8))
def test_tiled_addressing_equals_permute(cuda_device, dtype, tile, bits):
    """quant_pack_tiles reads sqrt(gs) x sqrt(gs) spatial tiles in place: packed words, scale and
    min equal those of the flat kernel on the permuted copy (same hash counters); the tiled
    unpack writes what the flat unpack plus the inverse permute give.  Shapes include a partial
    last kernel tile and H != W."""
    from deep_optimization_b200 import codec
    g = torch.Generator().manual_seed(31 + tile + bits)
    N, C, H, W = 3, 5, 2 * tile, 3 * tile
    x = (torch.randn((N, C, H, W), generator=g) * 3).to(dtype).to(cuda_device)
    gs = tile * tile
    xp = x.reshape(N, C, H // tile, tile, W // tile, tile).permute(0, 1, 2, 4, 3, 5).reshape(-1, gs).contiguous()
    for flags in (0, 1):
        want = codec.quant_pack(xp, bits, gs, seed=5, offset=9, flags=flags)
        got = codec.quant_pack_tiles(x, bits, tile, seed=5, offset=9, flags=flags)
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]) and torch.equal(got[2], want[2])
    for out_dtype in (torch.bfloat16, torch.float32):
        flat = codec.dequant_unpack(*want, bits, gs, out_dtype=out_dtype)
        back = flat.reshape(N, C, H // tile, W // tile, tile, tile).permute(0, 1, 2, 4, 3, 5).reshape(N, C, H, W)
        y = codec.dequant_unpack_tiles(*got, bits, tile, (N, C, H, W), out_dtype=out_dtype)
        assert torch.equal(y, back)


def test_module_utils_uses_tiles(cuda_device):
    """The quantise boundary takes the in-place tiled kernels for spatially groupable inputs and
    returns the same tensors and meta as the permute path."""
    from deep_optimization_b200 import codec
    from deep_optimization_b200.modules import module_utils as mu
    from deep_optimization_b200.modules.tensor_act_reshape_utils import spatical_aware_act_tensor_reshape
    x = torch.randn(4, 6, 32, 48, device=cuda_device).to(torch.bfloat16)
    codec.manual_seed(77)
    (p, s, m), meta = mu.quantize(x, 2, False, 256, False, 4, False, 0, False, 0.0)
    groups, N, G, nh, nw, shape, pad_e, re_e, cm = spatical_aware_act_tensor_reshape(x, 256, False, False)
    assert meta == (2, False, 256, False, N, G, nh, nw, pad_e, re_e, cm, False, 0, shape)
    assert p.shape == (N * G, 16) and s.shape == (N, G) and m.shape == (N, G)
    y = mu.dequantize((p, s, m), meta)
    assert y.shape == x.shape and y.dtype == torch.bfloat16
    step = s.reshape(4, 6, 2, 3, 1, 1).expand(4, 6, 2, 3, 16, 16).permute(0, 1, 2, 4, 3, 5).reshape(4, 6, 32, 48)
    assert ((y.float() - x.float()).abs() <= step * 1.01 + 0.02 * x.float().abs()).all()


@pytest.mark.parametrize("dtype", DTYPES, ids=("f32", "bf16", "f16"))
@pytest.mark.parametrize("gs", GROUPS)
def test_three_bit_planes(oracle, cuda_device, dtype, gs):
    """3-bit codes in the bit-plane layout (cpp_extension pack3 / unpack3): packed words, scale
    and min bit-exact with the oracle in the noise-tensor, hash and nearest modes on an odd
    number of groups; decoded values bit-exact; adversarial groups included."""
    c = _codec()
    x = torch.cat([relu_normal((75, gs), seed=3 + gs, dtype=dtype), adversarial_groups(gs).to(dtype)])
    u = uniform_noise(x.shape, seed=2)
    arr, tag = to_numpy(x)
    xd, ud = x.to(cuda_device), u.to(cuda_device)
    F = oracle
    for name, gkw, okw in (("noise tensor", dict(noise=ud), dict(noise=u.numpy())),
                           ("hash noise", dict(seed=1234, offset=77), dict(seed=1234, offset=77)),
                           ("round nearest", dict(flags=F.FLAG_ROUND_NEAREST), dict(flags=F.FLAG_ROUND_NEAREST))):
        got = c.quant_pack(xd, 3, gs, planes3=True, **gkw)
        want = oracle.quant_pack(arr, gs, 3, dtype=tag, **okw)
        _cmp_pack(oracle, got, want, f"3-bit {name} {tag} g{gs}")
    ok = np.isfinite(want[2]) & np.isfinite(want[1])         # NaN payloads are not compared
    y = c.dequant_unpack(got[0], got[1], got[2], 3, gs, out_dtype=dtype, planes3=True)
    yw = oracle.dequant_unpack(want[0], want[1], want[2], gs, 3, out=tag)
    g, _ = to_numpy(y)
    assert np.array_equal(g.view(np.uint8).reshape(len(ok), -1)[ok], yw.view(np.uint8).reshape(len(ok), -1)[ok])
    with pytest.raises(ValueError):
        c.quant_pack(xd, 3, gs)                      # the act_lib contract: bits in (1,2,4,8)


@pytest.mark.parametrize("dtype", DTYPES, ids=("f32", "bf16", "f16"))
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("avg", (2, 4, 8))
def test_sub_group_averaging(oracle, cuda_device, dtype, bits, avg):
    """AVG_ALAM (one code per `avg` neighbours): packed words, scale and min bit-exact with the
    oracle in the four modes, decoded values bit-exact, odd group counts, all group sizes that
    give whole words."""
    c = _codec()
    F = oracle
    for gs in GROUPS:
        if (gs * bits) % (32 * avg):
            with pytest.raises(ValueError):
                c.quant_pack_avg(torch.zeros(gs, device=cuda_device), bits, gs, avg)
            continue
        x = relu_normal((37, gs), seed=bits + gs + avg, dtype=dtype)
        u = uniform_noise(x.shape, seed=2)
        arr, tag = to_numpy(x)
        xd, ud = x.to(cuda_device), u.to(cuda_device)
        ref = F.FLAG_REF_COMPAT | F.FLAG_META_BF16 | F.FLAG_REF_CLAMP
        for name, gkw, okw in (("noise tensor", dict(noise=ud), dict(noise=u.numpy())),
                               ("hash noise", dict(seed=1234, offset=77), dict(seed=1234, offset=77)),
                               ("round nearest", dict(flags=F.FLAG_ROUND_NEAREST), dict(flags=F.FLAG_ROUND_NEAREST)),
                               ("ref compat", dict(flags=ref, clamp_alpha=1.5), dict(flags=ref, clamp_alpha=1.5))):
            got = c.quant_pack_avg(xd, bits, gs, avg, **gkw)
            want = oracle.quant_pack_avg(arr, gs, bits, avg, dtype=tag, **okw)
            _cmp_pack(oracle, got, want, f"avg{avg} {name} {tag} b{bits} g{gs}")
        y = c.dequant_unpack_avg(got[0], got[1], got[2], bits, gs, avg, out_dtype=dtype)
        yw = oracle.dequant_unpack_avg(want[0], want[1], want[2], gs, bits, avg, out=tag)
        g, _ = to_numpy(y)
        assert np.array_equal(g.view(np.uint8), yw.view(np.uint8))


def test_avg_alam_through_the_operators(cuda_device):
    """quantize / dequantize with AVG_ALAM set: the packed tensor shrinks by alam_bits and the
    decoded activation is piecewise constant over alam_bits neighbours, near the input's local mean."""
    from deep_optimization_b200.modules.module_utils import unified_dequantize, unified_quantize
    meta = {"t": {"bits": 2, "pack_only": False, "group_size": 256, "act_padding": False, "N": 4,
                  "AVG_ALAM": True, "ALAM_BITS": 4, "DIVISION": None}}
    x = torch.relu(torch.randn(4, 8, 10, 32, device=cuda_device)).to(torch.bfloat16)   # flat grouping (H % 16 != 0)
    q, q_meta, _ = unified_quantize(x, None, "t", meta, clamp=False, clamp_alpha=0.0)
    assert q[0].shape == (x.numel() // 256, 256 * 2 // 32 // 4)
    y = unified_dequantize(q, q_meta, None)
    assert y.shape == x.shape
    yg = y.float().reshape(-1, 4)
    assert (yg == yg[:, :1]).all()
    step = q[1].float().reshape(-1, 1).repeat_interleave(64, 0)
    assert ((yg[:, :1] - x.float().reshape(-1, 4).mean(1, keepdim=True)).abs() <= step * 1.05 + 0.02).all()
