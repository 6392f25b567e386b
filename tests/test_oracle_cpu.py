"""CPU tests: the C oracle against its numpy restatement and against properties
of the scheme.  No GPU, no product code."""
import numpy as np
import pytest

from tests.inputs import adversarial_groups, relu_normal, to_numpy, uniform_noise

BITS = (1, 2, 4, 8)
GROUPS = (32, 64, 128, 256, 512, 1024)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("gs", GROUPS)
def test_c_matches_numpy(oracle, bits, gs):
    x = relu_normal((48, gs), seed=bits * 100 + gs).numpy()
    u = uniform_noise(x.shape, seed=3).numpy()
    modes = (dict(noise=u), dict(seed=11, offset=5), dict(flags=oracle.FLAG_ROUND_NEAREST),
             dict(flags=oracle.FLAG_REF_COMPAT | oracle.FLAG_META_BF16))
    for kw in modes:
        a = oracle.quant_pack(x, gs, bits, **kw)
        b = oracle.np_quant_pack(x, gs, bits, **kw)
        for p, q in zip(a, b):
            assert np.array_equal(p.view(np.uint32), q.view(np.uint32)), kw.keys()
    y = oracle.dequant_unpack(*a, gs, bits)
    assert np.array_equal(y, oracle.np_dequant(*a, gs, bits))


@pytest.mark.parametrize("dtype", ("bf16", "f16"))
def test_16bit_inputs(oracle, dtype):
    import torch
    t = relu_normal((16, 128), seed=5, dtype=torch.bfloat16 if dtype == "bf16" else torch.float16)
    arr, tag = to_numpy(t)
    u = uniform_noise(t.shape).numpy()
    a = oracle.quant_pack(arr, 128, 2, noise=u, dtype=tag)
    b = oracle.quant_pack(t.float().numpy(), 128, 2, noise=u)       # widening is exact
    for p, q in zip(a, b):
        assert np.array_equal(p.view(np.uint32), q.view(np.uint32))


def test_layout_known_answer(oracle):
    """Hand-computed case: values on the code points, u = 0 -> code i of word w at bits [2i,2i+2)."""
    gs = 32
    x = (np.arange(gs) % 4).astype(np.float32)[None, :]
    packed, scale, mn = oracle.quant_pack(x, gs, 2, noise=np.zeros_like(x))
    assert scale[0] == 1.0 and mn[0] == 0.0
    word = sum((i % 4) << (2 * i) for i in range(16))
    assert packed.tolist() == [[word, word]]
    assert packed.view(np.uint8)[0, 0] == 0b11100100       # 4 codes per byte, little end first
    y = oracle.dequant_unpack(packed, scale, mn, gs, 2)
    assert np.array_equal(y, x)


def test_degenerate_and_nonfinite(oracle):
    x = adversarial_groups(64).numpy()
    packed, scale, mn = oracle.quant_pack(x, 64, 2, noise=np.full(x.shape, 0.5, np.float32))
    assert scale[0] == 1.0 and scale[1] == 1.0 and scale[2] == 1.0      # constant groups
    assert np.signbit(mn[2])                                            # -0 orders below +0
    assert (packed[:3] == 0).all()
    assert np.isnan(mn[9]) and scale[9] == 1.0 and (packed[9] == 0).all()   # NaN poisons its group


@pytest.mark.parametrize("bits", BITS)
def test_round_trip_bound(oracle, bits):
    x = relu_normal((64, 256), seed=2).numpy()
    u = uniform_noise(x.shape).numpy()
    packed, scale, mn = oracle.quant_pack(x, 256, bits, noise=u)
    y = oracle.dequant_unpack(packed, scale, mn, 256, bits)
    assert (np.abs(y - x) <= scale[:, None] * 1.0001 + 1e-6).all()      # stochastic: within one step
    packed, scale, mn = oracle.quant_pack(x, 256, bits, flags=oracle.FLAG_ROUND_NEAREST)
    y = oracle.dequant_unpack(packed, scale, mn, 256, bits)
    # nearest on the 1/256 fixed-point grid: within half a step plus the grid's own rounding
    assert (np.abs(y - x) <= scale[:, None] * (0.5 + 1.0 / 128) + 1e-6).all()


def test_stochastic_rounding_unbiased(oracle):
    x = np.full((4096, 32), 0.3, np.float32)
    x[:, 0], x[:, 1] = 0.0, 1.0                       # range [0,1], 1-bit: P(code=1) = 0.3
    packed, _, _ = oracle.quant_pack(x, 32, 1, seed=9)
    codes = oracle.np_unpack_codes(packed, 32, 1)[:, 2:]
    assert abs(codes.mean() - 0.3) < 0.01


def test_mask_pack_round_trip(oracle):
    rng = np.random.default_rng(0)
    for bits in BITS:
        x = rng.integers(0, 1 << bits, (7, 128)).astype(np.int8)
        p = oracle.pack_bits(x, 128, bits)
        assert np.array_equal(oracle.unpack_bits(p, 128, bits).view(np.uint8), x.view(np.uint8))
        assert np.array_equal(oracle.np_unpack_codes(p, 128, bits).astype(np.uint8), x.view(np.uint8))


def test_hash_noise_restatement(oracle):
    for seed, off in ((0, 0), (5, 9), (2**63 + 1, 2**40)):
        assert np.array_equal(oracle.hash_noise(seed, off, 3, 4099), oracle.np_hash_noise(seed, off, 3, 4099))


def test_hash_noise_statistics(oracle):
    """The noise bytes are uniform, free of pair structure at the lags the kernel's lane
    layout produces, and unrelated across seeds and offsets (chi-square with 255 degrees of
    freedom: mean 255, sd 22.6; the bound is mean + 5.5 sd)."""
    n = 1 << 21
    bound = 255 + 5.5 * 22.6
    chi = lambda c, e: float(((c - e) ** 2 / e).sum())
    streams = {}
    for seed, off in ((0, 0), (1, 0), (0, 1), (12345, 999), (7, 2**40)):
        h = oracle.np_hash_bytes(seed, off, 0, n).astype(np.int64)
        streams[(seed, off)] = h
        assert chi(np.bincount(h, minlength=256), n / 256) < bound
        for lag in (1, 2, 3, 4, 7, 8, 9, 16, 64, 128, 1024):
            c = np.bincount((h[:-lag] >> 4) * 16 + (h[lag:] >> 4), minlength=256)
            assert chi(c, (n - lag) / 256) < bound, (seed, off, lag)
            c = np.bincount((h[:-lag] & 15) * 16 + (h[lag:] & 15), minlength=256)
            assert chi(c, (n - lag) / 256) < bound, (seed, off, lag)
        u = h / 256.0
        assert abs(u.mean() - 255 / 512) < 4 * 0.2887 / np.sqrt(n)
    keys = list(streams)
    for i in range(len(keys)):
        for j in range(i + 1, len(keys)):
            a, b = streams[keys[i]], streams[keys[j]]
            assert abs(np.corrcoef(a, b)[0, 1]) < 5 / np.sqrt(n)
            c = np.bincount((a >> 4) * 16 + (b >> 4), minlength=256)
            assert chi(c, n / 256) < bound


def test_hash_mode_is_unbiased_fixed_point(oracle):
    """In hash mode the mean code over many noise streams is Q/256 = RNE(q*256)/256."""
    x = np.linspace(0.0, 1.0, 128, dtype=np.float32).reshape(1, 128)
    acc = np.zeros(128)
    reps = 4000
    for off in range(reps):
        p, s, mn = oracle.quant_pack(x, 128, 2, seed=3, offset=off)
        acc += oracle.np_unpack_codes(p, 128, 2)[0]
    q = (x[0] - mn[0]) / s[0]
    assert np.abs(acc / reps - q).max() < 4 * 0.5 / np.sqrt(reps) + 1 / 256


def test_exact_fma_agrees(oracle):
    rng = np.random.default_rng(1)
    s = rng.random(200).astype(np.float32)
    m = rng.standard_normal(200).astype(np.float32)
    packed = np.full((200, 1), 0xE4E4E4E4, np.uint32)        # codes 0,1,2,3 repeating, 16 per word
    y = oracle.dequant_unpack(np.repeat(packed, 2, 1), s, m, 32, 2)
    for g in range(200):
        for c in range(4):
            assert y[g, c] == oracle.exact_fma_f32(c, s[g], m[g])


def test_division_sequence(oracle):
    rng = np.random.default_rng(3)
    n = 4_000_000
    s = (np.exp2(rng.uniform(-58, 50, n)) * rng.uniform(1, 2, n)).astype(np.float32)
    qmax = rng.choice([1, 3, 15, 255], n).astype(np.float32)
    a = (s * qmax * rng.random(n, dtype=np.float32)).astype(np.float32)
    assert oracle.check_div_sequence(a, s) == 0
    assert oracle.check_div_sequence((s * qmax).astype(np.float32), s) == 0


def test_calc_precision(oracle):
    out = oracle.calc_precision([8, 8, 8, 8], [10, 200, 3000, 5], [1, 1, 1, 1], 20.0)
    assert out.sum() <= 20 and out.tolist() == [4, 6, 7, 3]
    with pytest.raises(ValueError):
        oracle.calc_precision([2, 2], [1, 1], [1, 1], -5.0)


def test_minmax(oracle):
    x = relu_normal((9, 333), seed=4).numpy() - 0.5
    mn, mx = oracle.minmax(x)
    assert np.array_equal(mn, x.min(1)) and np.array_equal(mx, x.max(1))


def test_e4m3_decode(oracle):
    import torch
    b = np.arange(256, dtype=np.uint8)
    ref = torch.from_numpy(b).view(torch.float8_e4m3fn).float().numpy()
    got = oracle.e4m3_decode(b)
    assert np.array_equal(np.isnan(ref), np.isnan(got))
    assert np.array_equal(ref[~np.isnan(ref)], got[~np.isnan(got)])


def test_fp8_gemm_small(oracle):
    import torch
    g = torch.Generator().manual_seed(0)
    A = torch.randn(8, 64, generator=g); B = torch.randn(64, 12, generator=g)
    sa = A.abs().amax(1) / 448; sb = B.abs().amax(0) / 448
    A8 = (A / sa[:, None]).to(torch.float8_e4m3fn); B8 = (B / sb[None, :]).to(torch.float8_e4m3fn)
    C, Cf = oracle.fp8_gemm(A8.view(torch.uint8).numpy(), B8.view(torch.uint8).numpy(), sa.numpy(), sb.numpy())
    ref = (A8.double() @ B8.double()).float() * sa[:, None] * sb[None, :]
    assert np.array_equal(Cf, ref.numpy())
    assert np.allclose(Cf, (A @ B).numpy(), rtol=0.2, atol=0.5)


@pytest.mark.parametrize("gs", GROUPS)
def test_three_bit_planes(oracle, gs):
    """3-bit codes (the cpp_extension pack3 / unpack3 width): C against numpy in the three
    non-reference modes, codes <= 7, round trip within one step, and the bit-plane layout on a
    hand-made case: element l of a 32-element chunk with code c sets bit l of word p for every
    set bit p of c."""
    x = relu_normal((20, gs), seed=300 + gs).numpy()
    u = uniform_noise(x.shape, seed=3).numpy()
    for kw in (dict(noise=u), dict(seed=11, offset=5), dict(flags=oracle.FLAG_ROUND_NEAREST)):
        a = oracle.quant_pack(x, gs, 3, **kw)
        b = oracle.np_quant_pack(x, gs, 3, **kw)
        for p, q in zip(a, b):
            assert np.array_equal(p.view(np.uint32), q.view(np.uint32)), kw.keys()
        assert a[0].shape == (20, gs * 3 // 32)
        codes = oracle.np_unpack_codes(a[0], gs, 3)
        assert codes.max() <= 7
        y = oracle.dequant_unpack(*a, gs, 3)
        assert np.array_equal(y, oracle.np_dequant(*a, gs, 3))
        assert (np.abs(y - x) <= a[1][:, None] * (1 + 1e-6)).all()
    with pytest.raises(ValueError):
        oracle.quant_pack(x, gs, 3, flags=oracle.FLAG_REF_COMPAT)
    # values on the code points, no noise: code of element i is i % 8
    ramp = np.tile(np.arange(8, dtype=np.float32), gs // 8)[None, :]
    packed, scale, mn = oracle.quant_pack(ramp, gs, 3, noise=np.zeros_like(ramp))
    assert scale[0] == 1.0 and mn[0] == 0.0
    want = [sum(((l % 8) >> p & 1) << l for l in range(32)) for p in range(3)]
    assert packed[0, :3].tolist() == want and packed[0, -3:].tolist() == want


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("avg", (2, 4, 8))
def test_sub_group_averaging(oracle, bits, avg):
    """AVG_ALAM: one code per `avg` neighbours.  C against numpy in all four modes; the decoded
    value of a sub-group is one number, within one step of the sub-group's mean."""
    for gs in (64, 256, 1024):
        if (gs * bits) % (32 * avg):
            with pytest.raises(ValueError):
                oracle.quant_pack_avg(np.zeros(gs, np.float32), gs, bits, avg)
            continue
        x = relu_normal((24, gs), seed=bits * 10 + avg + gs).numpy()
        u = uniform_noise(x.shape, seed=3).numpy()
        for kw in (dict(noise=u), dict(seed=11, offset=5), dict(flags=oracle.FLAG_ROUND_NEAREST),
                   dict(flags=oracle.FLAG_REF_COMPAT)):
            a = oracle.quant_pack_avg(x, gs, bits, avg, **kw)
            b = oracle.np_quant_pack_avg(x, gs, bits, avg, **kw)
            for p, q in zip(a, b):
                assert np.array_equal(p.view(np.uint32), q.view(np.uint32)), (gs, kw.keys())
            assert a[0].shape == (24, gs * bits // (32 * avg))
            y = oracle.dequant_unpack_avg(*a, gs, bits, avg).reshape(24, gs // avg, avg)
            assert (y == y[:, :, :1]).all()
            mean = x.reshape(24, gs // avg, avg).mean(2)
            assert (np.abs(y[:, :, 0] - mean) <= a[1][:, None] * 1.001 + 1e-6).all()


# ------------------------------------------------------------- ballot-plane codec (legacy)
def test_sgd_noise_known_answers(oracle):
    """The reference's index hash (cpp_extension/include/quant_common.h:32-43): the C oracle
    against a restatement in Python integers, on fixed keys with their values written out (worked
    by hand from the three steps: x ^= x >> 32; x *= 0xD6E8FEB86659FD93; x ^= x >> 32; top 24
    bits / 2^24 - 0.5) and on random keys."""
    keys = np.array([0, 1, (5 << 32) ^ 42, (123456789 << 32) ^ 0xDEADBEEF, 2 ** 64 - 1], np.uint64)
    want = np.array([-0.5, 0.33949267864227295, -0.044788897037506104, -0.2671549320220947, 0.10018932819366455],
                    np.float32)
    assert np.array_equal(oracle.sgd_noise(keys), want)
    # key 1 by hand: 1 ^ 0 = 1; 1 * M = 0xD6E8FEB86659FD93; ^= >> 32 leaves the top 32 bits, 0xD6E8FEB8;
    # top 24 bits 0xD6E8FE = 14084350; 14084350 / 2^24 - 0.5
    assert want[1] == np.float32(np.float32(14084350) * np.float32(2.0 ** -24) - np.float32(0.5))
    rng = np.random.default_rng(0)
    rk = rng.integers(0, 2 ** 63, size=2000, dtype=np.uint64) * np.uint64(2) + rng.integers(0, 2, size=2000, dtype=np.uint64)
    got = oracle.sgd_noise(rk)
    assert all(got[i] == np.float32(oracle.py_sgd_noise(int(rk[i]))) for i in range(rk.size))
    assert got.min() >= -0.5 and got.max() < 0.5 and abs(float(got.mean())) < 0.02


@pytest.mark.parametrize("bits", (1, 2, 3, 4, 8))
def test_ballot_layout_and_round_trip(oracle, bits):
    """Bit p of a code sits at bit `lane` of word p of its 32-element chunk; decode inverts it;
    the unbiased rounding stays within one step and is unbiased, the reference's variant sits
    half a step lower."""
    rng = np.random.default_rng(bits)
    gs, ng = 64, 40
    x = rng.random((ng, gs), dtype=np.float32) * 4 - 1
    mn, mx = x.min(1), x.max(1)
    packed, scale = oracle.pack_ballot(x, mn, mx, gs, bits, seed=11)
    words = packed.reshape(ng, gs // 32, bits)
    codes = np.zeros((ng, gs), np.int64)
    for p in range(bits):
        codes += (((words[:, :, p, None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(ng, gs).astype(np.int64)) << p
    y = oracle.unpack_ballot(packed, scale, mn, gs, bits)
    assert np.array_equal(y, (codes.astype(np.float32) / scale[:, None] + mn[:, None]).astype(np.float32))
    step = 1.0 / scale[:, None]
    assert (np.abs(y - x) <= step * 1.0001).all()
    assert abs(float(((y - x) / step).mean())) < 0.03
    pb, _ = oracle.pack_ballot(x, mn, mx, gs, bits, seed=11, flags=oracle.FLAG_BALLOT_REF_BIAS)
    yb = oracle.unpack_ballot(pb, scale, mn, gs, bits)
    bias = float(((yb - x) / step).mean())
    assert -0.56 < bias < (-0.2 if bits == 1 else -0.44)      # clipped at code 0, hence above -0.5
