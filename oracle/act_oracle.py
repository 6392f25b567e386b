"""ctypes front end of the CPU oracle plus an independent numpy restatement.

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and
by the CPU-baseline / reference legs of ``bench.py`` as the checker.  Nothing in
the product package imports this module.

Two implementations live here on purpose:

* ``lib`` functions (``quant_pack``, ``dequant_unpack`` ...) call the C file
  ``act_oracle.c`` (built by ``oracle/Makefile``).  That is the oracle of record
  and the timed CPU baseline.
* ``np_*`` functions restate the same arithmetic with numpy only, written
  separately, so the C file is cross-checked by a second formulation.

The arithmetic and the reference lines each function follows are listed at the
top of ``act_oracle.c``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from fractions import Fraction

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libact_oracle.so")

DT_F32, DT_BF16, DT_F16 = 0, 1, 2
FLAG_ROUND_NEAREST = 1
FLAG_REF_COMPAT = 2
FLAG_REF_CLAMP = 4
FLAG_REF_TANH = 8
FLAG_META_BF16 = 16
FLAG_BALLOT_REF_BIAS = 32

HALF_C = np.float32(0.5) - np.float32(1e-6)


def build(force: bool = False) -> str:
    """Compile act_oracle.c with the Makefile beside it; returns the .so path."""
    src = os.path.join(_HERE, "act_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libact_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        vp, i32, i64, u64, f32 = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64,
                                  ctypes.c_uint64, ctypes.c_float)
        L.oracle_quant_pack.argtypes = [vp, i32, i64, i32, i32, vp, u64, u64, i32, f32, vp, vp, vp]
        L.oracle_quant_pack_slice.argtypes = [vp, i32, i64, i32, i32, vp, u64, u64, i32, f32, vp, vp, vp, i64]
        L.oracle_dequant_unpack.argtypes = [vp, vp, vp, i64, i32, i32, i32, vp]
        L.oracle_quant_pack_avg.argtypes = [vp, i32, i64, i32, i32, i32, vp, u64, u64, i32, f32, vp, vp, vp]
        L.oracle_dequant_unpack_avg.argtypes = [vp, vp, vp, i64, i32, i32, i32, i32, vp]
        L.oracle_pack_bits.argtypes = [vp, i64, i32, i32, vp]
        L.oracle_unpack_bits.argtypes = [vp, i64, i32, i32, vp]
        L.oracle_minmax.argtypes = [vp, i32, i64, i64, vp, vp]
        L.oracle_calc_precision.argtypes = [vp, vp, vp, i64, ctypes.c_double]
        L.oracle_fp8_gemm.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32]
        L.oracle_e4m3_decode.argtypes = [vp, i64, vp]
        L.oracle_hash_noise.argtypes = [u64, u64, i64, i64, vp]
        L.oracle_hash_noise.restype = None
        L.oracle_check_div_sequence.argtypes = [vp, vp, i64]
        L.oracle_check_div_sequence.restype = i64
        L.oracle_num_threads.restype = i32
        L.oracle_set_threads.argtypes = [i32]
        L.oracle_set_threads.restype = None
        L.oracle_sgd_noise.argtypes = [vp, i64, vp]
        L.oracle_sgd_noise.restype = None
        L.oracle_pack_ballot.argtypes = [vp, i32, i64, i32, i32, vp, vp, u64, i32, vp, vp]
        L.oracle_unpack_ballot.argtypes = [vp, vp, vp, i32, i64, i32, i32, vp]
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _dtype_code(a: np.ndarray, dtype: str | None) -> int:
    """numpy has no bfloat16: bf16 data travels as uint16 with dtype='bf16'."""
    if dtype is not None:
        return {"f32": DT_F32, "bf16": DT_BF16, "f16": DT_F16}[dtype]
    if a.dtype == np.float32:
        return DT_F32
    if a.dtype == np.float16:
        return DT_F16
    raise TypeError("pass dtype='bf16' with a uint16 array for bfloat16 data")


def set_threads(n: int) -> None:
    lib().oracle_set_threads(int(n))


def num_threads() -> int:
    return int(lib().oracle_num_threads())


# ------------------------------------------------------------------ C oracle

def quant_pack(x: np.ndarray, group_size: int, bits: int, noise: np.ndarray | None = None,
               seed: int = 0, offset: int = 0, flags: int = 0, clamp_alpha: float = 0.0,
               dtype: str | None = None, first_group: int = 0):
    """x: any shape whose element count is a multiple of group_size (row-major groups).
    Returns (packed uint32 [NG, group_size*bits/32], scale f32 [NG], min f32 [NG]).
    `first_group` places x as a slice of a larger tensor (it shifts the hash counters)."""
    x = np.ascontiguousarray(x)
    code = _dtype_code(x, dtype)
    ng, rem = divmod(x.size, group_size)
    assert rem == 0
    packed = np.empty((ng, group_size * bits // 32), np.uint32)
    scale = np.empty(ng, np.float32)
    mn = np.empty(ng, np.float32)
    if noise is not None:
        noise = np.ascontiguousarray(noise, np.float32)
        assert noise.size == x.size
    rc = lib().oracle_quant_pack_slice(_ptr(x), code, ng, group_size, bits, _ptr(noise), seed, offset,
                                       flags, clamp_alpha, _ptr(packed), _ptr(scale), _ptr(mn), first_group)
    if rc:
        raise ValueError(f"oracle_quant_pack rejected bits={bits} group_size={group_size}")
    return packed, scale, mn


def dequant_unpack(packed: np.ndarray, scale: np.ndarray, mn: np.ndarray, group_size: int,
                   bits: int, out: str = "f32") -> np.ndarray:
    """Returns [NG, group_size]: float32, float16, or uint16 holding bf16 bits."""
    packed = np.ascontiguousarray(packed, np.uint32)
    scale = np.ascontiguousarray(scale, np.float32)
    mn = np.ascontiguousarray(mn, np.float32)
    ng = scale.size
    code = {"f32": DT_F32, "bf16": DT_BF16, "f16": DT_F16}[out]
    y = np.empty((ng, group_size), {DT_F32: np.float32, DT_BF16: np.uint16, DT_F16: np.float16}[code])
    rc = lib().oracle_dequant_unpack(_ptr(packed), _ptr(scale), _ptr(mn), ng, group_size, bits,
                                     code, _ptr(y))
    if rc:
        raise ValueError("oracle_dequant_unpack rejected its arguments")
    return y


def quant_pack_avg(x: np.ndarray, group_size: int, bits: int, avg: int, noise: np.ndarray | None = None,
                   seed: int = 0, offset: int = 0, flags: int = 0, clamp_alpha: float = 0.0,
                   dtype: str | None = None):
    """Sub-group averaging: one code per `avg` consecutive elements.  Returns (packed uint32
    [NG, group_size*bits/(32*avg)], scale f32 [NG], min f32 [NG])."""
    x = np.ascontiguousarray(x)
    code = _dtype_code(x, dtype)
    ng, rem = divmod(x.size, group_size)
    assert rem == 0
    packed = np.empty((ng, group_size * bits // (32 * avg)), np.uint32)
    scale = np.empty(ng, np.float32)
    mn = np.empty(ng, np.float32)
    if noise is not None:
        noise = np.ascontiguousarray(noise, np.float32)
    rc = lib().oracle_quant_pack_avg(_ptr(x), code, ng, group_size, bits, avg, _ptr(noise), seed, offset,
                                     flags, clamp_alpha, _ptr(packed), _ptr(scale), _ptr(mn))
    if rc:
        raise ValueError(f"oracle_quant_pack_avg rejected bits={bits} group_size={group_size} avg={avg}")
    return packed, scale, mn


def dequant_unpack_avg(packed: np.ndarray, scale: np.ndarray, mn: np.ndarray, group_size: int,
                       bits: int, avg: int, out: str = "f32") -> np.ndarray:
    packed = np.ascontiguousarray(packed, np.uint32)
    scale = np.ascontiguousarray(scale, np.float32)
    mn = np.ascontiguousarray(mn, np.float32)
    ng = scale.size
    code = {"f32": DT_F32, "bf16": DT_BF16, "f16": DT_F16}[out]
    y = np.empty((ng, group_size), {DT_F32: np.float32, DT_BF16: np.uint16, DT_F16: np.float16}[code])
    rc = lib().oracle_dequant_unpack_avg(_ptr(packed), _ptr(scale), _ptr(mn), ng, group_size, bits, avg,
                                         code, _ptr(y))
    if rc:
        raise ValueError("oracle_dequant_unpack_avg rejected its arguments")
    return y


def np_quant_pack_avg(x: np.ndarray, group_size: int, bits: int, avg: int, noise: np.ndarray | None = None,
                      seed: int = 0, offset: int = 0, flags: int = 0):
    """numpy restatement of oracle_quant_pack_avg (finite fp32 inputs; no clamp/tanh, fp32 meta)."""
    qmax = (1 << bits) - 1
    vpw = 32 // bits
    v = np.ascontiguousarray(x, np.float32).reshape(-1, group_size)
    ng = v.shape[0]
    mn, mx = np_group_minmax(v)
    r = (mx - mn).astype(np.float32)
    s = (r / np.float32(qmax)).astype(np.float32)
    s = np.where(s > 0, s, np.float32(1.0)).astype(np.float32)
    a = (v - mn[:, None]).astype(np.float32)
    if flags & FLAG_REF_COMPAT:
        inv = (np.float32(1.0) / s).astype(np.float32)
        q = ((a * inv[:, None]).astype(np.float32) + HALF_C).astype(np.float32)
    else:
        q = (a / s[:, None]).astype(np.float32)
    q = q.reshape(ng, group_size // avg, avg)
    total = q[:, :, 0].copy()
    for k in range(1, avg):
        total = (total + q[:, :, k]).astype(np.float32)
    m = (total * np.float32(1.0 / avg)).astype(np.float32)
    if flags & FLAG_REF_COMPAT:
        codes = np.clip(np.trunc(m), 0, qmax).astype(np.uint32)
    else:
        if flags & FLAG_ROUND_NEAREST:
            u = np.full(m.shape, HALF_C, np.float32)
        elif noise is not None:
            u = np.ascontiguousarray(noise, np.float32).reshape(ng, group_size // avg, avg)[:, :, 0]
        else:
            h = np_hash_bytes(seed, offset, 0, v.size).reshape(ng, group_size // avg, avg)[:, :, 0]
            u = h.astype(np.float32) * np.float32(1.0 / 256.0)
        t = (m + u).astype(np.float32)
        codes = np.where(t >= 0, np.minimum(np.floor(t), qmax), 0).astype(np.uint32)
    shifts = (np.arange(vpw, dtype=np.uint32) * np.uint32(bits))
    words = (codes.reshape(ng, -1, vpw) << shifts).sum(axis=2, dtype=np.uint64).astype(np.uint32)
    return words, s, mn.astype(np.float32)


def pack_bits(x: np.ndarray, group_size: int, bits: int) -> np.ndarray:
    x = np.ascontiguousarray(x, np.int8)
    ng = x.size // group_size
    packed = np.empty((ng, group_size * bits // 32), np.uint32)
    if lib().oracle_pack_bits(_ptr(x), ng, group_size, bits, _ptr(packed)):
        raise ValueError("oracle_pack_bits rejected its arguments")
    return packed


def unpack_bits(packed: np.ndarray, group_size: int, bits: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, np.uint32)
    ng = packed.size * 32 // (bits * group_size)
    y = np.empty((ng, group_size), np.int8)
    if lib().oracle_unpack_bits(_ptr(packed), ng, group_size, bits, _ptr(y)):
        raise ValueError("oracle_unpack_bits rejected its arguments")
    return y


def minmax(x: np.ndarray, dtype: str | None = None):
    x = np.ascontiguousarray(x)
    rows, cols = x.shape
    mn = np.empty(rows, np.float32)
    mx = np.empty(rows, np.float32)
    if lib().oracle_minmax(_ptr(x), _dtype_code(x, dtype), rows, cols, _ptr(mn), _ptr(mx)):
        raise ValueError("oracle_minmax rejected its arguments")
    return mn, mx


def calc_precision(b: np.ndarray, C: np.ndarray, w: np.ndarray, target: float) -> np.ndarray:
    b = np.array(b, np.int32)
    C = np.ascontiguousarray(C, np.int32)
    w = np.ascontiguousarray(w, np.int32)
    rc = lib().oracle_calc_precision(_ptr(b), _ptr(C), _ptr(w), b.size, float(target))
    if rc:
        raise ValueError(f"oracle_calc_precision failed ({rc})")
    return b


def fp8_gemm(A8: np.ndarray, B8: np.ndarray, sa: np.ndarray, sb: np.ndarray):
    """A8 [M,K] uint8 (e4m3 bits), B8 [K,N] uint8.  Returns (bf16 bits uint16 [M,N], f32 [M,N])."""
    A8 = np.ascontiguousarray(A8, np.uint8)
    B8 = np.ascontiguousarray(B8, np.uint8)
    sa = np.ascontiguousarray(sa, np.float32)
    sb = np.ascontiguousarray(sb, np.float32)
    M, K = A8.shape
    K2, N = B8.shape
    assert K == K2
    C = np.empty((M, N), np.uint16)
    Cf = np.empty((M, N), np.float32)
    lib().oracle_fp8_gemm(_ptr(A8), _ptr(B8), _ptr(sa), _ptr(sb), _ptr(C), _ptr(Cf), M, N, K, K, N, N)
    return C, Cf


def sgd_noise(keys: np.ndarray) -> np.ndarray:
    """The reference's index hash (cpp_extension/include/quant_common.h:32-43) on uint64 keys."""
    keys = np.ascontiguousarray(keys, np.uint64)
    out = np.empty(keys.shape, np.float32)
    lib().oracle_sgd_noise(_ptr(keys), keys.size, _ptr(out))
    return out


def py_sgd_noise(key: int) -> float:
    """The same hash in Python integers (an independent restatement for known-answer tests)."""
    x = key & 0xFFFFFFFFFFFFFFFF
    x ^= x >> 32
    x = (x * 0xD6E8FEB86659FD93) & 0xFFFFFFFFFFFFFFFF
    x ^= x >> 32
    return float(np.float32(np.float32(x >> 40) * np.float32(1.0 / 16777216.0)) - np.float32(0.5))


def pack_ballot(x: np.ndarray, mn: np.ndarray, mx: np.ndarray, group_size: int, bits: int, seed: int = 0,
                flags: int = 0, dtype: str | None = None):
    """Ballot-plane codec of the reference's cpp extension.  x, mn, mx in one dtype (bf16 as
    uint16 bits).  Returns (packed uint32 [NG * group_size/32 * bits], scale in that dtype)."""
    code = _dtype_code(x, dtype)
    x = np.ascontiguousarray(x)
    mn, mx = np.ascontiguousarray(mn), np.ascontiguousarray(mx)
    ng = x.size // group_size
    packed = np.empty(ng * (group_size // 32) * bits, np.uint32)
    scale = np.empty(ng, mn.dtype)
    rc = lib().oracle_pack_ballot(_ptr(x), code, ng, group_size, bits, _ptr(mn), _ptr(mx), seed & 0xFFFFFFFFFFFFFFFF,
                                  flags, _ptr(packed), _ptr(scale))
    assert rc == 0
    return packed, scale


def unpack_ballot(packed: np.ndarray, scale: np.ndarray, mn: np.ndarray, group_size: int, bits: int,
                  dtype: str | None = None) -> np.ndarray:
    code = _dtype_code(scale, dtype)
    packed = np.ascontiguousarray(packed, np.uint32)
    ng = scale.size
    y = np.empty((ng, group_size), scale.dtype)
    rc = lib().oracle_unpack_ballot(_ptr(packed), _ptr(np.ascontiguousarray(scale)), _ptr(np.ascontiguousarray(mn)),
                                    code, ng, group_size, bits, _ptr(y))
    assert rc == 0
    return y


def e4m3_decode(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, np.uint8)
    out = np.empty(a.shape, np.float32)
    lib().oracle_e4m3_decode(_ptr(a), a.size, _ptr(out))
    return out


def hash_noise(seed: int, offset: int, first: int, count: int) -> np.ndarray:
    out = np.empty(count, np.float32)
    lib().oracle_hash_noise(seed, offset, first, count, _ptr(out))
    return out


def check_div_sequence(a: np.ndarray, s: np.ndarray) -> int:
    a = np.ascontiguousarray(a, np.float32)
    s = np.ascontiguousarray(s, np.float32)
    return int(lib().oracle_check_div_sequence(_ptr(a), _ptr(s), a.size))


# ------------------------------------------------------------ numpy helpers

def bf16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(f: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(f, np.float32).view(np.uint32).astype(np.uint64)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    r = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    r = np.where(nan, (b >> 16) | 0x40, r)
    return r.astype(np.uint16)


def _as_f32(x: np.ndarray, dtype: str | None) -> np.ndarray:
    if dtype == "bf16":
        return bf16_bits_to_f32(x)
    return x.astype(np.float32)


def np_hash_bytes(seed: int, offset: int, first: int, count: int) -> np.ndarray:
    """numpy restatement of the counter hash (act_oracle.c: hash_byte): one noise byte per element."""
    e = np.arange(first, first + count, dtype=np.uint64)
    ctr = e >> np.uint64(3)
    M64 = 0xFFFFFFFFFFFFFFFF

    def splitmix(v):
        z = (v + 0x9E3779B97F4A7C15) & M64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        return z ^ (z >> 31)

    key = splitmix((splitmix(seed & M64) + (offset & M64)) & M64)
    L = (ctr & np.uint64(0xFFFFFFFF))
    R = (ctr >> np.uint64(32)) ^ np.uint64(key >> 32)
    k = key & 0xFFFFFFFF
    for _ in range(4):
        p = np.uint64(0xD256D193) * L
        hi, lo = p >> np.uint64(32), p & np.uint64(0xFFFFFFFF)
        L, R = (hi ^ np.uint64(k) ^ R) & np.uint64(0xFFFFFFFF), lo
        k = (k + 0x9E3779B9) & 0xFFFFFFFF
    w = np.where((e & np.uint64(4)) != 0, R, L)
    return ((w >> (np.uint64(8) * (e & np.uint64(3)))) & np.uint64(0xFF)).astype(np.uint32)


def np_hash_noise(seed: int, offset: int, first: int, count: int) -> np.ndarray:
    """The hash noise as a fraction, h / 256."""
    return np_hash_bytes(seed, offset, first, count).astype(np.float32) * np.float32(1.0 / 256.0)


def np_group_minmax(v: np.ndarray):
    """min/max per row with -0 ordered below +0 (NaN-free input)."""
    mn = v.min(axis=1)
    mx = v.max(axis=1)
    neg0 = ((v == 0) & np.signbit(v)).any(axis=1)
    pos0 = ((v == 0) & ~np.signbit(v)).any(axis=1)
    mn = np.where((mn == 0) & neg0, np.float32(-0.0), mn)
    mn = np.where((mn == 0) & ~neg0, np.float32(0.0), mn)
    mx = np.where((mx == 0) & pos0, np.float32(0.0), mx)
    mx = np.where((mx == 0) & ~pos0, np.float32(-0.0), mx)
    return mn.astype(np.float32), mx.astype(np.float32)


def np_quant_pack(x: np.ndarray, group_size: int, bits: int, noise: np.ndarray | None = None,
                  seed: int = 0, offset: int = 0, flags: int = 0, clamp_alpha: float = 0.0,
                  dtype: str | None = None):
    """Independent numpy restatement of oracle_quant_pack (finite inputs only)."""
    qmax = (1 << bits) - 1
    vpw = 32 // bits
    v = _as_f32(np.ascontiguousarray(x), dtype).reshape(-1, group_size)
    ref = bool(flags & FLAG_REF_COMPAT)
    if ref and flags & FLAG_REF_CLAMP:
        v = np.clip(v, np.float32(-clamp_alpha), np.float32(clamp_alpha))
    if ref and flags & FLAG_REF_TANH:
        v = (np.tanh((v / np.float32(0.5)).astype(np.float32)).astype(np.float32) * np.float32(0.5))
    ng = v.shape[0]
    mn, mx = np_group_minmax(v)
    with np.errstate(all="ignore"):
        r = (mx - mn).astype(np.float32)
        s = (r / np.float32(qmax)).astype(np.float32)
        s = np.where(s > 0, s, np.float32(1.0)).astype(np.float32)
        a = (v - mn[:, None]).astype(np.float32)
        if ref:
            inv = (np.float32(1.0) / s).astype(np.float32)
            t = ((a * inv[:, None]).astype(np.float32) + HALF_C).astype(np.float32)
            codes = np.clip(np.trunc(t), 0, qmax).astype(np.uint32)
        else:
            nearest = bool(flags & FLAG_ROUND_NEAREST)
            hashed = nearest or noise is None                      # the two fixed-point modes
            if nearest:
                u = np.full(v.shape, HALF_C, np.float32)
                h = np.full(v.shape, 127, np.uint32)
            elif noise is not None:
                u = np.ascontiguousarray(noise, np.float32).reshape(v.shape)
            else:
                h = np_hash_bytes(seed, offset, 0, v.size).reshape(v.shape)
                u = h.astype(np.float32) * np.float32(1.0 / 256.0)
            q = (a / s[:, None]).astype(np.float32)
            t = (q + u).astype(np.float32)
            codes = np.where(t >= 0, np.minimum(np.floor(t), qmax), 0).astype(np.uint32)
            if hashed:
                # regular groups: Q = RNE(a * (1/s) * 256) from the exact float64 product,
                # code = (Q + h) >> 8; the others keep the float formula above
                inv = (np.float32(1.0) / s).astype(np.float32)
                z = a.astype(np.float64) * inv[:, None].astype(np.float64) * 256.0
                fl = np.floor(z)
                frac = z - fl
                Q = fl + ((frac > 0.5) | ((frac == 0.5) & (np.mod(fl, 2) == 1)))
                fx = ((Q.astype(np.int64) + h.astype(np.int64)) >> 8).astype(np.uint32)
                regular = (r == 0) | ((r >= np.float32(2.0 ** -50)) & (r <= np.float32(2.0 ** 50)))
                codes = np.where(regular[:, None], fx, codes)
    if bits == 3:
        # bit planes: word p of a 32-element chunk holds bit p of its 32 codes, element l at bit l
        ch = codes.reshape(ng, group_size // 32, 1, 32)
        planes = (ch >> np.arange(3, dtype=np.uint32).reshape(1, 1, 3, 1)) & np.uint32(1)
        words = (planes.astype(np.uint64) << np.arange(32, dtype=np.uint64)).sum(axis=3, dtype=np.uint64)
        packed = words.reshape(ng, group_size * 3 // 32).astype(np.uint32)
    else:
        shifts = (np.arange(vpw, dtype=np.uint32) * np.uint32(bits))
        words = (codes.reshape(ng, group_size // vpw, vpw) << shifts).sum(axis=2, dtype=np.uint64)
        packed = words.astype(np.uint32)
    if flags & FLAG_META_BF16:
        s = bf16_bits_to_f32(f32_to_bf16_bits(s))
        mn = bf16_bits_to_f32(f32_to_bf16_bits(mn))
    return packed, s.astype(np.float32), mn.astype(np.float32)


def np_unpack_codes(packed: np.ndarray, group_size: int, bits: int) -> np.ndarray:
    if bits == 3:
        w = np.ascontiguousarray(packed, np.uint32).reshape(-1, group_size // 32, 3, 1)
        b = (w >> np.arange(32, dtype=np.uint32)) & np.uint32(1)              # [NG, chunks, 3, 32]
        c = b[:, :, 0] | (b[:, :, 1] << np.uint32(1)) | (b[:, :, 2] << np.uint32(2))
        return c.reshape(c.shape[0], group_size)
    vpw = 32 // bits
    packed = np.ascontiguousarray(packed, np.uint32).reshape(-1, group_size // vpw)
    shifts = (np.arange(vpw, dtype=np.uint32) * np.uint32(bits))
    c = (packed[:, :, None] >> shifts) & np.uint32((1 << bits) - 1)
    return c.reshape(packed.shape[0], group_size)


def exact_fma_f32(c: float, s: float, m: float) -> np.float32:
    """fma(c, s, m) rounded once to binary32, through exact rational arithmetic.
    Finite operands only (callers keep non-finite groups out of this path)."""
    exact = Fraction(float(c)) * Fraction(float(s)) + Fraction(float(m))
    # float(Fraction) rounds correctly to binary64; binary32 needs its own rounding
    if exact == 0:
        return np.float32(0.0)
    sign = -1 if exact < 0 else 1
    mag = abs(exact)
    e = mag.numerator.bit_length() - mag.denominator.bit_length()
    if Fraction(2) ** e > mag:
        e -= 1
    e = max(e, -126)
    ulp = Fraction(2) ** (e - 23)
    n = mag / ulp
    fl = n.numerator // n.denominator
    frac = n - fl
    if frac > Fraction(1, 2) or (frac == Fraction(1, 2) and fl % 2 == 1):
        fl += 1
    return np.float32(sign * float(fl * ulp))


def np_dequant(packed: np.ndarray, scale: np.ndarray, mn: np.ndarray, group_size: int,
               bits: int) -> np.ndarray:
    """float64 evaluation of code*scale+min, rounded to float32: equal to the single
    rounding of an FMA except in double-rounding ties (rarer than 1 in 2**28)."""
    c = np_unpack_codes(packed, group_size, bits).astype(np.float64)
    y = c * scale.astype(np.float64)[:, None] + mn.astype(np.float64)[:, None]
    return y.astype(np.float32)
