"""CPU checks of the boundary: the shared library loads, exports every symbol the
header declares, and rejects bad arguments without touching a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from deep_optimization_b200 import _lib, build
    build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "act_b200.h")).read()
    return sorted(set(re.findall(r"ACT_API\s+[\w\s\*]+?\b(act_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert "act_quant_pack" in names and "act_dequant_unpack" in names
    for n in names:
        assert hasattr(lib, n), n


def test_python_signature_table_covers_header():
    from deep_optimization_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_argument_errors_need_no_gpu(lib):
    from deep_optimization_b200 import _lib
    bad = ctypes.c_void_p(16)
    qp = lib.act_quant_pack
    assert qp(bad, 7, 1, 128, 2, None, 0, 0, 0, 0.0, bad, bad, bad, None) == 1      # dtype
    assert qp(bad, 0, 1, 128, 5, None, 0, 0, 0, 0.0, bad, bad, bad, None) == 2      # bits
    assert qp(bad, 0, 1, 96, 2, None, 0, 0, 0, 0.0, bad, bad, bad, None) == 3       # group
    assert qp(bad, 0, -1, 128, 2, None, 0, 0, 0, 0.0, bad, bad, bad, None) == 5     # size
    assert qp(None, 0, 1, 128, 2, None, 0, 0, 0, 0.0, bad, bad, bad, None) == 6     # null
    assert qp(ctypes.c_void_p(24), 0, 1, 128, 2, None, 0, 0, 0, 0.0, bad, bad, bad, None) == 4  # align
    assert qp(bad, 0, 0, 128, 2, None, 0, 0, 0, 0.0, bad, bad, bad, None) == 0      # empty input
    assert lib.act_dequant_unpack(bad, bad, bad, 0, 128, 2, 1, bad, None) == 0
    assert lib.act_dequant_unpack(bad, bad, bad, 1, 128, 5, 1, bad, None) == 2
    assert b"bits" in lib.act_strerror(2)
    with pytest.raises(_lib.ActLibraryError):
        _lib.check(3, "x")


def test_calc_precision_matches_oracle(lib, oracle):
    import numpy as np
    import torch
    from deep_optimization_b200 import codec
    rng = np.random.default_rng(0)
    for _ in range(20):
        n = int(rng.integers(1, 40))
        b = rng.integers(2, 9, n).astype(np.int32)
        C = rng.integers(1, 10000, n).astype(np.int32)
        w = np.ones(n, np.int32)
        target = float(b.sum() * rng.uniform(0.4, 0.9))
        want = oracle.calc_precision(b, C, w, target)
        got = codec.calc_precision(torch.from_numpy(b.copy()), torch.from_numpy(C), torch.from_numpy(w), target)
        assert got.tolist() == want.tolist()


def test_cpu_tensors_are_refused():
    import torch
    from deep_optimization_b200 import codec
    with pytest.raises(RuntimeError):
        codec.quant_pack(torch.zeros(4, 128), 2, 128)
    with pytest.raises(ValueError):
        codec._bits_consts(3, 128)
