"""This library's reference-compatible mode against the reference's own Triton operators run on
the same GPU (baseline/reference_triton.py in a child process: both register `act_lib::`
operators, so they cannot share a process).  Skipped when baseline/_ref has not been installed
(baseline/install_reference.py) or Triton cannot compile for the device.

What can and cannot be exact: Triton compiles `1/scale` and `rng/QMAX` to the approximate
`div.full.f32`, lets the compiler contract `(x-min)*inv + c` into an FMA and uses libdevice's
tanh; this library divides with IEEE rounding, keeps the two roundings apart and uses the CUDA
math library's tanhf.  Each of those differs in the last bit on a few inputs, so a code can fall
on the other side of a rounding boundary.  Asserted: the word layout (every code within one step,
at most 1 % off by one), the group minimum and the stored bf16 scale within one bf16 ulp with at
least 99 % identical, the degenerate-range rule exactly, and the dequantised output of the
reference's own packed tensors within one bf16 ulp.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNNER = os.path.join(ROOT, "baseline", "reference_triton.py")


def _reference_outputs(tmp_path, groups, gs, bits, clamp):
    if not os.path.exists(os.path.join(ROOT, "baseline", "_ref", "act_triton_kernel.py")):
        pytest.skip("baseline/_ref not installed (baseline/install_reference.py)")
    out = str(tmp_path / "ref.npz")
    r = subprocess.run([sys.executable, RUNNER, "dump", "--out", out, "--groups", str(groups), "--group-size", str(gs),
                        "--bits", str(bits), "--clamp", str(clamp)], capture_output=True, text=True, timeout=600)
    last = r.stdout.strip().splitlines()[-1] if r.stdout.strip() else "{}"
    info = json.loads(last) if last.startswith("{") else {}
    if "unavailable" in info or not os.path.exists(out):
        pytest.skip("reference Triton path unavailable on this box: " + info.get("unavailable", r.stderr[-200:]))
    return np.load(out)


def _bf16(bits16):
    return torch.from_numpy(bits16.astype(np.int16)).view(torch.bfloat16)


def _ulp_distance(a16, b16):
    """Distance in bf16 steps between two arrays of bf16 bit patterns of equal sign."""
    return np.abs(a16.astype(np.int32) - b16.astype(np.int32))


@pytest.mark.parametrize("bits,gs,clamp", [(2, 128, 0.0), (4, 256, 0.0), (2, 128, 1.0), (8, 64, 0.0), (1, 128, 0.0)])
def test_ref_compat_against_reference_operators(cuda_device, oracle, tmp_path, bits, gs, clamp):
    from deep_optimization_b200 import _lib, codec
    ng = 4096
    fx = _reference_outputs(tmp_path, ng, gs, bits, clamp)
    x = _bf16(fx["x"]).to(cuda_device).view(ng, gs)
    flags = _lib.ACT_FLAG_REF_COMPAT | _lib.ACT_FLAG_REF_TANH | _lib.ACT_FLAG_META_BF16
    if clamp > 0:
        flags |= _lib.ACT_FLAG_REF_CLAMP
    packed, scale, mn = codec.quant_pack(x, bits, gs, flags=flags, clamp_alpha=clamp)
    got_codes = oracle.np_unpack_codes(packed.cpu().numpy().view(np.uint32), gs, bits).astype(np.int64)
    want_codes = oracle.np_unpack_codes(fx["packed"], gs, bits).astype(np.int64)
    diff = np.abs(got_codes - want_codes)
    frac = float((diff != 0).mean())
    print(f"bits {bits} group {gs} clamp {clamp}: codes differing {frac:.5f}, max step {int(diff.max())}")
    assert diff.max() <= 1 and frac <= 0.01
    # metadata: this library keeps fp32 buffers holding bf16-rounded values
    s16 = scale.to(torch.bfloat16).cpu().view(torch.int16).numpy().view(np.uint16)
    m16 = mn.to(torch.bfloat16).cpu().view(torch.int16).numpy().view(np.uint16)
    assert torch.equal(scale.to(torch.bfloat16).float(), scale) and torch.equal(mn.to(torch.bfloat16).float(), mn)
    ds, dm = _ulp_distance(s16, fx["scale"]), _ulp_distance(m16, fx["min"])
    print(f"  scale identical {float((ds == 0).mean()):.5f}, min identical {float((dm == 0).mean()):.5f}")
    assert ds.max() <= 1 and (ds == 0).mean() >= 0.99
    assert dm.max() <= 1 and (dm == 0).mean() >= 0.99
    assert _bf16(fx["scale"])[0].item() == 1.0 and scale[0].item() == 1.0      # constant group
    # decode the reference's own tensors with this library: q*scale+min, bf16 out
    y = codec.dequant_unpack(torch.from_numpy(fx["packed"].view(np.int32)).to(cuda_device),
                             _bf16(fx["scale"]).float().to(cuda_device), _bf16(fx["min"]).float().to(cuda_device),
                             bits, gs, out_dtype=torch.bfloat16)
    y16 = y.cpu().view(torch.int16).numpy().view(np.uint16).reshape(ng, gs)
    got_y, want_y = _bf16(y16).float().numpy(), _bf16(fx["y"]).float().numpy()
    same = float((y16 == fx["y"]).mean())
    print(f"  dequantised identical {same:.5f}")
    # one bf16 step is at most 2^-7 of the value; near zero, of the group's scale
    step = np.maximum(np.abs(want_y), _bf16(fx["scale"]).float().numpy()[:, None]) * 2.0 ** -7
    assert (np.abs(got_y - want_y) <= step).all() and same >= 0.99
