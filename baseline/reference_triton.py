"""Runs the reference's own Triton operators, unmodified, on the current CUDA device.

The reference registers its operators under the same `act_lib::` names as this package, so the
two cannot live in one process: the benchmark and the parity test start this file as a child
process.  It needs `baseline/_ref/` (see baseline/install_reference.py) and a GPU Triton can
compile for; every failure is reported as {"unavailable": "<one line>"} with exit code 0.

    python baseline/reference_triton.py time  [--steps K] [--warmup W]
        -> one JSON line: device time of torch.ops.act_lib.quant_pack_triton /
           dequant_unpack_triton on the benchmark's workloads and of Triton_Linear on the
           three GEMM shapes (CUDA events on the launch stream, rotating inputs)
    python baseline/reference_triton.py dump --out FILE.npz [--groups 4096] [--group-size 128]
                                             [--bits 2] [--seed 0] [--clamp ALPHA]
        -> the operators' outputs on a seeded activation, for the parity test
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _import_reference():
    if not os.path.exists(os.path.join(REF, "act_triton_kernel.py")):
        raise RuntimeError("baseline/_ref is empty: run baseline/install_reference.py first")
    sys.path.insert(0, REF)
    import act_triton_kernel  # noqa: F401  (registers torch.ops.act_lib.*)
    import linear
    return act_triton_kernel, linear


def _time(fn, steps, warmup):
    import torch
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps          # ms


def cmd_time(args):
    import torch
    import triton
    import triton.language as tl
    ref, linear = _import_reference()
    dev = torch.device("cuda")
    out = {"triton": triton.__version__, "device": torch.cuda.get_device_name(0)}
    rot = 3
    # the two codec workloads: bf16 conv activation [256,256,28,28] group 128 (the headline) and
    # fp32 [128,64,56,56] group 256; the operators take [N, G, group] and return bf16 scale/min
    for name, shape, gs, dtype, sbytes in (("conv_bf16_256x256x28x28_g128_b2", (256, 256, 28, 28), 128, torch.bfloat16, 2),
                                           ("fp32_128x64x56x56_g256_b2", (128, 64, 56, 56), 256, torch.float32, 4)):
        n = 1
        for d in shape:
            n *= d
        N = shape[0]
        xs = [torch.relu(torch.randn(shape, device=dev)).to(dtype).view(N, n // N // gs, gs) for _ in range(rot)]
        res = [None] * rot

        def pack(i):
            res[i % rot] = torch.ops.act_lib.quant_pack_triton(xs[i % rot], 2, gs, False, 0, False, 0.0)

        def unpack(i):
            p, s, m = res[i % rot]
            torch.ops.act_lib.dequant_unpack_triton(p, s, m, 2, gs, False, 0)

        tp = _time(pack, args.steps, args.warmup)
        tu = _time(unpack, args.steps, args.warmup)
        ng = n // gs
        pb = n * sbytes + n // 4 + 8 * ng            # same algorithmic-byte formula as the benchmark
        ub = n * 2 + n // 4 + 8 * ng                 # the reference always writes bf16
        out[name] = {"pack_ms": tp, "unpack_ms": tu, "pack_GBps": pb / tp / 1e6, "unpack_GBps": ub / tu / 1e6,
                     "pack_plus_unpack_GBps": (pb + ub) / (tp + tu) / 1e6,
                     "note": "includes the operator's own allocations and its x.contiguous() view"}
        del xs, res
        torch.cuda.empty_cache()
    # Triton_Linear on e4m3 operands, bf16 output, its own autotuner choosing the tile shape
    gem = {}
    for (M, K, N) in ((8192, 4096, 4096), (50432, 768, 3072), (50432, 3072, 768)):
        A = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
        B = torch.randn(K, N, device=dev).to(torch.float8_e4m3fn)
        C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        grid = lambda meta: (triton.cdiv(M, meta["BLOCK_SIZE_M"]) * triton.cdiv(N, meta["BLOCK_SIZE_N"]),)

        def run(i):
            linear.Triton_Linear[grid](A, B, C, M, N, K, A.stride(0), A.stride(1), B.stride(0), B.stride(1),
                                       C.stride(0), C.stride(1), OUT_DTYPE=tl.bfloat16)
        try:
            t = _time(run, max(3, args.steps // 4), 2)
            gem[f"M{M}_K{K}_N{N}"] = {"ms": t, "TFLOPs": 2.0 * M * N * K / t / 1e9,
                                      "config": str(getattr(linear.Triton_Linear, "best_config", ""))[:120]}
        except Exception as ex:                      # noqa: BLE001 - reported, not hidden
            gem[f"M{M}_K{K}_N{N}"] = {"unavailable": f"{type(ex).__name__}: {str(ex)[:160]}"}
        del A, B, C
    out["triton_linear_fp8"] = gem
    print(json.dumps(out), flush=True)


def cmd_dump(args):
    import numpy as np
    import torch
    ref, _ = _import_reference()
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(args.seed)
    gs, bits, ng = args.group_size, args.bits, args.groups
    x = torch.relu(torch.randn(ng * gs, generator=g)).to(torch.bfloat16)
    x[:gs] = 0.25                                   # one constant group: the degenerate-range rule
    xd = x.to(dev).view(ng // 16, 16, gs)
    clamp = args.clamp > 0
    packed, scale, mn = torch.ops.act_lib.quant_pack_triton(xd, bits, gs, False, 0, clamp, float(args.clamp))
    y = torch.ops.act_lib.dequant_unpack_triton(packed, scale, mn, bits, gs, False, 0)
    torch.cuda.synchronize()
    b16 = lambda t: t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
    np.savez(args.out, x=b16(x), packed=packed.cpu().numpy().view(np.uint32), scale=b16(scale.reshape(-1)),
             min=b16(mn.reshape(-1)), y=b16(y.reshape(ng, gs)))
    print(json.dumps({"ok": True, "groups": ng}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("cmd", choices=("time", "dump"))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out")
    ap.add_argument("--groups", type=int, default=4096)
    ap.add_argument("--group-size", type=int, default=128)
    ap.add_argument("--bits", type=int, default=2)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--clamp", type=float, default=0.0)
    args = ap.parse_args()
    try:
        (cmd_time if args.cmd == "time" else cmd_dump)(args)
    except Exception as ex:                          # noqa: BLE001 - the caller records the reason
        print(json.dumps({"unavailable": f"{type(ex).__name__}: {str(ex).splitlines()[0][:200] if str(ex) else ''}"}), flush=True)


if __name__ == "__main__":
    main()
