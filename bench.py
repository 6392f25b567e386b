#!/usr/bin/env python
"""Benchmark of the activation-compression hot path on B200.

One "step" = quantise-and-pack followed by unpack-and-dequantise of one saved
activation (the forward and the backward half of the codec).  Workload: the bf16
conv activation [256,256,28,28] = ReLU(N(0,1)), group 128, 2-bit codes, in-kernel
stochastic rounding.  The tensors are synthetic and seeded; they stand in for
ImageNet activations, which are not available offline.

`python bench.py --gpus N --steps K --warmup W` prints ONE JSON line (rank 0).
With N > 1 (torchrun) every rank runs the same per-GPU workload on its own data:
the codec needs no exchange between GPUs, so ranks are independent replicas and
the value is the sum over ranks (weak scaling).

`--impl reference` times the CPU restatement of the reference codec (oracle/) on
the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPE = (256, 256, 28, 28)
GROUP = 128
BITS = 2
ROTATE = 4                      # distinct buffer sets cycled through: working set >> 126 MB L2
REGIONS = 25                    # timed regions of K steps each; the median region is reported
METRIC = "act_quant_pack_unpack_GBps"
UNIT = "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the pack kernel on this
# workload, from the ncu capture summarised under profiles/.
NCU_PACK_TRAFFIC_BYTES = 109_140_000      # profiles/quant_pack_bf16_g128_b2_ncu.md (mean of 2 launches)


def algorithmic_bytes(n_elems: int, group: int, bits: int, elem_bytes: int):
    """(pack, unpack) bytes: E*(s + b/8) + 8*NG each way."""
    ng = n_elems // group
    one = n_elems * elem_bytes + n_elems * bits // 8 + 8 * ng
    return one, one


def workload_name():
    return (f"bf16 conv activation {list(SHAPE)} ReLU(N(0,1)), group {GROUP}, {BITS}-bit, "
            f"quant-pack + dequant-unpack")


def config_dict(world: int):
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": workload_name(), "input_dtype": "bf16", "group_size": GROUP, "bits": BITS,
            "noise": "in-kernel counter hash, 8 noise bits, fixed-point mode",
            "cache": f"{ROTATE} rotating buffer sets (0.9 GB working set, larger than L2)",
            "parallelism": f"replicas x{world} (no data-path collective)"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            f = [p.strip() for p in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons),
                "note": "sampled every 20 ms over the timed region and an identical untimed continuation"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def make_inputs(seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.relu(torch.randn(SHAPE, generator=g, dtype=torch.float32)).to(torch.bfloat16)


def cpu_baseline(x_host, threads: int, reps: int = 3, fraction: int = 4):
    """Times the CPU oracle on the first 1/fraction of the workload's groups."""
    import numpy as np
    import torch
    from oracle import act_oracle as oracle
    oracle.set_threads(threads)
    arr = x_host.view(-1, GROUP)
    n_groups = arr.shape[0] // fraction
    arr = arr[:n_groups].contiguous().view(torch.int16).numpy().view(np.uint16)
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        p, s, m = oracle.quant_pack(arr, GROUP, BITS, dtype="bf16", seed=1, offset=0)
        oracle.dequant_unpack(p, s, m, GROUP, BITS, out="bf16")
        best = min(best, time.perf_counter() - t0)
    pb, ub = algorithmic_bytes(arr.size, GROUP, BITS, 2)
    return (pb + ub) / best / 1e9, f"first 1/{fraction} of the workload's groups ({n_groups} groups), best of {reps}"


def run_reference(args):
    """Reference arm: the CPU restatement of the reference codec on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle import act_oracle as oracle
    threads = os.cpu_count() or 1
    x = make_inputs(0)
    # warm-up builds/loads the oracle and touches the pages
    cpu_baseline(x, threads, reps=max(1, args.warmup), fraction=16)
    fraction = 4
    vals = []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        v, sample = cpu_baseline(x, threads, reps=1, fraction=fraction)
        vals.append(v)
    dt = time.perf_counter() - t0
    value = sum(vals) / len(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config_dict(int(os.environ.get("WORLD_SIZE", "1"))),
        "baseline_kind": "CPU port of the reference codec (oracle/), not the reference's GPU path",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"each step: {sample}"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _time_launches(fn, reps):
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def _median_launch_ms(fn, reps=20, regions=7):
    """Median over `regions` of the mean of `reps` back-to-back launches (CUDA events)."""
    import torch
    for i in range(3):
        fn(i)
    vals = []
    for r in range(regions):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            fn(r * reps + i)
        e1.record()
        torch.cuda.synchronize()
        vals.append(e0.elapsed_time(e1) / reps)
    vals.sort()
    return vals[len(vals) // 2]


def run_contract_modes(dev):
    """The arithmetic the evaluation configuration states word for word (fp32 min and scale, true
    division, code = clamp(floor((x-min)/scale + u)) with a caller-supplied fp32 noise tensor u)
    beside the in-kernel hash mode the headline uses, on configuration 1 (fp32 [128,64,56,56],
    group 256, 2 bits) and on the headline workload.  The noise tensor adds 4 bytes of reads per
    element; fractions are given with those bytes counted (what the kernel moves) and without
    (the codec's own algorithmic bytes)."""
    import torch
    from deep_optimization_b200 import codec
    peak, _ = load_peaks()
    out = {}
    rot = 3
    for name, shape, gs, dtype, sbytes in (("config1_fp32_128x64x56x56_g256_b2", (128, 64, 56, 56), 256, torch.float32, 4),
                                           ("headline_bf16_256x256x28x28_g128_b2", SHAPE, GROUP, torch.bfloat16, 2)):
        n = 1
        for d in shape:
            n *= d
        ng = n // gs
        xs = [torch.relu(torch.randn(shape, device=dev)).to(dtype) for _ in range(rot)]
        us = [torch.rand(shape, device=dev) for _ in range(2)]
        outs = [(torch.empty((ng, gs * BITS // 32), dtype=torch.int32, device=dev),
                 torch.empty(ng, device=dev), torch.empty(ng, device=dev)) for _ in range(rot)]
        ys = [torch.empty((ng, gs), dtype=dtype, device=dev) for _ in range(rot)]
        pb, ub = algorithmic_bytes(n, gs, BITS, sbytes)
        t_noise = _median_launch_ms(lambda i: codec.quant_pack(xs[i % rot], BITS, gs, noise=us[i % 2], out=outs[i % rot]))
        t_hash = _median_launch_ms(lambda i: codec.quant_pack(xs[i % rot], BITS, gs, seed=3, offset=i, out=outs[i % rot]))
        t_un = _median_launch_ms(lambda i: codec.dequant_unpack(*outs[i % rot], BITS, gs, out_dtype=dtype, out=ys[i % rot]))
        fr = lambda b, t: b / t / 1e6 / peak
        out[name] = {
            "pack_noise_tensor": {"ms_per_launch": t_noise, "frac_with_noise_bytes": fr(pb + 4 * n, t_noise),
                                  "frac_codec_bytes_only": fr(pb, t_noise)},
            "pack_hash": {"ms_per_launch": t_hash, "frac": fr(pb, t_hash)},
            "unpack": {"ms_per_launch": t_un, "frac": fr(ub, t_un)},
            "pack_plus_unpack_frac_noise_tensor": fr(pb + 4 * n + ub, t_noise + t_un),
            "pack_plus_unpack_frac_hash": fr(pb + ub, t_hash + t_un)}
        del xs, us, outs, ys
    torch.cuda.empty_cache()
    return out


def run_extras(dev):
    """Untimed-region extras on rank 0: the fp32 configuration of the codec and the three
    FP8 GEMM shapes.  Each number is the mean of back-to-back launches between two CUDA
    events on the launch stream, buffers rotated so inputs do not sit in L2."""
    import torch
    from deep_optimization_b200 import codec
    from deep_optimization_b200.gemm import fp8_gemm, quantize_e4m3
    peak, _ = load_peaks()
    out = {}
    rot = 4
    # bit-width and shape sweep of the bf16 configuration: conv [256,256,28,28] = ReLU(N(0,1)) and
    # ViT [256,197,768] = GELU(N(0,1)), group 128, bits 1/2/4/8
    sweep = {}
    for name, shp, fn in (("conv_256x256x28x28", SHAPE, torch.relu),
                          ("vit_256x197x768", (256, 197, 768), torch.nn.functional.gelu)):
        n = 1
        for d in shp:
            n *= d
        xs = [fn(torch.randn(shp, device=dev)).to(torch.bfloat16) for _ in range(rot)]
        ys = [torch.empty((n // GROUP, GROUP), dtype=torch.bfloat16, device=dev) for _ in range(rot)]
        for b in (1, 2, 4, 8):
            outs = [(torch.empty((n // GROUP, GROUP * b // 32), dtype=torch.int32, device=dev),
                     torch.empty(n // GROUP, device=dev), torch.empty(n // GROUP, device=dev)) for _ in range(rot)]
            pb, ub = algorithmic_bytes(n, GROUP, b, 2)
            tp = _time_launches(lambda i=0: codec.quant_pack(xs[i % rot], b, GROUP, seed=3, offset=i, out=outs[i % rot]), 40)
            tu = _time_launches(lambda i=0: codec.dequant_unpack(*outs[i % rot], b, GROUP, out_dtype=torch.bfloat16, out=ys[i % rot]), 40)
            sweep[f"{name}_b{b}"] = {"pack_frac": pb / tp / 1e6 / peak, "unpack_frac": ub / tu / 1e6 / peak,
                                     "pack_us": tp * 1e3, "unpack_us": tu * 1e3}
            del outs
        del xs, ys
    out["codec_bf16_g128_sweep"] = sweep
    # fused batch-norm kernels on a ResNet-50 stage-1 activation, bf16 [256,64,56,56], group 256,
    # 2 bits: algorithmic bytes = what each kernel must read and write once
    shp = (256, 64, 56, 56)
    n = shp[0] * shp[1] * shp[2] * shp[3]
    for tag, fmt in (("", torch.contiguous_format), ("_channels_last", torch.channels_last)):
        xb = [torch.randn(shp, device=dev).to(torch.bfloat16).contiguous(memory_format=fmt) for _ in range(rot)]
        dyb = [torch.randn(shp, device=dev).to(torch.bfloat16).contiguous(memory_format=fmt) for _ in range(2)]
        w = torch.ones(shp[1], device=dev)
        b = torch.zeros(shp[1], device=dev)
        params = codec.bn_stats(xb[0], 1e-5, w, b)
        _, pk, sc, mnn, mask = codec.bn_fwd_norm_quant_pack(xb[0], None, None, w, b, 2, 256, params=params, relu=True)
        # the constants of dx as bn_bwd_coef's [C][4] table (built once: the wrapper would otherwise
        # stack three vectors into it on every call, which is host time, not the kernel's)
        coef = torch.ones((shp[1], 4), device=dev)
        t_stats = _time_launches(lambda i=0: codec.bn_stats(xb[i % rot], 1e-5, w, b), 40)
        t_fwd = _time_launches(lambda i=0: codec.bn_fwd_norm_quant_pack(xb[i % rot], None, None, w, b, 2, 256,
                                                                         params=params, relu=True), 40)
        t_red = _time_launches(lambda i=0: codec.bn_bwd_reduce(pk, sc, mnn, dyb[i % 2], 2, 256, mask=mask), 40)
        t_dx = _time_launches(lambda i=0: codec.bn_bwd_dx(pk, sc, mnn, dyb[i % 2], None, None, None, 2, 256, mask=mask, coef=coef), 40)
        meta_b = 8 * (n // 256)
        by = {"stats": 2 * n, "norm_relu_quant_pack": 2 * n + 2 * n + n // 4 + n // 8 + meta_b,
              "bwd_reduce": 2 * n + n // 4 + n // 8 + meta_b, "bwd_dx": 2 * n + n // 4 + n // 8 + meta_b + 2 * n}
        out["bn_relu_fused_bf16_256x64x56x56_g256_b2" + tag] = {
            k: {"GBps": by[k] / t / 1e6, "frac": by[k] / t / 1e6 / peak, "ms_per_launch": t}
            for k, t in (("stats", t_stats), ("norm_relu_quant_pack", t_fwd), ("bwd_reduce", t_red), ("bwd_dx", t_dx))}
        del xb, dyb, pk, sc, mnn, mask
    # fused activation kernels on the ViT MLP activation, bf16 [256,197,3072], group 128, 2 bits:
    # forward writes y and the packed derivative, backward multiplies dy by the decoded derivative;
    # ReLU on the conv activation keeps one mask bit per element (wrapper time included)
    shp = (256, 197, 3072)
    n = shp[0] * shp[1] * shp[2]
    xa = [torch.randn(shp, device=dev).to(torch.bfloat16) for _ in range(2)]
    _, pk, sc, mnn = codec.activation_fwd_quant_pack(xa[0], "gelu", BITS, GROUP)
    t_gf = _time_launches(lambda i=0: codec.activation_fwd_quant_pack(xa[i % 2], "gelu", BITS, GROUP), 20)
    t_gb = _time_launches(lambda i=0: codec.mul_dequant_unpack(pk, sc, mnn, xa[i % 2], BITS, GROUP), 20)
    b_gf = 2 * n + 2 * n + n * BITS // 8 + 8 * (n // GROUP)
    fused = {"gelu_fwd_quant_pack": {"GBps": b_gf / t_gf / 1e6, "frac": b_gf / t_gf / 1e6 / peak, "ms_per_launch": t_gf},
             "gelu_bwd_dequant_mul": {"GBps": b_gf / t_gb / 1e6, "frac": b_gf / t_gb / 1e6 / peak, "ms_per_launch": t_gb}}
    del xa, pk, sc, mnn
    n = 1
    for d in SHAPE:
        n *= d
    xr = [torch.randn(SHAPE, device=dev).to(torch.bfloat16) for _ in range(rot)]
    _, mbits = codec.relu_fwd_pack(xr[0])
    t_rf = _time_launches(lambda i=0: codec.relu_fwd_pack(xr[i % rot]), 40)
    t_rb = _time_launches(lambda i=0: codec.relu_bwd_unpack(mbits, xr[i % rot]), 40)
    b_r = 2 * n + 2 * n + n // 8
    fused["relu_fwd_mask_pack"] = {"GBps": b_r / t_rf / 1e6, "frac": b_r / t_rf / 1e6 / peak, "ms_per_launch": t_rf}
    fused["relu_bwd_mask_unpack"] = {"GBps": b_r / t_rb / 1e6, "frac": b_r / t_rb / 1e6 / peak, "ms_per_launch": t_rb}
    out["fused_activation_kernels_bf16"] = fused
    del xr, mbits
    out["fp8_gemm"] = run_gemm_shapes(dev)
    out["dw_from_packed"] = run_dw_shapes(dev)
    out["write_stream"] = run_write_stream(dev)
    out["reference_triton"] = run_reference_triton()
    return out


GEMM_SHAPES = ((8192, 4096, 4096), (50432, 768, 3072), (50432, 3072, 768))      # (M, K, N)


def run_gemm_shapes(dev, shapes=GEMM_SHAPES, reps=20):
    """The FP8 GEMM on the evaluation shapes, B in both layouts, beside cuBLASLt's scaled matmul
    on the same operands.  Before a time is reported the kernel's abort word must be clear and 64
    sampled rows of C must match the float64 product.  Fractions: of the nominal dense FP8 peak
    of a B200 (4.5 PFLOP/s) and of twice the measured bf16 cuBLAS burst (no FP8 figure is
    measured on this pool)."""
    import torch
    from deep_optimization_b200.gemm import fp8_gemm, gemm_status, quantize_e4m3
    bf16_peak = None
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            bf16_peak = float(json.load(f).get("bf16_tflops", 0)) or None
    gem = {}
    for (M, K, N) in shapes:
        A8, sa = quantize_e4m3(torch.randn(M, K, device=dev), 1)
        B8, sb = quantize_e4m3(torch.randn(K, N, device=dev), 0)
        Bt = B8.t().contiguous()
        C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        ws = torch.empty(N * K, dtype=torch.uint8, device=dev)
        rows = torch.linspace(0, M - 1, 64, device=dev).long()
        ref = (A8[rows].double() @ B8.double()) * sa[rows].double()[:, None] * sb.double()[None, :]
        entry = {}
        for tag, fn in (("B_nk", lambda i=0: fp8_gemm(A8, Bt, sa, sb, b_is_nk=True, out=C)),
                        ("B_kn", lambda i=0: fp8_gemm(A8, B8, sa, sb, out=C, workspace=ws))):
            C.fill_(float("nan"))
            fn()
            status = gemm_status()
            got = C[rows].double()
            tol = ref.abs() * 2.0 ** -8 + ref.abs().max() * 2.0 ** -12 + 1e-6
            if status != 0 or torch.isnan(C).any() or not bool(((got - ref).abs() <= tol).all()):
                raise SystemExit(f"fp8_gemm {tag} M={M} K={K} N={N}: wrong result (abort word {status})")
            t = _median_launch_ms(fn, reps=reps, regions=5)
            if gemm_status() != 0:
                raise SystemExit(f"fp8_gemm {tag} M={M} K={K} N={N}: aborted inside the timing loop")
            entry["TFLOPs_" + tag] = 2.0 * M * N * K / t / 1e9
            entry["ms_" + tag] = t
        entry["checked"] = "abort word 0; 64 sampled rows within 2^-8 |ref| + 2^-12 max|ref| of the float64 product"
        entry["frac_of_nominal_fp8_4500"] = entry["TFLOPs_B_nk"] / 4500.0
        entry["frac_of_nominal_fp8_4500_B_kn"] = entry["TFLOPs_B_kn"] / 4500.0
        if bf16_peak:
            entry["frac_of_2x_measured_bf16"] = entry["TFLOPs_B_nk"] / (2.0 * bf16_peak)
        try:
            sa2, sb2 = sa.view(M, 1).contiguous(), sb.view(1, N).contiguous()
            t2 = _median_launch_ms(lambda i=0: torch._scaled_mm(A8, Bt.t(), scale_a=sa2, scale_b=sb2,
                                                                out_dtype=torch.bfloat16), reps=reps, regions=5)
            entry["cublaslt_scaled_mm_TFLOPs"] = 2.0 * M * N * K / t2 / 1e9
            entry["vs_cublaslt"] = t2 / entry["ms_B_nk"]
        except Exception as ex:        # noqa: BLE001 - a library yardstick only
            entry["cublaslt_scaled_mm_TFLOPs"] = f"unavailable: {str(ex)[:80]}"
        gem[f"M{M}_K{K}_N{N}"] = entry
        del A8, B8, C, ws, Bt, ref
    torch.cuda.empty_cache()
    return gem


def run_dw_shapes(dev, shapes=((50432, 3072, 768), (50432, 768, 3072)), reps=10):
    """The weight gradient of a linear layer from its 2-bit packed input (group 128), decoded
    inside the GEMM, beside the unfused sequence it replaces: dequant_unpack to bf16, then
    cuBLAS dy^T @ x.  (M, N, K) are the two MLP layers of ViT-B/16 at batch 256.  Checked first:
    abort word clear and the result within 2^-10 of the float64 product on 64 sampled rows."""
    import torch
    from deep_optimization_b200 import codec
    from deep_optimization_b200.gemm import dw_from_packed, dw_status
    out = {}
    for (M, N, K) in shapes:
        x = torch.nn.functional.gelu(torch.randn(M, K, device=dev)).to(torch.bfloat16)
        dy = (torch.randn(M, N, device=dev) * 0.1).to(torch.bfloat16)
        packed, scale, mn = codec.quant_pack(x, BITS, GROUP, seed=3, offset=1)
        xq = torch.empty((M, K), dtype=torch.bfloat16, device=dev)
        dw = torch.empty((N, K), dtype=torch.float32, device=dev)
        dw_from_packed(dy, packed, scale, mn, BITS, GROUP, K, out=dw)
        status = dw_status()
        codec.dequant_unpack(packed, scale, mn, BITS, GROUP, out_dtype=torch.bfloat16, out=xq.view(-1, GROUP))
        rows = torch.linspace(0, N - 1, 64, device=dev).long()
        ref = dy[:, rows].double().t() @ xq.double()
        tol = ref.abs() * 2.0 ** -10 + ref.abs().max() * 2.0 ** -13 + 1e-6
        if status != 0 or not bool(((dw[rows].double() - ref).abs() <= tol).all()):
            raise SystemExit(f"dw_from_packed M={M} N={N} K={K}: wrong result (abort word {status})")
        del ref
        t_fused = _median_launch_ms(lambda i=0: dw_from_packed(dy, packed, scale, mn, BITS, GROUP, K, out=dw), reps=reps, regions=5)

        def unfused(i=0):
            codec.dequant_unpack(packed, scale, mn, BITS, GROUP, out_dtype=torch.bfloat16, out=xq.view(-1, GROUP))
            return dy.t().mm(xq)
        t_unfused = _median_launch_ms(unfused, reps=reps, regions=5)
        t_mm = _median_launch_ms(lambda i=0: dy.t().mm(xq), reps=reps, regions=5)
        fl = 2.0 * M * N * K
        out[f"M{M}_N{N}_K{K}"] = {"fused_ms": t_fused, "fused_TFLOPs": fl / t_fused / 1e9,
                                   "dequant_plus_cublas_ms": t_unfused, "cublas_mm_alone_ms": t_mm,
                                   "speedup_vs_unfused": t_unfused / t_fused,
                                   "checked": "abort word 0; 64 sampled rows within 2^-10 |ref| + 2^-13 max|ref|"}
        del x, dy, packed, scale, mn, xq, dw
    torch.cuda.empty_cache()
    return out


def run_write_stream(dev):
    """What a pure write stream reaches on this GPU: the runtime's memset (through the library's
    act_fill_zero) on outputs of the size the unpack kernel (102.8 MB) and the K = 768 GEMM
    (309.9 MB) write, rotating buffers; torch's fill kernel beside it (it is much slower and was
    once mistaken here for the pace of the memory system)."""
    import torch
    from deep_optimization_b200 import _lib
    lib = _lib.load()
    peak, _ = load_peaks()
    out = {}
    st = torch.cuda.current_stream(dev).cuda_stream
    for name, nbytes in (("unpack_output_102.8MB", 102_760_448), ("gemm_output_309.9MB", 309_854_208)):
        bufs = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(4)]
        t = _median_launch_ms(lambda i: lib.act_fill_zero(bufs[i % 4].data_ptr(), nbytes, st))
        t_torch = _median_launch_ms(lambda i: bufs[i % 4].zero_())
        out[name] = {"ms": t, "GBps": nbytes / t / 1e6, "frac_of_copy_peak": nbytes / t / 1e6 / peak,
                     "torch_fill_ms": t_torch, "torch_fill_GBps": nbytes / t_torch / 1e6}
        del bufs
    torch.cuda.empty_cache()
    return out


def run_reference_triton(steps=20, warmup=3):
    """The reference's own Triton operators on this GPU, in a child process (they register the
    same operator names as this package): baseline/reference_triton.py, which needs the
    reference's two Triton modules under baseline/_ref (baseline/install_reference.py)."""
    runner = os.path.join(ROOT, "baseline", "reference_triton.py")
    if not os.path.exists(os.path.join(ROOT, "baseline", "_ref", "act_triton_kernel.py")):
        return {"unavailable": "reference Triton path unavailable on this box: baseline/_ref not installed"}
    try:
        r = subprocess.run([sys.executable, runner, "time", "--steps", str(steps), "--warmup", str(warmup)],
                           capture_output=True, text=True, timeout=900)
    except subprocess.TimeoutExpired:
        return {"unavailable": "reference Triton path unavailable on this box: timed out after 900 s"}
    lines = [ln for ln in r.stdout.strip().splitlines() if ln.startswith("{")]
    if not lines:
        return {"unavailable": "reference Triton path unavailable on this box: " + (r.stderr.strip().splitlines() or ["no output"])[-1][:200]}
    res = json.loads(lines[-1])
    if "unavailable" in res:
        res["unavailable"] = "reference Triton path unavailable on this box: " + res["unavailable"]
    return res


DDP_BUCKET_MB = 25
FUSED_DW = True         # Linear weight gradients straight from the packed input (--no-fused-dw: dequantise + cuBLAS)
STALL_RATIO = 2.0       # a training-leg region whose slowest step exceeds this multiple of its median is timed once more
FUSE_ADD_LN = True      # x + branch formed inside the following LayerNorm's kernels (--no-fuse-add-ln: separate additions)
DP_MODE = "flat"         # how the training legs average gradients over ranks; see run_train


class FlatGradientAllReduce:
    """Data-parallel gradient averaging with one NCCL all-reduce per step: every gradient is copied
    into one flat fp32 buffer by a multi-tensor copy, the buffer is all-reduced (average) and
    copied back the same way.  The views into the buffer carry each parameter's own strides, so a
    channels-last weight gradient is copied as it lies.  Against DistributedDataParallel this
    trades the overlap of communication with backward for two things that matter more on a step
    of 28 ms that the host thread barely keeps ahead of: no per-parameter hook, copy and scale
    launches on the backward path (322 small launches per ResNet-50 step), and no collective
    holding SM slots while the codec's one-wave kernels run."""

    def __init__(self, params, world):
        import torch
        self.params = [p for p in params if p.requires_grad]
        self.world = world
        n = sum(p.numel() for p in self.params)
        self.flat = torch.zeros(n, dtype=torch.float32, device=self.params[0].device)
        self.views = None

    def _make_views(self, grads):
        # Each view has exactly the strides of the gradient it mirrors (a dense gradient is
        # contiguous in some dimension order, as a channels-last weight gradient is; the order of
        # size-1 dimensions differs between a 1x1 convolution's weight and its gradient): only
        # then do the two multi-tensor copies run as one kernel each instead of one per tensor.
        import torch
        views, off = [], 0
        for g in grads:
            dense = g.is_contiguous() or (g.dim() == 4 and g.is_contiguous(memory_format=torch.channels_last))
            views.append(self.flat.as_strided(g.size(), g.stride(), off) if dense
                         else self.flat[off:off + g.numel()].view(g.shape))
            off += g.numel()
        return views

    def __call__(self):
        import torch
        import torch.distributed as dist
        grads = [p.grad for p in self.params]
        if self.views is None or any(v.stride() != g.stride() for v, g in zip(self.views, grads)):
            self.views = self._make_views(grads)
        torch._foreach_copy_(self.views, grads)
        dist.all_reduce(self.flat)
        self.flat.mul_(1.0 / self.world)
        torch._foreach_copy_(grads, self.views)


def run_train(name, dev, world, local, steps=20, warmup=12, act=True, batch=256, channels_last=False,
              profiler=None):
    """One end-to-end configuration: `name` in (resnet50, vit_b16), ACT 2-bit on every
    supported layer whose activation exceeds 10 MiB, bf16 autocast, batch 256 per GPU of
    synthetic N(0,1) images with uniform labels, DDP (NCCL all-reduce) when world > 1.
    `channels_last` keeps model and images in NHWC memory (cuDNN's native layout for bf16
    convolutions; the fused batch-norm, ReLU and codec kernels then work channel-minor).
    Returns images/s over all ranks (device-timed, max over ranks) and peak memory.  Twelve warm-up
    steps (lazy initialisation in the libraries underneath still shows up as single steps of 30-430 ms
    among a process's first ten), then twenty timed steps."""
    import torch
    import torch.distributed as dist
    from torch import nn
    from deep_optimization_b200 import codec
    from deep_optimization_b200.controller import Controller
    from deep_optimization_b200.payload import resnet50, vit_b16
    # what earlier legs left behind (their traced modules sit in reference cycles, and with them
    # their device memory) is collected and handed back before this leg allocates anything
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    torch.manual_seed(0)
    model = (resnet50() if name == "resnet50" else vit_b16()).to(dev)
    if act:
        cfg = dict(default_bits=2, auto_precision=None, batch_size=batch, fused_dw=FUSED_DW,
                   fuse_add_layer_norm=FUSE_ADD_LN)
        net = Controller(model, cfg, input_shape=(3, 224, 224), test=False, device=dev).traced_model
    else:
        net = model.train()
    if channels_last:
        net = net.to(memory_format=torch.channels_last)
    reduce_grads = None
    if world > 1 and DP_MODE == "flat":
        reduce_grads = FlatGradientAllReduce(net.parameters(), world)
    elif world > 1:
        net = nn.parallel.DistributedDataParallel(net, device_ids=[local], static_graph=True,
                                                  bucket_cap_mb=DDP_BUCKET_MB, broadcast_buffers=False,
                                                  gradient_as_bucket_view=(DP_MODE == "ddp-view"))
    if name == "resnet50":
        opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9, fused=True)
    else:
        # PyTorch's one-kernel AdamW, as the reference's own training cells construct it
        # (Activation_Compression/test8.ipynb:399); the default implementation makes seven passes
        opt = torch.optim.AdamW(net.parameters(), lr=1e-3, fused=True)
    g = torch.Generator(device=dev).manual_seed(1234 + local)
    x = torch.randn((batch, 3, 224, 224), device=dev, generator=g).to(torch.bfloat16)
    y = torch.randint(0, 1000, (batch,), device=dev, generator=g)
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    codec.manual_seed(99)
    torch.cuda.reset_peak_memory_stats(dev)

    def one_step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = nn.functional.cross_entropy(net(x), y)
        opt.zero_grad(set_to_none=(DP_MODE != "ddp-view"))
        loss.backward()
        if reduce_grads is not None:
            reduce_grads()
        opt.step()
        return loss

    for _ in range(warmup):
        one_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    import contextlib
    # The interpreter's cyclic garbage collector is held off during the timed steps (collected
    # before, re-enabled after), as a training loop that cares about step-time jitter does: one
    # collection in a 20-step region otherwise shows up as a 40-70 ms step.  An event after every
    # step gives the median and the slowest step beside the mean.
    import gc
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]

    def timed_region():
        gc.collect()
        gc.disable()
        try:
            with (profiler if profiler is not None else contextlib.nullcontext()):
                e0.record()
                for i in range(steps):
                    last = one_step()
                    marks[i].record()
                e1.record()
                torch.cuda.synchronize()
        finally:
            gc.enable()
        return last, [(marks[i - 1] if i else e0).elapsed_time(marks[i]) for i in range(steps)]

    loss, in_order = timed_region()
    per_step = sorted(in_order)
    # A region with a stalled step is timed once more, and says so: now and then one early step of a
    # region takes 0.2-0.4 s (seen at the second timed step of a leg, in about one leg in ten, on any
    # model; its cause is not known), which would stand for a third of a 20-step mean.
    stall = torch.tensor([1.0 if per_step[-1] > STALL_RATIO * per_step[steps // 2] else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(stall, op=dist.ReduceOp.MAX)
    discarded = None
    if stall.item() > 0 and profiler is None:
        discarded = {"ms_each_step": [round(v, 1) for v in in_order],
                     "reason": "a step of %.0f ms against a median of %.1f ms: region timed again" % (per_step[-1], per_step[steps // 2])}
        loss, in_order = timed_region()
        per_step = sorted(in_order)
    ms = torch.tensor([e0.elapsed_time(e1) / steps, per_step[steps // 2], per_step[-1]], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    out = {"img_per_s": batch * world / (ms[0].item() * 1e-3), "ms_per_step": ms[0].item(),
           "ms_per_step_median": ms[1].item(), "ms_per_step_max": ms[2].item(),
           "img_per_s_median_step": batch * world / (ms[1].item() * 1e-3),
           "ms_each_step": [round(v, 1) for v in in_order],
           "peak_mem_GB": torch.cuda.max_memory_allocated(dev) / 2 ** 30, "final_loss": float(loss.detach())}
    if discarded is not None:
        out["discarded_region"] = discarded
    if reduce_grads is not None:
        # what the step pays for the gradient exchange: the all-reduce of the flat buffer alone,
        # and the whole exchange with its two multi-tensor copies, each timed over 5 repetitions
        def timed(fn):
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(5):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / 5
        out["gradient_bytes"] = reduce_grads.flat.numel() * 4
        out["allreduce_ms"] = timed(lambda: dist.all_reduce(reduce_grads.flat))
        out["gradient_exchange_ms"] = timed(reduce_grads)
    del net, opt, model
    torch.cuda.empty_cache()
    return out


def _bind_to_gpu_cpus(local):
    """Multi-rank runs: keep this rank's threads on the CPUs NVML lists as local to its GPU, before
    any pinned buffer is allocated, so that the e2e leg's host buffers are first touched on the
    GPU's own memory node (eight ranks that all allocate on one socket share that socket's memory
    and the inter-socket link: 8 GB/s per rank and direction instead of tens).  Reads NVML only;
    returns the CPU count it bound to, or None when NVML or the call is unavailable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        index = int(vis.split(",")[local]) if vis and all(v.strip().isdigit() for v in vis.split(",")) else local
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:       # noqa: BLE001 - an optimisation of the host side only
        return None


def run_ours(args):
    import torch
    import torch.distributed as dist
    from deep_optimization_b200 import _lib, codec

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the codec has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = _bind_to_gpu_cpus(local) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    n_elems = 1
    for d in SHAPE:
        n_elems *= d
    pack_bytes, unpack_bytes = algorithmic_bytes(n_elems, GROUP, BITS, 2)

    # ROTATE distinct inputs (different seeds per rank), resident in HBM before timing
    host = [make_inputs(1000 * rank + i) for i in range(ROTATE)]
    xs = [h.to(dev) for h in host]
    ng = n_elems // GROUP
    # outputs are preallocated per buffer set: the timed region launches kernels only
    outs = [(torch.empty((ng, GROUP * BITS // 32), dtype=torch.int32, device=dev),
             torch.empty((ng,), dtype=torch.float32, device=dev),
             torch.empty((ng,), dtype=torch.float32, device=dev)) for _ in range(ROTATE)]
    ys = [torch.empty((ng, GROUP), dtype=torch.bfloat16, device=dev) for _ in range(ROTATE)]

    def step(i):
        k = i % ROTATE
        codec.quant_pack(xs[k], BITS, GROUP, seed=17, offset=i * (n_elems // 4), out=outs[k])
        codec.dequant_unpack(*outs[k], BITS, GROUP, out_dtype=torch.bfloat16, out=ys[k])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()

    # ---- device-resident timing ---------------------------------------------------
    # REGIONS timed regions of K steps each, every one bracketed by barrier + synchronize and
    # two CUDA events on the launch stream; per region the max over ranks, then the median
    # over regions is the value (a single region of K = 20 steps lasts about a millisecond,
    # and one such sample moved by +-5 % from box to box and run to run).
    K = args.steps
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # the same load, untimed, while the sampler starts: the GPU must not idle (and drop its
    # clocks) right before the timed regions
    t_end = time.perf_counter() + 0.3
    i = 0
    while time.perf_counter() < t_end:
        for _ in range(50):
            step(i)
            i += 1
        torch.cuda.synchronize()

    def regions_of(fn, regions, sync_ranks):
        out = []
        for r in range(regions):
            if sync_ranks:
                barrier()
            else:
                torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(K):
                fn(r * K + i)
            b.record()
            if sync_ranks:
                barrier()
            else:
                torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return out

    region_ms = regions_of(step, REGIONS, True)

    # ---- per-kernel durations for the roofline: K launches of one kernel back to back on the
    # rotating buffer sets between two events on the same stream (an event between every two
    # launches would add the launch gap, about 4 us, to each of them), REGIONS times over
    pack_region_ms = regions_of(lambda i: codec.quant_pack(xs[i % ROTATE], BITS, GROUP, seed=17,
                                                           offset=i * (n_elems // 4), out=outs[i % ROTATE]),
                                REGIONS, False)
    unpack_region_ms = regions_of(lambda i: codec.dequant_unpack(*outs[i % ROTATE], BITS, GROUP,
                                                                 out_dtype=torch.bfloat16, out=ys[i % ROTATE]),
                                  REGIONS, False)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: pinned host input -> H2D -> pack -> unpack -> D2H ----------
    # Three streams, double-buffered, so the copy in of step i+1 and the copy out of step
    # i-1 overlap the kernels of step i (PCIe is full duplex); every step still moves its
    # own input from pinned host memory and its own result back inside the timed region.
    pin_in = [h.pin_memory() for h in host[:2]]
    pin_out = [torch.empty((ng, GROUP), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    dbuf = [torch.empty_like(xs[0]) for _ in range(2)]
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]        # kernels of the step using buffer k finished
    ev_out = [torch.cuda.Event() for _ in range(2)]         # result of buffer k is back on the host

    def e2e_run(n_steps):
        for i in range(n_steps):
            k = i % 2
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_done[k])                  # dbuf[k] no longer read by step i-2
                dbuf[k].copy_(pin_in[k], non_blocking=True)
                ev_in[k].record(s_in)
            main.wait_event(ev_in[k])
            main.wait_event(ev_out[k])                       # ys[k] of step i-2 already copied out
            codec.quant_pack(dbuf[k], BITS, GROUP, seed=17, offset=i, out=outs[k])
            codec.dequant_unpack(*outs[k], BITS, GROUP, out_dtype=torch.bfloat16, out=ys[k])
            ev_done[k].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[k])
                pin_out[k].copy_(ys[k], non_blocking=True)
                ev_out[k].record(s_out)
        main.wait_event(ev_out[0])
        main.wait_event(ev_out[1])

    e2e_run(4)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    KE = max(4, min(K, 40))
    e0.record()
    e2e_run(KE)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / KE

    contract = run_contract_modes(dev) if rank == 0 else None
    extras = None
    if rank == 0 and not args.no_extras:
        extras = run_extras(dev)
    train = None
    if not args.no_train:
        # every rank takes part: these are the data-parallel end-to-end configurations
        legs = {"resnet50_act2bit": dict(name="resnet50"),
                "resnet50_no_act": dict(name="resnet50", act=False),
                "resnet50_act2bit_channels_last": dict(name="resnet50", channels_last=True),
                "resnet50_no_act_channels_last": dict(name="resnet50", act=False, channels_last=True),
                "vit_b16_act2bit": dict(name="vit_b16"),
                "vit_b16_no_act": dict(name="vit_b16", act=False)}
        train = {"config": "batch 256 per GPU, bf16 autocast, synthetic images, ACT 2-bit via Controller; "
                           + ("one rank" if world == 1 else
                              {"flat": "gradients averaged by one NCCL all-reduce of a flat buffer per step",
                               "ddp": f"DistributedDataParallel, {DDP_BUCKET_MB} MB buckets",
                               "ddp-view": f"DistributedDataParallel, {DDP_BUCKET_MB} MB buckets, gradients as bucket views"}[DP_MODE])}
        for leg, kw in legs.items():
            if args.legs is None or leg in args.legs:
                train[leg] = run_train(kw.pop("name"), dev, world, local, **kw)

    # ---- max over ranks (per region), then the median over regions -------------------
    t = torch.tensor([region_ms, pack_region_ms, unpack_region_ms, [e2e_ms] * REGIONS], device=dev,
                     dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    region_ms, pack_region_ms, unpack_region_ms = (sorted(v) for v in t[:3].tolist())
    e2e_ms = float(t[3][0])
    med = lambda v: v[len(v) // 2]
    total_ms, pack_ms, unpack_ms = med(region_ms), med(pack_region_ms) / K, med(unpack_region_ms) / K

    if rank == 0:
        step_bytes = pack_bytes + unpack_bytes
        gbps = lambda ms: world * step_bytes * K / (ms * 1e-3) / 1e9
        value = gbps(total_ms)
        e2e_value = world * step_bytes / (e2e_ms * 1e-3) / 1e9
        peak, peak_kind = load_peaks()
        achieved = pack_bytes / (pack_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / K, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(world),
            "regions": {"count": REGIONS, "steps_each": K, "value": "median region",
                        "value_min": gbps(region_ms[-1]), "value_max": gbps(region_ms[0]),
                        "spread": (region_ms[-1] - region_ms[0]) / total_ms,
                        "frac_of_hbm_peak": value / world / peak},
            "roofline": {"bound": "hbm", "kernel": "quant_pack_kernel<bf16,2,hash>",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"{peak_kind} (copy bandwidth)", "traffic": NCU_PACK_TRAFFIC_BYTES,
                         "traffic_source": "one ncu capture of this kernel on this workload (profiles/quant_pack_bf16_g128_b2_ncu.md)",
                         "algorithmic_bytes_per_launch": pack_bytes, "ms_per_launch": pack_ms,
                         "ms_per_launch_min_max": [pack_region_ms[0] / K, pack_region_ms[-1] / K],
                         "timing": f"median of {REGIONS} regions of K back-to-back launches on rotating buffers, "
                                   "CUDA events on the launch stream",
                         "unpack": {"kernel": "dequant_unpack_kernel<bf16,2>",
                                    "achieved": unpack_bytes / (unpack_ms * 1e-3) / 1e9,
                                    "frac": unpack_bytes / (unpack_ms * 1e-3) / 1e9 / peak,
                                    "ms_per_launch": unpack_ms,
                                    "ms_per_launch_min_max": [unpack_region_ms[0] / K, unpack_region_ms[-1] / K]},
                         "pack_plus_unpack_frac": step_bytes / ((pack_ms + unpack_ms) * 1e-3) / 1e9 / peak},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": n_elems * 2,
                    "d2h_bytes_per_step": n_elems * 2, "ms_per_step": e2e_ms,
                    "per_rank_h2d_GBps": n_elems * 2 / (e2e_ms * 1e-3) / 1e9,
                    "per_rank_d2h_GBps": n_elems * 2 / (e2e_ms * 1e-3) / 1e9,
                    "cpus_bound_to_gpu": numa,
                    "bound": "host memory and PCIe: the two copies of a step run concurrently with the kernels"},
            "gpu_launches": 2 * K,        # per timed region of K steps; there are REGIONS of them
            "clocks": clocks,
        }
        if contract is not None:
            line["roofline"]["contract_modes"] = contract
        if extras is not None:
            line["other_configs"] = extras
        if train is not None:
            line["train"] = train
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            v, sample = cpu_baseline(host[0], cores)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_only(args):
    """Small single-purpose runs for profilers (`--only`): a handful of launches of one part of
    the benchmark, so that a capture of them ends by itself.

    --only gemm --shape M K N [--reps R]          the FP8 GEMM on one shape (checked, then timed)
    --only dw --shape M N K [--reps R]            the weight gradient from the packed input on one shape
    --only bn --shape N C H W [--channels-last]   the five kernels of one fused BatchNorm+ReLU layer
    --only ln --shape R C [--reps R]              LayerNorm fused with the codec, forward and backward
    --only train-profile --model resnet50|vit_b16 [--channels-last] [--no-act] [--rows R]
                                                  two training steps under torch.profiler; under
                                                  torchrun every rank runs them (DDP), rank 0 prints
    """
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.only == "gemm":
        shapes = (tuple(args.shape),) if args.shape else GEMM_SHAPES      # M K N; default: all evaluation shapes
        print(json.dumps(run_gemm_shapes(dev, shapes, reps=args.reps)), flush=True)
    elif args.only == "dw":
        M, N, K = args.shape
        print(json.dumps(run_dw_shapes(dev, ((M, N, K),), reps=args.reps)), flush=True)
    elif args.only == "bn":
        from deep_optimization_b200 import codec
        N, C, H, W = args.shape
        fmt = torch.channels_last if args.channels_last else torch.contiguous_format
        mk = lambda: torch.randn((N, C, H, W), device=dev).to(torch.bfloat16).contiguous(memory_format=fmt)
        w, b = torch.ones(C, device=dev), torch.zeros(C, device=dev)
        for _ in range(args.reps):
            x, dy = mk(), mk()
            params = codec.bn_stats(x, 1e-5, w, b)
            y, packed, scale, mn, mask = codec.bn_fwd_norm_quant_pack(x, None, None, w, b, BITS, 256,
                                                                      params=params, relu=True)
            s1, s2 = codec.bn_bwd_reduce(packed, scale, mn, dy, BITS, 256, mask=mask)
            coef = codec.bn_bwd_coef(s1._base, params, N * H * W)
            codec.bn_bwd_dx(packed, scale, mn, dy, None, None, None, BITS, 256, mask=mask, coef=coef)
        torch.cuda.synchronize()
        print("ok", flush=True)
    elif args.only == "ln":
        from deep_optimization_b200 import codec
        R, C = args.shape
        x = [torch.randn(R, C, device=dev).to(torch.bfloat16) for _ in range(3)]
        w, b = torch.ones(C, device=dev), torch.zeros(C, device=dev)
        for i in range(args.reps):
            if args.residual:       # the pair with the residual addition in front of the LayerNorm
                _, y, mean, rstd, packed, scale, mn = codec.ln_fwd_quant_pack(x[i % 3], w, b, 1e-6, BITS, GROUP,
                                                                              residual=x[(i + 2) % 3])
                codec.ln_bwd_from_packed(x[(i + 1) % 3], packed, scale, mn, BITS, GROUP, mean, rstd, w, dy2=x[i % 3])
                continue
            y, mean, rstd, packed, scale, mn = codec.ln_fwd_quant_pack(x[i % 3], w, b, 1e-6, BITS, GROUP)
            codec.ln_bwd_from_packed(x[(i + 1) % 3], packed, scale, mn, BITS, GROUP, mean, rstd, w)
        torch.cuda.synchronize()
        print("ok", flush=True)
    elif args.only == "train-profile":
        import torch.distributed as dist
        from torch.profiler import ProfilerActivity, profile
        if world > 1:
            dist.init_process_group("nccl", device_id=dev)
        prof = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA])
        res = run_train(args.model, dev, world, local, steps=2, warmup=3, act=not args.no_act,
                        channels_last=args.channels_last, profiler=prof)
        if rank == 0:
            print(json.dumps(res))
            print(prof.key_averages().table(sort_by="self_cuda_time_total", row_limit=args.rows,
                                            max_name_column_width=70), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the fp32 codec and GEMM side measurements")
    ap.add_argument("--no-train", action="store_true", help="skip the ResNet-50 / ViT-B/16 training steps")
    ap.add_argument("--only", choices=("codec", "gemm", "dw", "bn", "ln", "train-profile"),
                    help="codec: the headline alone; the others: small runs for profilers (see run_only)")
    ap.add_argument("--shape", type=int, nargs="+", help="--only gemm: M K N; --only bn: N C H W")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--model", default="resnet50", choices=("resnet50", "vit_b16"))
    ap.add_argument("--channels-last", action="store_true")
    ap.add_argument("--no-act", action="store_true")
    ap.add_argument("--rows", type=int, default=45)
    ap.add_argument("--ddp-bucket-mb", type=int, default=None, help="gradient bucket size of the DDP training legs")
    ap.add_argument("--dp-mode", choices=("flat", "ddp", "ddp-view"), default=None,
                    help="gradient averaging of the training legs: one flat all-reduce per step (default), "
                         "DistributedDataParallel, or DDP with gradients as bucket views")
    ap.add_argument("--no-fused-dw", action="store_true",
                    help="training legs: Linear layers dequantise and call cuBLAS for dW instead of act_dw_from_packed")
    ap.add_argument("--residual", action="store_true",
                    help="--only ln: the kernels that take the residual addition / the second gradient")
    ap.add_argument("--stall-ratio", type=float, default=None,
                    help="training legs: re-time a region whose slowest step exceeds this multiple of the median (default 2)")
    ap.add_argument("--no-fuse-add-ln", action="store_true",
                    help="training legs: residual additions in front of a LayerNorm stay separate kernels")
    ap.add_argument("--legs", nargs="+", default=None, help="training legs to run (default: all six)")
    args = ap.parse_args()
    global DDP_BUCKET_MB, DP_MODE, FUSED_DW, FUSE_ADD_LN, STALL_RATIO
    if args.stall_ratio:
        STALL_RATIO = args.stall_ratio
    FUSED_DW = not args.no_fused_dw
    FUSE_ADD_LN = not args.no_fuse_add_ln
    if args.ddp_bucket_mb:
        DDP_BUCKET_MB = args.ddp_bucket_mb
    if args.dp_mode:
        DP_MODE = args.dp_mode
    if args.only == "codec":
        args.no_extras = args.no_train = True
    elif args.only:
        return run_only(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
