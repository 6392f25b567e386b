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
        "data": "synthetic", "config": {"workload": workload_name()},
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


def run_extras(dev):
    """Untimed-region extras on rank 0: the fp32 configuration of the codec and the three
    FP8 GEMM shapes.  Each number is the mean of back-to-back launches between two CUDA
    events on the launch stream, buffers rotated so inputs do not sit in L2."""
    import torch
    from deep_optimization_b200 import codec
    from deep_optimization_b200.gemm import fp8_gemm, quantize_e4m3
    peak, _ = load_peaks()
    out = {}
    # fp32 [128,64,56,56], group 256, 2 bits
    shape, gs, bits, rot = (128, 64, 56, 56), 256, 2, 4
    n = 128 * 64 * 56 * 56
    xs = [torch.relu(torch.randn(shape, device=dev)) for _ in range(rot)]
    outs = [(torch.empty((n // gs, gs * bits // 32), dtype=torch.int32, device=dev),
             torch.empty(n // gs, device=dev), torch.empty(n // gs, device=dev)) for _ in range(rot)]
    ys = [torch.empty((n // gs, gs), device=dev) for _ in range(rot)]
    pb, ub = algorithmic_bytes(n, gs, bits, 4)
    tp = _time_launches(lambda i=0: codec.quant_pack(xs[i % rot], bits, gs, seed=3, offset=i, out=outs[i % rot]), 40)
    tu = _time_launches(lambda i=0: codec.dequant_unpack(*outs[i % rot], bits, gs, out_dtype=torch.float32, out=ys[i % rot]), 40)
    out["codec_fp32_128x64x56x56_g256_b2"] = {
        "pack_GBps": pb / tp / 1e6, "pack_frac": pb / tp / 1e6 / peak,
        "unpack_GBps": ub / tu / 1e6, "unpack_frac": ub / tu / 1e6 / peak,
        "pack_plus_unpack_frac": (pb + ub) / (tp + tu) / 1e6 / peak}
    del xs, outs, ys
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
    # the other rounding modes on the bench workload (bf16 [256,256,28,28], group 128, 2 bits):
    # caller-supplied fp32 noise (exact-division float formula; its algorithmic bytes include
    # the 4 bytes of noise read per element) and round-to-nearest
    n = 1
    for d in SHAPE:
        n *= d
    xs = [torch.relu(torch.randn(SHAPE, device=dev)).to(torch.bfloat16) for _ in range(rot)]
    us = [torch.rand(SHAPE, device=dev) for _ in range(2)]
    outs = [(torch.empty((n // GROUP, GROUP * BITS // 32), dtype=torch.int32, device=dev),
             torch.empty(n // GROUP, device=dev), torch.empty(n // GROUP, device=dev)) for _ in range(rot)]
    pb, _ = algorithmic_bytes(n, GROUP, BITS, 2)
    tt = _time_launches(lambda i=0: codec.quant_pack(xs[i % rot], BITS, GROUP, noise=us[i % 2], out=outs[i % rot]), 40)
    tn = _time_launches(lambda i=0: codec.quant_pack(xs[i % rot], BITS, GROUP, flags=1, out=outs[i % rot]), 40)
    out["pack_modes_bf16_g128_b2"] = {
        "noise_tensor": {"GBps_with_noise_bytes": (pb + 4 * n) / tt / 1e6, "frac": (pb + 4 * n) / tt / 1e6 / peak,
                         "ms_per_launch": tt},
        "round_to_nearest": {"GBps": pb / tn / 1e6, "frac": pb / tn / 1e6 / peak, "ms_per_launch": tn}}
    del xs, us, outs
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
        k1 = torch.ones(shp[1], device=dev)
        t_stats = _time_launches(lambda i=0: codec.bn_stats(xb[i % rot], 1e-5, w, b), 40)
        t_fwd = _time_launches(lambda i=0: codec.bn_fwd_norm_quant_pack(xb[i % rot], None, None, w, b, 2, 256,
                                                                         params=params, relu=True), 40)
        t_red = _time_launches(lambda i=0: codec.bn_bwd_reduce(pk, sc, mnn, dyb[i % 2], 2, 256, mask=mask), 40)
        t_dx = _time_launches(lambda i=0: codec.bn_bwd_dx(pk, sc, mnn, dyb[i % 2], k1, k1, k1, 2, 256, mask=mask), 40)
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
    # FP8 GEMM shapes (M, K, N); peak = nominal dense FP8 of a B200
    gem = {}
    bf16_peak = None
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            bf16_peak = float(json.load(f).get("bf16_tflops", 0)) or None
    for (M, K, N) in ((8192, 4096, 4096), (50432, 768, 3072), (50432, 3072, 768)):
        A8, sa = quantize_e4m3(torch.randn(M, K, device=dev), 1)
        B8, sb = quantize_e4m3(torch.randn(K, N, device=dev), 0)
        C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        ws = torch.empty(N * K, dtype=torch.uint8, device=dev)
        t = _time_launches(lambda i=0: fp8_gemm(A8, B8, sa, sb, out=C, workspace=ws), 20)
        Bt = B8.t().contiguous()
        t_nk = _time_launches(lambda i=0: fp8_gemm(A8, Bt, sa, sb, b_is_nk=True, out=C), 20)
        fl = 2.0 * M * N * K
        gem[f"M{M}_K{K}_N{N}"] = {"TFLOPs_B_kn": fl / t / 1e9, "TFLOPs_B_nk": fl / t_nk / 1e9,
                                   "frac_of_nominal_fp8_4500": fl / t_nk / 1e9 / 4500.0}
        if bf16_peak:
            # no FP8 figure is measured on this pool; twice the measured bf16 cuBLAS burst stands in
            gem[f"M{M}_K{K}_N{N}"]["frac_of_2x_measured_bf16"] = fl / t_nk / 1e9 / (2.0 * bf16_peak)
        del A8, B8, C, ws, Bt
    out["fp8_gemm"] = gem
    return out


def run_train(name, dev, world, local, steps=8, warmup=3, act=True, batch=256, channels_last=False):
    """One end-to-end configuration: `name` in (resnet50, vit_b16), ACT 2-bit on every
    supported layer whose activation exceeds 10 MiB, bf16 autocast, batch 256 per GPU of
    synthetic N(0,1) images with uniform labels, DDP (NCCL all-reduce) when world > 1.
    `channels_last` keeps model and images in NHWC memory (cuDNN's native layout for bf16
    convolutions; the fused batch-norm, ReLU and codec kernels then work channel-minor).
    Returns images/s over all ranks (device-timed, max over ranks) and peak memory."""
    import torch
    import torch.distributed as dist
    from torch import nn
    from deep_optimization_b200 import codec
    from deep_optimization_b200.controller import Controller
    from deep_optimization_b200.payload import resnet50, vit_b16
    torch.manual_seed(0)
    model = (resnet50() if name == "resnet50" else vit_b16()).to(dev)
    if act:
        cfg = dict(default_bits=2, auto_precision=None, batch_size=batch)
        net = Controller(model, cfg, input_shape=(3, 224, 224), test=False, device=dev).traced_model
    else:
        net = model.train()
    if channels_last:
        net = net.to(memory_format=torch.channels_last)
    if world > 1:
        net = nn.parallel.DistributedDataParallel(net, device_ids=[local], static_graph=True,
                                                  bucket_cap_mb=25, broadcast_buffers=False)
    if name == "resnet50":
        opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
    else:
        opt = torch.optim.AdamW(net.parameters(), lr=1e-3)
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
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss

    for _ in range(warmup):
        one_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = one_step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    out = {"img_per_s": batch * world / (ms.item() * 1e-3), "ms_per_step": ms.item(),
           "peak_mem_GB": torch.cuda.max_memory_allocated(dev) / 2 ** 30, "final_loss": float(loss.detach())}
    del net, opt, model
    torch.cuda.empty_cache()
    return out


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

    # ---- device-resident timing: K steps between two events on the launch stream ----
    K = args.steps
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_begin.record()
    for i in range(K):
        step(i)
    e_end.record()
    barrier()
    total_ms = e_begin.elapsed_time(e_end)

    # ---- per-kernel durations for the roofline: K launches of one kernel back to back on the
    # rotating buffer sets, between two events on the same stream (an event between every two
    # launches would add the launch gap, about 4 us, to each of them)
    def kernel_loop(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(K):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / K

    pack_ms = kernel_loop(lambda i: codec.quant_pack(xs[i % ROTATE], BITS, GROUP, seed=17,
                                                     offset=i * (n_elems // 4), out=outs[i % ROTATE]))
    unpack_ms = kernel_loop(lambda i: codec.dequant_unpack(*outs[i % ROTATE], BITS, GROUP,
                                                           out_dtype=torch.bfloat16, out=ys[i % ROTATE]))
    if rank == 0:
        # the timed region is short; keep the same load running (untimed) until the
        # sampler has at least half a second of samples under load
        t_end = time.perf_counter() + 0.5
        i = K
        while time.perf_counter() < t_end:
            for _ in range(50):
                step(i)
                i += 1
            torch.cuda.synchronize()
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

    extras = None
    if rank == 0 and not args.no_extras:
        extras = run_extras(dev)
    train = None
    if not args.no_train:
        # every rank takes part: these are the data-parallel end-to-end configurations
        train = {"config": "batch 256 per GPU, bf16 autocast, synthetic images, ACT 2-bit via Controller",
                 "resnet50_act2bit": run_train("resnet50", dev, world, local),
                 "resnet50_no_act": run_train("resnet50", dev, world, local, act=False),
                 "resnet50_act2bit_channels_last": run_train("resnet50", dev, world, local, channels_last=True),
                 "resnet50_no_act_channels_last": run_train("resnet50", dev, world, local, act=False, channels_last=True),
                 "vit_b16_act2bit": run_train("vit_b16", dev, world, local),
                 "vit_b16_no_act": run_train("vit_b16", dev, world, local, act=False)}

    # ---- max over ranks ----------------------------------------------------------
    t = torch.tensor([total_ms, e2e_ms, pack_ms, unpack_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, pack_ms, unpack_ms = t.tolist()

    if rank == 0:
        step_bytes = pack_bytes + unpack_bytes
        value = world * step_bytes * K / (total_ms * 1e-3) / 1e9
        e2e_value = world * step_bytes / (e2e_ms * 1e-3) / 1e9
        peak, peak_kind = load_peaks()
        achieved = pack_bytes / (pack_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / K, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(), "input_dtype": "bf16", "group_size": GROUP,
                       "bits": BITS, "noise": "in-kernel counter hash, 8 noise bits, fixed-point mode",
                       "cache": f"{ROTATE} rotating buffer sets (0.9 GB working set, larger than L2)",
                       "parallelism": f"replicas x{world} (no data-path collective)"},
            "roofline": {"bound": "hbm", "kernel": "quant_pack_kernel<bf16,2,hash>",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"{peak_kind} (copy bandwidth)", "traffic": NCU_PACK_TRAFFIC_BYTES,
                         "algorithmic_bytes_per_launch": pack_bytes, "ms_per_launch": pack_ms,
                         "timing": "mean of K back-to-back launches on rotating buffers, CUDA events on the launch stream",
                         "unpack": {"kernel": "dequant_unpack_kernel<bf16,2>",
                                    "achieved": unpack_bytes / (unpack_ms * 1e-3) / 1e9,
                                    "frac": unpack_bytes / (unpack_ms * 1e-3) / 1e9 / peak,
                                    "ms_per_launch": unpack_ms},
                         "pack_plus_unpack_frac": step_bytes / ((pack_ms + unpack_ms) * 1e-3) / 1e9 / peak},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": n_elems * 2,
                    "d2h_bytes_per_step": n_elems * 2, "ms_per_step": e2e_ms},
            "gpu_launches": 2 * K,        # inside the timed steps; the two kernel loops launch 2K more
            "clocks": clocks,
        }
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the fp32 codec and GEMM side measurements")
    ap.add_argument("--no-train", action="store_true", help="skip the ResNet-50 / ViT-B/16 training steps")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
