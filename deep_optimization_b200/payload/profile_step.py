"""Kernel-level breakdown of one training step of a payload model:
`python -m deep_optimization_b200.payload.profile_step {resnet50|vit_b16} [--channels-last]
[--no-act] [--batch 256] [--rows 45]`.

Builds the model as `bench.py`'s training leg does (Controller with 2-bit ACT, bf16 autocast,
synthetic images), warms up, then runs two steps under `torch.profiler` and prints the
operators and kernels sorted by device time.  A profiling aid: nothing imports it.
"""
from __future__ import annotations

import argparse

import torch
from torch import nn
from torch.profiler import ProfilerActivity, profile

from ..controller import Controller
from . import resnet50, vit_b16


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("model", choices=("resnet50", "vit_b16"))
    ap.add_argument("--channels-last", action="store_true")
    ap.add_argument("--no-act", action="store_true")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--rows", type=int, default=45)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    model = (resnet50() if args.model == "resnet50" else vit_b16()).to(dev)
    if args.no_act:
        net = model.train()
    else:
        cfg = dict(default_bits=2, auto_precision=None, batch_size=args.batch)
        net = Controller(model, cfg, input_shape=(3, 224, 224), test=False, device=dev).traced_model
    x = torch.randn((args.batch, 3, 224, 224), device=dev).to(torch.bfloat16)
    y = torch.randint(0, 1000, (args.batch,), device=dev)
    if args.channels_last:
        net = net.to(memory_format=torch.channels_last)
        x = x.contiguous(memory_format=torch.channels_last)
    if args.model == "resnet50":
        opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
    else:
        opt = torch.optim.AdamW(net.parameters(), lr=1e-3)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = nn.functional.cross_entropy(net(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            step()
        torch.cuda.synchronize()
    print(prof.key_averages().table(sort_by="self_cuda_time_total", row_limit=args.rows,
                                    max_name_column_width=70))


if __name__ == "__main__":
    main()
