"""One rank of the two-GPU check of DOSyncBatchNorm2d (started by test_multirank_gpu.py through
torch.distributed.run): forward, running statistics and gradients against nn.SyncBatchNorm on the
same split batch.  Plain NCCL, in-switch reduction switched off by the caller."""
import os
import sys

import torch
import torch.distributed as dist
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from deep_optimization_b200.modules.normalization.normalization_layers import DOSyncBatchNorm2d
    C, per = 16, 8
    meta = {"b": {"bits": 8, "pack_only": False, "group_size": 256, "act_padding": False, "N": per,
                  "AVG_ALAM": False, "ALAM_BITS": 0, "DIVISION": None}}
    torch.manual_seed(0)                                   # the same full batch on every rank
    full = torch.randn(per * world, C, 12, 12, device=dev) * 2 + 0.5
    gfull = torch.randn(per * world, C, 12, 12, device=dev)
    w0, b0 = torch.rand(C, device=dev) + 0.5, torch.randn(C, device=dev) * 0.1
    ours = DOSyncBatchNorm2d(C, target_name="b", meta=meta).to(dev).train()
    ref = nn.SyncBatchNorm(C).to(dev).train()
    for m in (ours, ref):
        m.weight.data.copy_(w0); m.bias.data.copy_(b0)
    x = full[rank * per:(rank + 1) * per].clone().requires_grad_()
    xr = x.detach().clone().requires_grad_()
    g = gfull[rank * per:(rank + 1) * per]
    y, yr = ours(x), ref(xr)
    y.backward(g); yr.backward(g)
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()
    checks = {
        "y": torch.allclose(y, yr, atol=2e-4, rtol=1e-4),
        "running_mean": torch.allclose(ours.running_mean, ref.running_mean, atol=1e-5),
        "running_var": torch.allclose(ours.running_var, ref.running_var, atol=1e-5, rtol=1e-5),
        "dx": rel(x.grad, xr.grad) < 0.02,                 # x_hat is kept as 8-bit codes
        "dweight": rel(ours.weight.grad, ref.weight.grad) < 0.03,
        "dbias": torch.allclose(ours.bias.grad, ref.bias.grad, atol=1e-3, rtol=1e-4),
    }
    # and against one process normalising the whole batch
    bn = nn.BatchNorm2d(C).to(dev).train()
    bn.weight.data.copy_(w0); bn.bias.data.copy_(b0)
    checks["whole_batch"] = torch.allclose(y, bn(full)[rank * per:(rank + 1) * per], atol=2e-4, rtol=1e-4)
    ok = torch.tensor([1 if all(checks.values()) else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("SYNCBN_OK" if int(ok) == 1 else f"SYNCBN_FAIL rank0 {checks}", flush=True)
    elif not all(checks.values()):
        print(f"SYNCBN_FAIL rank{rank} {checks}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
