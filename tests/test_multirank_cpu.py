"""world_size-2 gloo tests (CPU) of the host logic that runs with more than one rank:
the SyncBN statistics exchange and the max-over-ranks / sum-over-ranks bookkeeping the
bench uses for replicas."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from deep_optimization_b200.modules.normalization.normalization_ops import sync_batch_stats
        g = torch.Generator().manual_seed(0)
        full = torch.randn(12, 5, 6, 6, generator=g) * 3 + 1          # the global batch
        part = full[:4] if rank == 0 else full[4:]                    # uneven split: 4 and 8 samples
        dims = [0, 2, 3]
        var, mean = torch.var_mean(part, dim=dims, unbiased=False)
        count = part.numel() // part.shape[1]
        m, v, total = sync_batch_stats(mean, var, count, None, world)
        vr, mr = torch.var_mean(full, dim=dims, unbiased=False)
        ok = torch.allclose(m, mr, atol=1e-5) and torch.allclose(v, vr, atol=1e-4) and int(total) == 12 * 36
        # replica bookkeeping: time = max over ranks, units = sum over ranks
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        units = torch.tensor([100.0], dtype=torch.float64)
        dist.all_reduce(units, op=dist.ReduceOp.SUM)
        ok = ok and t.item() == float(world) and units.item() == 100.0 * world
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret.get(0) is True and ret.get(1) is True
