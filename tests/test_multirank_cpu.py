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


# ---------------------------------------------------------------- SyncBN Function across two ranks
def _oracle_ops():
    """The two codec operators the quantise boundary calls, backed by the CPU oracle instead of the
    CUDA library (8-bit codes, noise from the counter hash), so that the cross-rank algebra of
    _DOSyncBatchNorm can run on gloo ranks without a GPU.  Test scaffolding only."""
    import numpy as np
    from oracle import act_oracle as oracle

    def quant_pack(x, bits, group_size, avg_alam, alam_bits, clamp, clamp_alpha):
        N, G, gs = x.shape
        p, s, m = oracle.quant_pack(x.detach().float().contiguous().numpy().reshape(-1, gs), gs, bits, seed=3, offset=0)
        return (torch.from_numpy(p.view(np.int32)), torch.from_numpy(s).view(N, G), torch.from_numpy(m).view(N, G))

    def dequant_unpack(packed, scale, xmin, bits, group_size, avg_alam, alam_bits):
        N, G = scale.shape
        y = oracle.dequant_unpack(packed.numpy().view(np.uint32), scale.reshape(-1).numpy(), xmin.reshape(-1).numpy(),
                                  group_size, bits, out="f32")
        return torch.from_numpy(y).view(N, G, group_size)

    return {"quant_pack_triton": quant_pack, "dequant_unpack_triton": dequant_unpack}


def _syncbn_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from deep_optimization_b200 import act_kernels, codec
        from deep_optimization_b200.modules.normalization.normalization_ops import _DOSyncBatchNorm
        act_kernels.IMPL.update(_oracle_ops())
        g = torch.Generator().manual_seed(0)
        C = 6
        full = torch.randn(12, C, 8, 8, generator=g) * 2 + 0.5            # the global batch
        gy = torch.randn(12, C, 8, 8, generator=g)
        w0 = torch.rand(C, generator=g) + 0.5
        b0 = torch.randn(C, generator=g)
        sl = slice(0, 4) if rank == 0 else slice(4, 12)                   # uneven split: 4 and 8 samples
        x = full[sl].clone().requires_grad_()
        w, b = w0.clone().requires_grad_(), b0.clone().requires_grad_()
        rm, rv = torch.zeros(C), torch.ones(C)
        meta = {"t": {"bits": 8, "pack_only": False, "group_size": 128, "act_padding": False, "N": x.shape[0],
                      "AVG_ALAM": False, "ALAM_BITS": 0, "DIVISION": None}}
        y = _DOSyncBatchNorm.apply(x, w, b, rm, rv, 1e-5, 0.1, None, world, "t", meta, None)
        y.backward(gy[sl])
        # the same on the whole batch in one process
        ref = torch.nn.BatchNorm2d(C, eps=1e-5, momentum=0.1)
        with torch.no_grad():
            ref.weight.copy_(w0); ref.bias.copy_(b0)
        xr = full.clone().requires_grad_()
        yr = ref.train()(xr)
        yr.backward(gy)
        rel = lambda a, c: ((a - c).norm() / c.norm()).item()
        ok = torch.allclose(y, yr[sl], atol=1e-4)
        ok = ok and torch.allclose(rm, ref.running_mean, atol=1e-5) and torch.allclose(rv, ref.running_var, atol=1e-4)
        ok = ok and rel(x.grad, xr.grad[sl]) < 0.02                        # x_hat went through 8-bit codes
        # weight / bias gradients are per-rank sums (DDP averages them afterwards): their sum is the global one
        gw, gb = w.grad.clone(), b.grad.clone()
        dist.all_reduce(gw); dist.all_reduce(gb)
        ok = ok and rel(gw, ref.weight.grad) < 0.02 and torch.allclose(gb, ref.bias.grad, atol=1e-3)
        # the default hash seed differs between ranks once a process group exists, rank 0 keeps the plain seed
        codec.manual_seed(1234)
        seeds = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(seeds, torch.tensor([codec._stream_seed() & 0x7FFFFFFFFFFFFFFF]))
        ok = ok and int(seeds[0]) == 1234 and int(seeds[1]) != 1234
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sync_batch_norm_function_two_ranks_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_syncbn_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert ret.get(0) is True and ret.get(1) is True


# ---------------------------------------------------------------- the bench's gradient averaging
def _flat_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import bench
        torch.manual_seed(0)
        net = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3), torch.nn.Conv2d(8, 4, 1), torch.nn.Flatten(),
                                  torch.nn.Linear(4 * 6 * 6, 5)).to(memory_format=torch.channels_last)
        reduce = bench.FlatGradientAllReduce(net.parameters(), world)
        x = torch.randn(4, 3, 8, 8, generator=torch.Generator().manual_seed(10 + rank))
        net(x).square().sum().backward()
        mine = [p.grad.clone() for p in net.parameters()]
        reduce()
        ok = True
        for p, g in zip(net.parameters(), mine):
            both = [torch.zeros_like(g) for _ in range(world)]
            dist.all_gather(both, g.contiguous())
            ok = ok and torch.allclose(p.grad, sum(both) / world, atol=1e-6) and p.grad.stride() == g.stride()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_flat_gradient_all_reduce_two_ranks_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 33500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_flat_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert ret.get(0) is True and ret.get(1) is True
