"""Batch sharding + the single all-reduce of the label-context gradient, with two gloo ranks on
CPU.  The per-rank layer is stood in for by the CPU oracle (the CUDA layer needs a GPU); what is
tested is the host logic: slices cover the batch exactly once and the reduced gradient equals the
full-batch gradient."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mplayers_b200 import parallel


def test_shard_bounds_cover_the_batch_exactly_once():
    for n in (1, 2, 7, 16, 33):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = parallel.shard_bounds(n, r, world)
                assert 0 <= lo <= hi <= n
                seen += list(range(lo, hi))
            assert seen == list(range(n))
    with pytest.raises(ValueError):
        parallel.shard_bounds(4, 2, 2)
    t = torch.arange(10).view(5, 2)
    assert torch.equal(parallel.shard_batch(t, 1, 2), t[3:5])


def _inputs():
    rng = np.random.default_rng(5)
    B, H, W, L, D, I = 4, 9, 11, 7, 4, 2
    unary = rng.standard_normal((B, 1, H, W, L)).astype(np.float32)
    a = np.triu(rng.uniform(0, 2, (L, L)), 1)
    ctx = (a + a.T).astype(np.float32)
    ew = rng.uniform(0.2, 1, (D, B, 1, H, W)).astype(np.float32)
    g = rng.uniform(0, 1, (B, 1, H, W, L)).astype(np.float32)
    return unary, ctx, ew, g, D, I


def _rank_main(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle
    unary, ctx, ew, g, D, I = _inputs()
    lo, hi = parallel.shard_bounds(unary.shape[0], rank, world)
    fw = oracle.forward("TRWP", unary[lo:hi], ctx, ew[:, lo:hi], D, I, n_threads=1)
    bw = oracle.backward("TRWP", ctx, ew[:, lo:hi], g[lo:hi], fw["min_idx"], fw["norm_idx"], n_threads=1)
    param = torch.nn.Parameter(torch.from_numpy(ctx.copy()))
    handle = parallel.attach_grad_allreduce(param)
    param.grad = None
    # emulate autograd accumulating this rank's gradient, which fires the hook
    (param * torch.from_numpy(bw["dctx"])).sum().backward()
    handle.remove()
    # a second path: explicit call on a tensor
    t = torch.from_numpy(bw["dctx"].copy())
    parallel.allreduce_label_context_grad(t)
    # a rank whose parameter received no gradient still takes part: its zeros are reduced and it
    # ends up with the other rank's gradient
    idle = torch.nn.Parameter(torch.zeros(3))
    if rank == 0:
        idle.grad = torch.tensor([1.0, 2.0, 3.0])
    parallel.allreduce_label_context_grad(idle)
    assert torch.equal(idle.grad, torch.tensor([1.0, 2.0, 3.0]))
    with pytest.raises(RuntimeError, match="every rank"):
        parallel.allreduce_label_context_grad(None)
    if rank == 0:
        np.save(out, np.stack([param.grad.numpy(), t.numpy()]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradient_allreduce_matches_full_batch(tmp_path):
    from oracle import oracle
    out = str(tmp_path / "reduced.npy")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(2, port, out), nprocs=2, join=True)
    got = np.load(out)
    unary, ctx, ew, g, D, I = _inputs()
    fw = oracle.forward("TRWP", unary, ctx, ew, D, I)
    want = oracle.backward("TRWP", ctx, ew, g, fw["min_idx"], fw["norm_idx"])["dctx"]
    scale = np.abs(want).max()
    assert np.abs(got[0] - want).max() <= 1e-5 * scale
    assert np.abs(got[1] - want).max() <= 1e-5 * scale
