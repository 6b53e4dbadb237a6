"""Direction-sharded ISGMR, host logic on CPU: the plan (which rank owns which directions) and the
orchestration (one all-reduce of the message sum per iteration, of the scatter sum per backward
iteration, of the two parameter gradients at the end) run as two gloo ranks with a pure-Python
stand-in for the per-direction sweeps, and must reproduce the CPU oracle's monolithic ISGMR."""
import os
import types

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mplayers_b200 import direction_sharding as ds
from tests.helpers import COST_RTOL, GRAD_RTOL, rel_err


def test_direction_shards_keep_pairs_together_and_cover_all():
    for n_dir in (2, 4, 8, 16):
        for world in (1, 2, 3, 4, 8, 9):
            plan = ds.direction_shards(n_dir, world)
            assert len(plan) == world
            seen = []
            for first, count in plan:
                assert first % 2 == 0 and count % 2 == 0
                seen += list(range(first, first + count))
            assert seen == list(range(n_dir))
            counts = [c for _, c in plan]
            assert max(counts) - min(counts) <= 2
    with pytest.raises(ValueError):
        ds.direction_shards(3, 2)


def test_shard_plan_splits_chains_when_ranks_outnumber_pairs():
    assert ds.shard_plan(8, 4) == [(0, 2, 0, 1), (2, 2, 0, 1), (4, 2, 0, 1), (6, 2, 0, 1)]
    plan = ds.shard_plan(8, 8)
    assert plan == [(2 * (r // 2), 2, r % 2, 2) for r in range(8)]
    plan = ds.shard_plan(4, 7)                       # 2 pairs, 3 ranks each, one rank left over
    assert plan[:6] == [(0, 2, 0, 3), (0, 2, 1, 3), (0, 2, 2, 3), (2, 2, 0, 3), (2, 2, 1, 3), (2, 2, 2, 3)]
    assert plan[6][1] == 0                           # owns nothing, still joins the collectives
    for n_dir, world in ((8, 16), (16, 8), (2, 5)):
        owned = {}
        for first, count, part, parts in ds.shard_plan(n_dir, world):
            for d in range(first, first + count):
                owned.setdefault(d, []).append((part, parts))
        assert sorted(owned) == list(range(n_dir))
        for d, lst in owned.items():                 # every part of every direction exactly once
            parts = lst[0][1]
            assert sorted(p for p, _ in lst) == list(range(parts)) and all(q == parts for _, q in lst)


def test_chunk_count_follows_the_world_size():
    f = ds.DirectionShardedISGMRFunction
    assert [f._chunks(w) for w in (1, 2, 4, 5, 8)] == [4, 4, 4, 1, 1]
    f.chunks = 2                                     # an explicit setting wins
    try:
        assert f._chunks(8) == 2
    finally:
        f.chunks = None


def _inputs():
    rng = np.random.default_rng(11)
    B, H, W, L, D, I = 1, 5, 6, 4, 8, 2
    unary = rng.standard_normal((B, 1, H, W, L)).astype(np.float32)
    a = np.triu(rng.uniform(0, 2, (L, L)), 1)
    ctx = (a + a.T).astype(np.float32)
    ew = rng.uniform(0.2, 1, (D, B, 1, H, W)).astype(np.float32)
    g = rng.uniform(0, 1, (B, 1, H, W, L)).astype(np.float32)
    return unary, ctx, ew, g, D, I


def _args(D, I):
    return types.SimpleNamespace(rho=1.0, mpnet_max_iter=I, mpnet_n_dirs=D, training=True, enable_sgm=False,
                                 enable_min_a_dir=False, enable_saving_label=False)


def _rank_main(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tests.cpu_direction_backend import CpuBackend
    unary, ctx, ew, g, D, I = _inputs()
    u = torch.from_numpy(unary).requires_grad_(True)
    c = torch.from_numpy(ctx).requires_grad_(True)
    e = torch.from_numpy(ew).requires_grad_(True)
    cost = ds.isgmr_direction_sharded(u, c, e, _args(D, I), backend=CpuBackend())
    cost.backward(torch.from_numpy(g))
    np.savez(out % rank, cost=cost.detach().numpy(), dunary=u.grad.numpy(), dctx=c.grad.numpy(), dew=e.grad.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 8])   # whole pairs per rank; two ranks per pair (chains split)
def test_gloo_ranks_reproduce_the_monolithic_layer(tmp_path, world):
    from oracle import oracle
    out = str(tmp_path / "rank%d.npz")
    port = 29500 + (os.getpid() + 7 + world) % 2000
    mp.spawn(_rank_main, args=(world, port, out), nprocs=world, join=True)
    unary, ctx, ew, g, D, I = _inputs()
    fw = oracle.forward("ISGMR", unary, ctx, ew, D, I)
    bw = oracle.backward("ISGMR", ctx, ew, g, fw["min_idx"], fw["norm_idx"])
    r0, r1 = np.load(out % 0), np.load(out % (world - 1))
    for k in ("cost", "dunary", "dctx", "dew"):
        assert np.array_equal(r0[k], r1[k]) or rel_err(r0[k], r1[k]) < 1e-6, k   # every rank ends with the whole result
    assert rel_err(r0["cost"], fw["cost"]) < COST_RTOL
    assert rel_err(r0["dunary"], bw["dunary"]) < GRAD_RTOL
    assert rel_err(r0["dctx"], bw["dctx"]) < GRAD_RTOL
    assert rel_err(r0["dew"], bw["dew"]) < GRAD_RTOL
