"""Direction-sharded ISGMR on the GPU through the iteration-level C ABI.

One-GPU cases run the ranks as threads of this process (every rank's kernels go to the same
stream, the all-reduce is a barrier plus a sum in rank order), which checks the sweeps over
direction subsets, the partial sums and the combine step against the monolithic layer.  The
two-GPU case runs real ranks over NCCL and is skipped on a single-GPU machine."""
import os
import threading
import types

import numpy as np
import pytest
import torch

from tests.helpers import COST_RTOL, GRAD_RTOL, rel_err

pytestmark = pytest.mark.gpu


class ThreadComm:
    """All-reduce among the threads of one process (one per emulated rank)."""

    def __init__(self, rank, world, shared):
        self.rank, self.world_size, self.s = rank, world, shared

    def all_reduce(self, t):
        s = self.s
        s["slots"][self.rank] = t
        s["barrier"].wait()
        total = s["slots"][0].clone()
        for r in range(1, self.world_size):
            total += s["slots"][r]
        s["barrier"].wait()
        t.copy_(total)
        s["barrier"].wait()
        return t


def _dyadic_case(seed, B, H, W, L, D):
    """Inputs on a coarse binary grid: every sum and product of the layer is then exact in fp32,
    so the result cannot depend on the order in which the directions are summed and the sharded
    run must equal the monolithic one bit for bit (ties included: same kernels, same tie rule)."""
    g = torch.Generator().manual_seed(seed)
    unary = torch.randint(0, 64, (B, 1, H, W, L), generator=g).float() / 8
    a = torch.triu(torch.randint(0, 16, (L, L), generator=g).float() / 4, 1)
    ctx = a + a.t()
    ew = torch.randint(1, 3, (D, B, 1, H, W), generator=g).float() / 2      # 0.5 or 1
    dcost = torch.randint(0, 16, (B, 1, H, W, L), generator=g).float() / 16
    return unary, ctx, ew, dcost


def _case(seed, B, H, W, L, D, rank2, weights=True):
    g = torch.Generator().manual_seed(seed)
    unary = torch.randn(B, 1, H, W, L, generator=g)
    if rank2:
        a = torch.triu(torch.rand(L, L, generator=g) * 2, 1)
        ctx = a + a.t()
    else:
        ctx = torch.minimum(torch.arange(L, dtype=torch.float32) * 0.4, torch.tensor(1.7))
    ew = torch.rand(D, B, 1, H, W, generator=g) * 0.8 + 0.2 if weights else None
    dcost = torch.rand(B, 1, H, W, L, generator=g)
    return unary, ctx, ew, dcost


def _args(D, I, sgm=False):
    return types.SimpleNamespace(rho=1.0, mpnet_max_iter=I, mpnet_n_dirs=D, training=True, enable_sgm=sgm,
                                 enable_min_a_dir=False, enable_saving_label=False)


def _monolithic(unary, ctx, ew, dcost, args):
    from mplayers_b200 import ISGMRFunction
    u = unary.cuda().requires_grad_(True)
    c = ctx.cuda().requires_grad_(True)
    e = ew.cuda().requires_grad_(True) if ew is not None else None
    cost, _ = ISGMRFunction.apply(u, c, e, args)
    cost.backward(dcost.cuda())
    return dict(cost=cost.detach().cpu().numpy(), dunary=u.grad.cpu().numpy(), dctx=c.grad.cpu().numpy(),
                dew=e.grad.cpu().numpy() if e is not None else None)


def _sharded_threads(world, unary, ctx, ew, dcost, args):
    from mplayers_b200 import direction_sharding as ds
    shared = dict(slots=[None] * world, barrier=threading.Barrier(world, timeout=120))
    results, errors = [None] * world, []

    def run(rank):
        try:
            torch.cuda.set_device(0)
            # The autograd engine would run every rank's backward on the one worker thread of the
            # device, where the first all-reduce waits for ranks queued behind it: call the two
            # halves of the Function directly on this thread instead.
            fn, cx = ds.DirectionShardedISGMRFunction, types.SimpleNamespace()
            e = ew.cuda() if ew is not None else None
            with torch.no_grad():
                cost = fn.forward(cx, unary.cuda(), ctx.cuda(), e, args, ThreadComm(rank, world, shared),
                                  ds.CudaBackend())
                dun, dctx, dew = fn.backward(cx, dcost.cuda())[:3]
            results[rank] = dict(cost=cost.cpu().numpy(), dunary=dun.cpu().numpy(), dctx=dctx.cpu().numpy(),
                                 dew=dew.cpu().numpy() if dew is not None else None)
        except Exception as exc:  # a failed rank must not leave the others waiting
            errors.append(exc)
            shared["barrier"].abort()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return results


def _mostly_equal(a, b, tol):
    """Gradients of two runs whose forward sums differ by rounding: where two candidates of a
    min were within rounding of each other the saved index may differ and the gradient then
    takes the other route, so a few entries may differ by O(1); all others agree to `tol`."""
    scale = max(np.abs(b).max(), 1e-30)
    return np.mean(np.abs(a.astype(np.float64) - b) > tol * scale) < 2e-3


def _check(results, want, exact=False):
    for r in results:
        if exact:
            for k in ("cost", "dunary", "dctx", "dew"):
                assert np.array_equal(r[k], want[k]), k
            continue
        assert rel_err(r["cost"], want["cost"]) < COST_RTOL
        assert _mostly_equal(r["dunary"], want["dunary"], GRAD_RTOL)
        assert rel_err(r["dctx"], want["dctx"]) < 2e-2
        if want["dew"] is not None:
            assert _mostly_equal(r["dew"], want["dew"], GRAD_RTOL)
    for r in results[1:]:   # every rank ends with the same complete result
        for k in ("cost", "dunary", "dctx"):
            assert np.array_equal(r[k], results[0][k]), k


@pytest.mark.parametrize("world,shape", [
    (1, (1, 12, 14, 21, 8, 3, True)),
    (2, (1, 12, 14, 21, 8, 3, True)),
    (4, (2, 20, 17, 21, 8, 2, True)),
    (3, (1, 18, 22, 64, 8, 2, True)),     # uneven split; two-labels-per-lane kernels
    (2, (1, 16, 19, 40, 4, 3, False)),    # 1-D context
    (8, (1, 9, 11, 12, 16, 2, True)),     # one pair per rank, 16 directions
    (8, (1, 20, 17, 21, 8, 2, True)),     # two ranks per pair: each walks half of the pair's lines
    (6, (2, 18, 22, 64, 4, 2, True)),     # three ranks per pair, two images, two-labels-per-lane kernels
    (5, (1, 14, 15, 40, 8, 2, False)),    # more ranks than pairs but not twice as many: one rank owns nothing
    (8, (1, 14, 15, 96, 8, 2, False)),    # 1-D context, 96 labels: the several-labels-per-lane kernels on half of a pair's lines
    (6, (1, 12, 18, 40, 4, 2, False)),    # 1-D context, three ranks per pair
])
def test_thread_ranks_match_the_monolithic_layer(world, shape):
    B, H, W, L, D, I, rank2 = shape
    unary, ctx, ew, dcost = _case(world * 10 + L, B, H, W, L, D, rank2)
    args = _args(D, I)
    want = _monolithic(unary, ctx, ew, dcost, args)
    _check(_sharded_threads(world, unary, ctx, ew, dcost, args), want)


@pytest.mark.parametrize("world,L", [(2, 21), (4, 64), (8, 64), (16, 21)])
def test_thread_ranks_bit_identical_on_exact_inputs(world, L):
    unary, ctx, ew, dcost = _dyadic_case(5, 1, 20, 24, L, 8)
    args = _args(8, 3)
    want = _monolithic(unary, ctx, ew, dcost, args)
    _check(_sharded_threads(world, unary, ctx, ew, dcost, args), want, exact=True)


def test_without_edge_weights_and_single_iteration_sgm():
    unary, ctx, _, dcost = _case(3, 1, 10, 13, 21, 8, True, weights=False)
    args = _args(8, 1, sgm=True)
    want = _monolithic(unary, ctx, None, dcost, args)
    _check(_sharded_threads(2, unary, ctx, None, dcost, args), want)


def test_rejects_ranges_that_split_a_pair():
    import ctypes
    from mplayers_b200 import _lib
    prob = _lib.Problem(1, 8, 1, 1, 4, 4, 5, 2, 0, 0, 0, 1.0)
    t = torch.zeros(8 * 4 * 4 * 5, device="cuda")
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    rc = _lib.lib().mpl_isgmr_forward_directions(ctypes.byref(prob), 1, 2, _lib.ptr(t), _lib.ptr(t), None,
                                                 _lib.ptr(t), _lib.ptr(t.clone()), None, None, _lib.ptr(ws), 4096, None)
    assert rc != 0 and b"pair" in _lib.lib().mpl_last_error()


def _nccl_rank(rank, world, port, out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from mplayers_b200 import direction_sharding as ds
    unary, ctx, ew, dcost = _dyadic_case(77, 1, 48, 56, 64, 8)
    u = unary.cuda().requires_grad_(True)
    c = ctx.cuda().requires_grad_(True)
    e = ew.cuda().requires_grad_(True)
    cost = ds.isgmr_direction_sharded(u, c, e, _args(8, 3))
    cost.backward(dcost.cuda())
    torch.cuda.synchronize()
    np.savez(out % rank, cost=cost.detach().cpu().numpy(), dunary=u.grad.cpu().numpy(), dctx=c.grad.cpu().numpy(),
             dew=e.grad.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpus_over_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    out = str(tmp_path / "rank%d.npz")
    port = 29500 + (os.getpid() + 13) % 2000
    mp.spawn(_nccl_rank, args=(2, port, out), nprocs=2, join=True)
    unary, ctx, ew, dcost = _dyadic_case(77, 1, 48, 56, 64, 8)
    want = _monolithic(unary, ctx, ew, dcost, _args(8, 3))
    _check([dict(np.load(out % r)) for r in range(2)], want, exact=True)
