"""(1) Calls on different CUDA streams with their own buffers may overlap on the GPU and must not
disturb each other (the library keeps no device-side state between calls).  (2) Seeded random
small problems -- shapes, label counts, direction counts, context kinds, weights present or not --
against the CPU oracle."""
import numpy as np
import pytest
import torch

import cases
from helpers import COST_RTOL, GRAD_RTOL, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_concurrent_streams_do_not_interfere():
    from mplayers_b200 import ISGMR, TRWP
    dev = "cuda"
    jobs = []
    for k, (mode, D, H, W, L, I) in enumerate([("TRWP", 4, 96, 128, 21, 3), ("ISGMR", 8, 64, 96, 21, 2),
                                               ("TRWP", 8, 80, 72, 32, 2), ("ISGMR", 4, 72, 88, 64, 2)]):
        g = torch.Generator().manual_seed(50 + k)
        u = torch.randn(1, 1, H, W, L, generator=g).to(dev)
        a = torch.triu(torch.rand(L, L, generator=g) * 2, 1)
        ctx = (a + a.t()).to(dev)
        ew = (torch.rand(D, 1, 1, H, W, generator=g) * 0.8 + 0.2).to(dev)
        jobs.append(dict(mode=mode, D=D, I=I, u=u, ctx=ctx, ew=ew, L=L))

    def run(j):
        u, D, I, L = j["u"], j["D"], j["I"], j["L"]
        z = lambda *s, **k: torch.zeros(*s, device=dev, **k)  # noqa: E731
        msg, cost = z(D, *u.shape), z(*u.shape)
        mi, ni = z(I, D, *u.shape, dtype=torch.uint8), z(I, D, *u.shape[:-1], dtype=torch.uint8)
        e0, e8 = torch.empty(0, device=dev), torch.empty(0, dtype=torch.uint8, device=dev)
        if j["mode"] == "TRWP":
            TRWP.forward(0.5, I, 0, u, j["ctx"], j["ew"], msg, cost, mi, ni, e0, e8)
        else:
            ISGMR.forward(0, 1.0, I, 0, u, j["ctx"], j["ew"], msg, cost, mi, ni, e0, z(D, *u.shape), e8)
        return cost, mi

    torch.cuda.synchronize()
    serial = [run(j) for j in jobs]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in jobs]
    overlapped = [None] * len(jobs)
    for rep in range(3):                     # several rounds so that launches really interleave
        for k, (j, s) in enumerate(zip(jobs, streams)):
            with torch.cuda.stream(s):
                overlapped[k] = run(j)
    torch.cuda.synchronize()
    for (c0, m0), (c1, m1) in zip(serial, overlapped):
        assert torch.equal(c0, c1) and torch.equal(m0, m1)


def _random_problem(rng):
    mode = rng.choice(["TRWP", "ISGMR"])
    D = int(rng.choice([2, 4, 8, 16]))
    B, CV = int(rng.integers(1, 3)), int(rng.integers(1, 3))
    H, W = int(rng.integers(1, 14)), int(rng.integers(1, 14))
    L = int(rng.choice([1, 2, 3, 5, 8, 13, 21, 24, 32, 33, 36, 48, 64, 65, 100]))
    I = int(rng.integers(1, 3))
    kind = rng.choice(["sym2d", "potts2d", "tl1d", "tq1d"])
    with_ew = bool(rng.integers(0, 2))
    return mode, D, B, CV, H, W, L, I, kind, with_ew


def _random_wide_problem(rng):
    """1-D contexts on 36..256 labels: the several-labels-per-lane kernels, forward and backward,
    with partly filled lanes, every direction count, short and long chains."""
    mode = rng.choice(["TRWP", "ISGMR"])
    D = int(rng.choice([4, 8, 16]))
    B, CV = int(rng.integers(1, 3)), 1
    H, W = int(rng.integers(2, 24)), int(rng.integers(2, 24))
    L = int(rng.choice([36, 64, 68, 96, 128, 132, 160, 192, 200, 252, 256]))
    I = int(rng.integers(1, 3))
    kind = rng.choice(["tl1d", "tq1d"])
    with_ew = bool(rng.integers(0, 2))
    return mode, D, B, CV, H, W, L, I, kind, with_ew


@pytest.mark.parametrize("seed", list(range(24)) + [100 + k for k in range(12)])
def test_random_small_problems_vs_oracle(seed):
    import gpu_runner as g
    rng = np.random.default_rng(7000 + seed)
    mode, D, B, CV, H, W, L, I, kind, with_ew = _random_problem(rng) if seed < 100 else _random_wide_problem(rng)
    unary = rng.standard_normal((B, CV, H, W, L)).astype(np.float32)
    ctx = cases.make_context(kind, L, rng)
    ew = rng.uniform(0.2, 1.5, size=(D, B, CV, H, W)).astype(np.float32) if with_ew else None
    dcost = rng.uniform(0, 1, size=(B, CV, H, W, L)).astype(np.float32)
    got = g.forward(mode, unary, ctx, ew, D, I, save_labels=True)
    want = oracle.forward(mode, unary, ctx, ew, D, I, save_labels=True)
    what = (mode, D, B, CV, H, W, L, I, kind, with_ew)
    assert np.array_equal(got["cost"], want["cost"]), what
    assert np.array_equal(got["norm_idx"], want["norm_idx"]), what
    assert np.array_equal(got["label_all"], want["label_all"]), what
    # also where training takes the windowed kernels: their tie rule is the dense evaluation's
    assert np.array_equal(got["min_idx"], want["min_idx"]), what
    bw = g.backward(mode, ctx, ew, dcost, want["min_idx"], want["norm_idx"])
    ref = oracle.backward(mode, ctx, ew, dcost, want["min_idx"], want["norm_idx"])
    assert rel_err(bw["dunary"], ref["dunary"]) < GRAD_RTOL, what
    assert rel_err(bw["dctx"], ref["dctx"]) < GRAD_RTOL, what
    if with_ew:
        assert rel_err(bw["dew"], ref["dew"]) < GRAD_RTOL, what
    ev = g.forward(mode, unary, ctx, ew, D, I, training=False)
    assert rel_err(ev["cost"], want["cost"]) < COST_RTOL, what
