"""Side by side with the reference's own CUDA extensions (recompiled unmodified for sm_100a by
`python oracle/build.py --ref-cuda` into oracle/_ref/cuda/): the same positional call
(MPLayers/TRWP/TRWP.cpp:245-256,285-295; MPLayers/ISGMR/ISGMR.cpp:300-313,344-356) goes to both
modules on identical tensors, at sizes up to the full segmentation configuration, which no CPU
checker reaches in test time.

Forward values, messages and every saved index must agree bit for bit; gradients within the
gradient tolerance (the reference accumulates them with floating-point atomics in arbitrary
order).  The tests also print both device times (CUDA events) -- informational, never asserted.
Skipped when the reference build is absent.
"""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oracle import ref_cuda  # noqa: E402
from tests.helpers import GRAD_RTOL, rel_err  # noqa: E402

pytestmark = pytest.mark.gpu


def _need(mode):
    if not ref_cuda.available(mode):
        pytest.skip("reference CUDA extension %s not built (python oracle/build.py --ref-cuda)" % mode)


def _inputs(seed, B, H, W, L, D, rank2, with_weights=True):
    import torch
    g = torch.Generator().manual_seed(seed)
    unary = torch.rand(B, 1, H, W, L, generator=g) * 4.0
    if rank2:
        a = torch.rand(L, L, generator=g)
        ctx = torch.triu(a + a.t(), 1)  # upper triangle, zero diagonal: what the L == 21 path reads
    else:
        ctx = torch.minimum(torch.arange(L, dtype=torch.float32) * 0.3, torch.tensor(2.0))
    ew = torch.rand(D, B, 1, H, W, generator=g) * 0.9 + 0.1 if with_weights else torch.ones(D, B, 1, H, W)
    dcost = torch.rand(B, 1, H, W, L, generator=g) - 0.5
    return [t.cuda().contiguous() for t in (unary, ctx, ew, dcost)]


def _timed(fn):
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    out = fn()
    e1.record()
    torch.cuda.synchronize()
    return out, e0.elapsed_time(e1)


def _run_module(mod, mode, unary, ctx, ew, dcost, D, I, rho, train):
    """One forward (+ backward) through an extension module with the reference's signature."""
    import torch
    B, cv, H, W, L = unary.shape
    z = lambda *s, **k: unary.new_zeros(*s, **k)  # noqa: E731
    msg, cost, uu = z(D, B, cv, H, W, L), z(B, cv, H, W, L), z(B, cv, H, W, L)
    e8 = torch.empty(0, dtype=torch.uint8, device=unary.device)
    mi = z(I, D, B, cv, H, W, L, dtype=torch.uint8) if train else e8
    ni = z(I, D, B, cv, H, W, dtype=torch.uint8) if train else e8
    lab = z(I, B, cv, H, W, dtype=torch.uint8)
    mu = z(D, B, cv, H, W, L) if mode == "ISGMR" else None

    def fwd():
        if mode == "TRWP":
            mod.forward(rho, I, 0, unary, ctx, ew, msg, cost, mi, ni, uu, lab)
        else:
            mod.forward(0, rho, I, 0, unary, ctx, ew, msg, cost, mi, ni, uu, mu, lab)

    _, t_f = _timed(fwd)
    out = dict(cost=cost, msg=msg, min_idx=mi, norm_idx=ni, label_all=lab, t_fwd=t_f)
    if train:
        dun, dmsg, duu, dew = z(B, cv, H, W, L), z(D, B, cv, H, W, L), z(B, cv, H, W, L), z(D, B, cv, H, W)
        dctx = torch.zeros_like(ctx)
        dmu = z(D, B, cv, H, W, L) if mode == "ISGMR" else None

        def bwd():
            if mode == "TRWP":
                mod.backward(rho, ctx, ew, dcost, mi, ni, dun, dctx, dew, dmsg, duu)
            else:
                mod.backward(0, rho, ctx, ew, dcost, mi, ni, dun, dctx, dew, dmsg, duu, dmu)

        _, t_b = _timed(bwd)
        out.update(dunary=dun, dcontext=dctx, dedge=dew, t_bwd=t_b)
    return out


def _compare(mode, B, H, W, L, D, I, rank2, train=True, seed=0, repeat=1):
    unary, ctx, ew, dcost = _inputs(seed, B, H, W, L, D, rank2)
    _compare_tensors(mode, unary, ctx, ew, dcost, D, I, train, repeat, "")


def _compare_tensors(mode, unary, ctx, ew, dcost, D, I, train, repeat, tag):
    import mplayers_b200
    ours_mod = mplayers_b200.TRWP if mode == "TRWP" else mplayers_b200.ISGMR
    ref_mod = ref_cuda._load(mode)
    rho = 0.5 if mode == "TRWP" else 1.0
    B, _, H, W, L = unary.shape
    assert ref_cuda.expressible(L, ctx.dim(), I if train else 1, D, B * H * W)
    for _ in range(repeat):  # the last repetition is the one timed warm
        ref = _run_module(ref_mod, mode, unary, ctx, ew, dcost, D, I, rho, train)
        got = _run_module(ours_mod, mode, unary, ctx, ew, dcost, D, I, rho, train)
    for k in ("cost", "msg", "label_all") + (("min_idx", "norm_idx") if train else ()):
        a, b = got[k].cpu().numpy(), ref[k].cpu().numpy()
        assert np.array_equal(a, b), "%s differs from the reference CUDA kernels (%d entries)" % (k, (a != b).sum())
    line = tag + "%s B%d %dx%d L%d D%d I%d: forward %.3f ms (reference CUDA %.3f ms)" % (
        mode, B, H, W, L, D, I, got["t_fwd"], ref["t_fwd"])
    if train:
        for k in ("dunary", "dcontext", "dedge"):
            err = rel_err(got[k].cpu().numpy(), ref[k].cpu().numpy())
            assert err < GRAD_RTOL, (k, err)
        line += ", backward %.3f ms (reference CUDA %.3f ms)" % (got["t_bwd"], ref["t_bwd"])
    print("\n[vs reference CUDA] " + line)


def test_trwp_small_training():
    _need("TRWP")
    _compare("TRWP", 1, 64, 64, 21, 4, 5, rank2=True)


def test_trwp_segmentation_full_size():
    """2 x 512 x 512 pixels, 21 labels, 4 directions, 5 iterations, training."""
    _need("TRWP")
    _compare("TRWP", 2, 512, 512, 21, 4, 5, rank2=True, repeat=2)


def test_trwp_rank1_inference():
    _need("TRWP")
    _compare("TRWP", 1, 96, 160, 64, 4, 2, rank2=False, train=False)


def test_trwp_sixteen_directions():
    _need("TRWP")
    _compare("TRWP", 1, 40, 56, 21, 16, 2, rank2=True)


def test_isgmr_small_training():
    _need("ISGMR")
    _compare("ISGMR", 1, 48, 64, 21, 8, 3, rank2=True)


def test_isgmr_rank1_training():
    _need("ISGMR")
    _compare("ISGMR", 2, 40, 72, 48, 8, 2, rank2=False)


@pytest.mark.parametrize("name,gen,kw,train", [
    ("segmentation", "config4_segmentation", {}, True),
    ("stereo", "config2_stereo", {}, False),
    ("denoise", "config3_denoise", {"n_iter": 10}, False),
    # the same inputs as training steps: the several-labels-per-lane kernels save every index the
    # reference's kernels save, at full size, and their gradients agree
    ("stereo training", "config2_stereo", {"training": True}, True),
    ("denoise training", "config3_denoise", {"n_iter": 3, "training": True}, True),
])
def test_benchmark_configurations_full_size(name, gen, kw, train):
    """The seeded synthetic inputs of the benchmark workloads at full size (the denoising one with
    10 of its 50 iterations: the reference needs ~40 ms per iteration)."""
    import torch
    from mplayers_b200 import synthetic
    cfg = getattr(synthetic, gen)(**kw)
    _need(cfg["mode"])
    unary = cfg["unary"].permute(0, 1, 3, 4, 2).contiguous().cuda()      # [B,cv,L,H,W] -> [B,cv,H,W,L]
    B, cv, H, W, L = unary.shape
    D = cfg["n_dir"]
    if cfg["edge_weights"] is not None:
        ew = cfg["edge_weights"].unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous().cuda()  # [D,B,cv,H,W]
    else:
        ew = torch.ones(D, B, cv, H, W, device="cuda")
    ctx = cfg["label_context"].contiguous().cuda()
    g = torch.Generator().manual_seed(99)
    dcost = (torch.rand(B, cv, H, W, L, generator=g) - 0.5).cuda()
    _compare_tensors(cfg["mode"], unary, ctx, ew, dcost, D, cfg["n_iter"], train, 2, name + ": ")


def _run_soft(mod, unary, ctx, ew, dcost, D, I, rho):
    import torch
    B, cv, H, W, L = unary.shape
    z = lambda *s, **k: unary.new_zeros(*s, **k)  # noqa: E731
    msg, cost, uu = z(D, B, cv, H, W, L), z(B, cv, H, W, L), z(B, cv, H, W, L)
    el = z(I, D, B, cv, H, W, L, L)
    ni = z(I, D, B, cv, H, W, dtype=torch.uint8)
    lab = z(I, B, cv, H, W, dtype=torch.uint8)
    _, t_f = _timed(lambda: mod.forward_soft(rho, I, unary, ctx, ew, msg, el, ni, cost, uu, lab))
    dun, dmsg, duu, dew = z(B, cv, H, W, L), z(D, B, cv, H, W, L), z(B, cv, H, W, L), z(D, B, cv, H, W)
    dctx = torch.zeros_like(ctx)
    _, t_b = _timed(lambda: mod.backward_soft(rho, dcost, ctx, ew, el, ni, dun, dctx, dew, dmsg, duu))
    return dict(cost=cost, msg=msg, edge_label=el, norm_idx=ni, label_all=lab, dunary=dun, dcontext=dctx,
                dedge=dew, t_fwd=t_f, t_bwd=t_b)


@pytest.mark.parametrize("shape", [(1, 40, 56, 21, 4, 2, True), (2, 24, 31, 21, 8, 2, True),
                                   (1, 30, 44, 12, 16, 1, False), (1, 128, 160, 21, 4, 3, True)],
                         ids=lambda s: "-".join(map(str, s)))
def test_soft_trwp(shape):
    """Soft (expected-value) TRWP against the reference's TRWP_hard_soft extension: forward costs,
    messages, saved edge values and normalisation indices bit-identical (same intrinsics and the
    same reduction order); gradients to the gradient tolerance."""
    _need("TRWP_hard_soft")
    import mplayers_b200
    B, H, W, L, D, I, rank2 = shape
    unary, ctx, ew, dcost = _inputs(5, B, H, W, L, D, rank2)
    assert ref_cuda.expressible(L, ctx.dim(), I, D, B * H * W * L)
    ref_mod = ref_cuda._load("TRWP_hard_soft")
    for _ in range(2):
        ref = _run_soft(ref_mod, unary, ctx, ew, dcost, D, I, 0.5)
        got = _run_soft(mplayers_b200.TRWP, unary, ctx, ew, dcost, D, I, 0.5)
    for k in ("cost", "msg", "edge_label", "norm_idx", "label_all"):
        a, b = got[k].cpu().numpy(), ref[k].cpu().numpy()
        assert np.array_equal(a, b), "%s differs from the reference CUDA kernels (%d entries)" % (k, (a != b).sum())
    for k in ("dunary", "dcontext", "dedge"):
        err = rel_err(got[k].cpu().numpy(), ref[k].cpu().numpy())
        assert err < GRAD_RTOL, (k, err)
    print("\n[vs reference CUDA] soft TRWP B%d %dx%d L%d D%d I%d: forward %.3f ms (reference CUDA %.3f ms), "
          "backward %.3f ms (reference CUDA %.3f ms)" % (B, H, W, L, D, I, got["t_fwd"], ref["t_fwd"],
                                                          got["t_bwd"], ref["t_bwd"]))
