"""Soft (expected-value) TRWP on the GPU against the golden vectors of the reference's PyTorch
implementation and against the CPU oracle.  The oracle uses expf, the kernels __expf (as the
reference's CUDA kernels do), so values agree to the cost tolerance, not bit for bit."""
import os
import types

import numpy as np
import pytest

import cases
from helpers import COST_RTOL, GRAD_RTOL, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _gpu():
    import gpu_runner
    return gpu_runner


def _compare(got, want, inp_ctx, ew, dcost, has_ew=True):
    g = _gpu()
    assert rel_err(got["cost"], want["cost"]) < COST_RTOL
    assert rel_err(got["msg"], want["msg"]) < COST_RTOL
    assert (got["norm_idx"] != want["norm_idx"]).mean() < 2e-3     # near-ties of the normalisation only
    scale = np.abs(want["edge_label"]).max()
    assert np.abs(got["edge_label"] - want["edge_label"]).max() <= COST_RTOL * scale
    # backward from the ORACLE's saved values, so that both replay the same forward
    bw = g.backward_soft(inp_ctx, ew, dcost, want["edge_label"], want["norm_idx"])
    ref = oracle.backward_soft(inp_ctx, ew, dcost, want["edge_label"], want["norm_idx"])
    assert rel_err(bw["dunary"], ref["dunary"]) < GRAD_RTOL
    assert rel_err(bw["dctx"], ref["dctx"]) < GRAD_RTOL
    if has_ew:
        assert rel_err(bw["dew"], ref["dew"]) < GRAD_RTOL
    return bw


@pytest.mark.parametrize("name", [n for n in cases.CASES if cases.is_soft(n)])
def test_soft_golden_cases(name):
    g = _gpu()
    inp = cases.make_inputs(name)
    gold = np.load(os.path.join(GOLD, name + ".npz"))
    got = g.forward_soft(inp["unary"], inp["ctx"], inp["ew"], inp["n_dir"], inp["n_iter"], save_labels=True)
    want = oracle.forward_soft(inp["unary"], inp["ctx"], inp["ew"], inp["n_dir"], inp["n_iter"], save_labels=True)
    assert rel_err(got["cost"], gold["cost"]) < COST_RTOL
    assert np.array_equal(got["norm_idx"], gold["norm_idx"])
    assert np.array_equal(got["label_all"], want["label_all"])
    bw = _compare(got, want, inp["ctx"], inp["ew"], inp["dcost"])
    # and end to end against the reference's autograd gradients
    own = g.backward_soft(inp["ctx"], inp["ew"], inp["dcost"], got["edge_label"], got["norm_idx"])
    assert rel_err(own["dunary"], gold["dunary"]) < GRAD_RTOL
    assert rel_err(own["dew"], gold["dew"]) < GRAD_RTOL
    assert rel_err(own["dctx"], gold["dctx"]) < GRAD_RTOL
    assert bw is not None


SHAPES = [
    (4, 1, 1, 1, 1, 2, 2, "sym2d"),     # single pixel
    (4, 1, 1, 1, 9, 3, 2, "sym2d"),     # one row
    (16, 2, 1, 5, 7, 4, 2, "sym2d"),    # image smaller than the largest step
    (4, 2, 2, 13, 17, 21, 2, "sym2d"),  # cv axis > 1, segmentation label count
    (8, 1, 1, 12, 11, 32, 2, "sym2d"),  # full warp
    (8, 1, 1, 10, 9, 17, 1, "tl1d"),    # rank-1 context
    (4, 1, 1, 40, 37, 21, 1, "sym2d"),  # chains longer than the staging ring
    (4, 1, 1, 9, 11, 33, 2, "sym2d"),   # first label count of the CTA-per-chain kernels
    (8, 2, 1, 10, 12, 64, 1, "sym2d"),  # their largest, diagonals, two images
    (4, 1, 2, 7, 9, 48, 2, "tl1d"),     # rank-1 context, cv axis
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "-".join(map(str, s)))
def test_soft_forward_backward_vs_oracle(shape):
    g = _gpu()
    D, B, CV, H, W, L, I, kind = shape
    rng = np.random.default_rng(1000 + SHAPES.index(shape))
    unary = rng.standard_normal((B, CV, H, W, L)).astype(np.float32)
    ctx = cases.make_context(kind, L, rng)
    ew = rng.uniform(0.3, 1.4, size=(D, B, CV, H, W)).astype(np.float32)
    dcost = rng.uniform(0, 1, size=(B, CV, H, W, L)).astype(np.float32)
    got = g.forward_soft(unary, ctx, ew, D, I)
    want = oracle.forward_soft(unary, ctx, ew, D, I)
    _compare(got, want, ctx, ew, dcost)
    ev = g.forward_soft(unary, ctx, ew, D, I, training=False)
    assert np.array_equal(ev["cost"], got["cost"])       # inference = training without the saves
    noew = g.forward_soft(unary, ctx, None, D, 1)
    assert rel_err(noew["cost"], oracle.forward_soft(unary, ctx, None, D, 1)["cost"]) < COST_RTOL


def test_soft_module_autograd_and_limits():
    import torch
    from mplayers_b200.MP_module_hard_soft import MPModule
    args = types.SimpleNamespace(mpnet_mrf_mode="TRWP", mpnet_max_iter=2, mpnet_n_dirs=4, n_classes=21,
                                 mpnet_smoothness_train=None, mpnet_term_weight=1.0, mpnet_diag_value=0.0,
                                 enable_symmetric=True, mpnet_enable_soft=True, enable_saving_label=False)
    layer = MPModule(args).cuda()
    gen = torch.Generator().manual_seed(4)
    a = torch.triu(torch.rand(21, 21, generator=gen), 1)
    ctx = torch.nn.Parameter((a + a.t()).cuda())
    layer.set_label_context(ctx, None, None)
    layer.train()
    u = torch.randn(2, 1, 21, 16, 20, generator=gen).cuda().requires_grad_(True)     # [B,cv,L,H,W]
    e = (torch.rand(2, 4, 16, 20, generator=gen) * 0.8 + 0.2).cuda().requires_grad_(True)
    cost, lc, _, vec, idx = layer(u, e)
    assert tuple(vec.shape) == (2, 4, 2, 1, 16, 20, 21, 21) and tuple(idx.shape) == (2, 4, 2, 1, 16, 20)
    g = torch.rand(cost.shape, generator=gen).cuda()
    (cost * g).sum().backward()
    uh = u.detach().permute(0, 1, 3, 4, 2).contiguous().cpu().numpy()
    eh = e.detach().unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous().cpu().numpy()
    fw = oracle.forward_soft(uh, ctx.detach().cpu().numpy(), eh, 4, 2)
    bw = oracle.backward_soft(ctx.detach().cpu().numpy(), eh, g.permute(0, 1, 3, 4, 2).contiguous().cpu().numpy(),
                              fw["edge_label"], fw["norm_idx"])
    assert rel_err(cost.detach().permute(0, 1, 3, 4, 2).cpu().numpy(), fw["cost"]) < COST_RTOL
    assert rel_err(u.grad.permute(0, 1, 3, 4, 2).cpu().numpy(), bw["dunary"]) < GRAD_RTOL
    assert rel_err(ctx.grad.cpu().numpy(), bw["dctx"]) < GRAD_RTOL
    assert rel_err(e.grad.unsqueeze(1).permute(2, 0, 1, 3, 4).cpu().numpy(), bw["dew"]) < GRAD_RTOL
    # more than 64 labels: refused with a message, nothing computed on the CPU
    args.n_classes = 70
    big = MPModule(args).cuda()
    big.set_label_context(torch.zeros(70, 70, device="cuda"), None, None)
    with pytest.raises(RuntimeError, match="n_disp <= 64"):
        big(torch.zeros(1, 1, 70, 4, 4, device="cuda"))
