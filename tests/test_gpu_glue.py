"""Fused score <-> cost glue against the torch expressions the reference's network uses around its
layer (mpnet.py:161-169), forward and backward, and timed side by side (informational)."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu


def _layer(mode, L, D, I):
    from mplayers_b200 import MPModule
    args = types.SimpleNamespace(mpnet_mrf_mode=mode, mpnet_max_iter=I, mpnet_n_dirs=D, n_classes=L,
                                 mpnet_smoothness_train=None, mpnet_term_weight=1.0, mpnet_diag_value=0.0,
                                 enable_symmetric=True)
    layer = MPModule(args).cuda()
    g = torch.Generator().manual_seed(2)
    a = torch.triu(torch.rand(L, L, generator=g) * 2, 1)
    layer.set_label_context(torch.nn.Parameter((a + a.t()).cuda()), None, None)
    layer.train()
    return layer


def _reference_glue(layer, scores, ew):
    costs = -scores
    costs = costs - costs.min(1, keepdim=True)[0]
    results = layer(costs.unsqueeze(1), edge_weights=ew)
    return -results[0].squeeze(1)


@pytest.mark.parametrize("mode,B,L,H,W,D", [("TRWP", 2, 21, 37, 45, 4), ("ISGMR", 1, 7, 5, 100, 8), ("TRWP", 1, 40, 33, 31, 4)])
def test_glue_equals_the_torch_expressions(mode, B, L, H, W, D):
    from mplayers_b200.glue import mp_on_scores
    layer = _layer(mode, L, D, 2)
    g = torch.Generator().manual_seed(9)
    scores0 = torch.randn(B, L, H, W, generator=g).cuda()
    ew0 = (torch.rand(B, D, H, W, generator=g) * 0.8 + 0.2).cuda()
    gout = torch.rand(B, L, H, W, generator=g).cuda()
    outs = []
    for fused in (False, True):
        s = scores0.clone().requires_grad_(True)
        e = ew0.clone().requires_grad_(True)
        layer.label_context.grad = None
        out = mp_on_scores(layer, s, e)[0] if fused else _reference_glue(layer, s, e)
        (out * gout).sum().backward()
        outs.append((out.detach(), s.grad.clone(), e.grad.clone(), layer.label_context.grad.clone()))
    (o0, s0, e0, c0), (o1, s1, e1, c1) = outs
    assert torch.equal(o0, o1)                       # same arithmetic: max - s == -s - min(-s)
    # the per-pixel sum of the cost gradient is formed in another order than torch's reduction
    for a, b in ((s0, s1), (e0, e1), (c0, c1)):
        assert float((a - b).abs().max()) <= 1e-4 * max(float(a.abs().max()), 1e-30)


def test_glue_timing_on_the_segmentation_shape():
    from mplayers_b200.glue import mp_on_scores
    layer = _layer("TRWP", 21, 4, 5)
    g = torch.Generator().manual_seed(1)
    scores = torch.randn(2, 21, 512, 512, generator=g).cuda().requires_grad_(True)
    ew = (torch.rand(2, 4, 512, 512, generator=g) * 0.8 + 0.2).cuda().requires_grad_(True)
    gout = torch.rand(2, 21, 512, 512, generator=g).cuda()

    def run(fused):
        scores.grad = None
        out = mp_on_scores(layer, scores, ew)[0] if fused else _reference_glue(layer, scores, ew)
        (out * gout).sum().backward()

    times = {}
    for fused in (False, True):
        for _ in range(3):
            run(fused)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            run(fused)
        e1.record()
        torch.cuda.synchronize()
        times[fused] = e0.elapsed_time(e1) / 10
    print("\n[glue] scores -> layer -> scores, fwd+bwd, B2 512x512 L21: torch expressions %.3f ms, fused glue %.3f ms"
          % (times[False], times[True]))


@pytest.mark.parametrize("shape", [(2, 1, 21, 37, 45), (1, 3, 64, 8, 130), (1, 1, 256, 5, 7), (3, 1, 1, 4, 4)])
def test_plain_layout_change_equals_torch_permute(shape):
    """LabelsLast / LabelsFirst (the module call's two permutes) against torch, values and gradients
    bit for bit (they only move data)."""
    import torch
    from mplayers_b200 import glue
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(*shape, generator=g).cuda().requires_grad_(True)
    y = glue.labels_last(x)
    assert y.is_contiguous() and torch.equal(y, x.permute(0, 1, 3, 4, 2))
    w = torch.randn(*y.shape, generator=g).cuda()
    (y * w).sum().backward()
    assert torch.equal(x.grad, w.permute(0, 1, 4, 2, 3))
    z = y.detach().requires_grad_(True)
    back = glue.labels_first(z)
    assert back.is_contiguous() and torch.equal(back, x.detach())
    w2 = torch.randn(*back.shape, generator=g).cuda()
    (back * w2).sum().backward()
    assert torch.equal(z.grad, w2.permute(0, 1, 3, 4, 2))
    xd = x.detach().double()   # other dtypes take the torch path
    assert torch.equal(glue.labels_last(xd), xd.permute(0, 1, 3, 4, 2))
