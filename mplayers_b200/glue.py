"""Fused layout glue between a network's class scores [B,L,H,W] and the layer's costs [B,1,H,W,L].

The reference's segmentation network does, around its message-passing layer (mpnet.py:161-169):
    costs = -scores;  costs = costs - costs.min(1, keepdim=True)[0]
    results = self.mp_layer(costs.unsqueeze(1), edge_weights=...)      # permutes inside, both ways
    scores = -results[0].squeeze(1)
i.e. six full passes over the volume around the layer (and as many in the backward).  Here the
input side and the output side are one kernel each, forward and backward, and the layer is called
in its native layout.  `mp_on_scores(layer, scores, edge_weights)` is the drop-in for those
three lines (without the optional `enable_score_scale` division, which stays in torch).
"""
import torch

from . import _lib


def _shape(t):
    b, l, h, w = t.shape
    return int(b), int(l), int(h), int(w)


class ScoresToCosts(torch.autograd.Function):
    """scores [B,L,H,W] -> costs [B,1,H,W,L] = max_l(scores) - scores."""

    @staticmethod
    def forward(ctx, scores):
        scores = scores.contiguous()
        _lib.require(scores, "scores", torch.float32)
        b, l, h, w = _shape(scores)
        costs = torch.empty(b, 1, h, w, l, dtype=torch.float32, device=scores.device)
        amax = torch.empty(b, h, w, dtype=torch.uint8, device=scores.device)
        with torch.cuda.device(scores.device):
            _lib.check(_lib.lib().mpl_scores_to_costs(_lib.ptr(scores), _lib.ptr(costs), _lib.ptr(amax), b, l, h, w,
                                                      _lib.stream_ptr(scores.device)))
        ctx.save_for_backward(amax)
        return costs

    @staticmethod
    def backward(ctx, dcosts):
        (amax,) = ctx.saved_tensors
        dcosts = dcosts.contiguous()
        b, _, h, w, l = dcosts.shape
        dscores = torch.empty(b, l, h, w, dtype=torch.float32, device=dcosts.device)
        with torch.cuda.device(dcosts.device):
            _lib.check(_lib.lib().mpl_scores_to_costs_backward(_lib.ptr(dcosts), _lib.ptr(amax), _lib.ptr(dscores),
                                                               int(b), int(l), int(h), int(w),
                                                               _lib.stream_ptr(dcosts.device)))
        return dscores


class CostsToScores(torch.autograd.Function):
    """cost_final [B,1,H,W,L] -> scores [B,L,H,W] = -cost_final."""

    @staticmethod
    def forward(ctx, costs):
        costs = costs.contiguous()
        _lib.require(costs, "costs", torch.float32)
        b, _, h, w, l = costs.shape
        out = torch.empty(b, l, h, w, dtype=torch.float32, device=costs.device)
        with torch.cuda.device(costs.device):
            _lib.check(_lib.lib().mpl_negate_hwl_to_lhw(_lib.ptr(costs), _lib.ptr(out), int(b), int(l), int(h), int(w),
                                                        _lib.stream_ptr(costs.device)))
        return out

    @staticmethod
    def backward(ctx, dscores):
        dscores = dscores.contiguous()
        b, l, h, w = _shape(dscores)
        out = torch.empty(b, 1, h, w, l, dtype=torch.float32, device=dscores.device)
        with torch.cuda.device(dscores.device):
            _lib.check(_lib.lib().mpl_negate_lhw_to_hwl(_lib.ptr(dscores), _lib.ptr(out), b, l, h, w,
                                                        _lib.stream_ptr(dscores.device)))
        return out


def mp_on_scores(layer, scores, edge_weights=None):
    """What mpnet.py:161-169 computes: message passing on costs derived from `scores` [B,L,H,W],
    result returned as scores again.  `layer` is an MPModule of this package; edge_weights
    [B,D,H,W] as the module takes them.  Returns (scores_out [B,L,H,W], label_context)."""
    costs = ScoresToCosts.apply(scores)
    ew = edge_weights.unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous() if edge_weights is not None else None
    cost_final, label_context = layer.forward_native(costs, ew)
    return CostsToScores.apply(cost_final), label_context


def _permute(name, x, out_shape, bc, l, h, w):
    out = torch.empty(out_shape, dtype=torch.float32, device=x.device)
    if out.numel():
        with torch.cuda.device(x.device):
            _lib.check(getattr(_lib.lib(), name)(_lib.ptr(x), _lib.ptr(out), bc, l, h, w, _lib.stream_ptr(x.device)))
    return out


class LabelsLast(torch.autograd.Function):
    """unary [B,cv,L,H,W] -> [B,cv,H,W,L]: the `permute(0, 1, 3, 4, 2).contiguous()` of the module
    call (pytorch/MP_module.py:198) as one kernel that is coalesced on both sides; the backward is
    the inverse change of layout."""

    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        _lib.require(x, "unary", torch.float32)
        b, cv, l, h, w = (int(v) for v in x.shape)
        return _permute("mpl_permute_lhw_to_hwl", x, (b, cv, h, w, l), b * cv, l, h, w)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        b, cv, h, w, l = (int(v) for v in g.shape)
        return _permute("mpl_permute_hwl_to_lhw", g, (b, cv, l, h, w), b * cv, l, h, w)


class LabelsFirst(torch.autograd.Function):
    """cost_final [B,cv,H,W,L] -> [B,cv,L,H,W] (pytorch/MP_module.py:232); inverse of LabelsLast."""

    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        _lib.require(x, "cost_final", torch.float32)
        b, cv, h, w, l = (int(v) for v in x.shape)
        return _permute("mpl_permute_hwl_to_lhw", x, (b, cv, l, h, w), b * cv, l, h, w)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        b, cv, l, h, w = (int(v) for v in g.shape)
        return _permute("mpl_permute_lhw_to_hwl", g, (b, cv, h, w, l), b * cv, l, h, w)


def labels_last(x):
    """[B,cv,L,H,W] -> contiguous [B,cv,H,W,L] (kernel for float32 tensors within its limits, torch otherwise)."""
    if x.dtype == torch.float32 and x.is_cuda and x.dim() == 5 and x.size(2) <= 256 and x.size(0) * x.size(1) <= 65535:
        return LabelsLast.apply(x)
    return x.permute(0, 1, 3, 4, 2).contiguous()


def labels_first(x):
    """[B,cv,H,W,L] -> contiguous [B,cv,L,H,W]."""
    if x.dtype == torch.float32 and x.is_cuda and x.dim() == 5 and x.size(4) <= 256 and x.size(0) * x.size(1) <= 65535:
        return LabelsFirst.apply(x)
    return x.permute(0, 1, 4, 2, 3).contiguous()
