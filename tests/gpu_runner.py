"""Runs the CUDA path (through the extension-level modules, i.e. the C ABI) on numpy inputs and
returns numpy outputs in the same form as oracle.oracle.forward / backward."""
import numpy as np
import torch

from mplayers_b200 import ISGMR, TRWP


def _dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device="cuda", dtype=dtype)


def forward(mode, unary, ctx, edge_weights, n_dir, n_iter, rho=None, training=True,
            save_labels=False, enable_sgm=False, enable_min_a_dir=False, msg_init=None, context_window=0,
            cost_labels_first=False):
    if rho is None:
        rho = 0.5 if mode == "TRWP" else 1.0
    u = _dev(unary)
    b, cv, h, w, l = u.shape
    c = _dev(ctx)
    e0 = torch.empty(0, device="cuda")
    e8 = torch.empty(0, dtype=torch.uint8, device="cuda")
    ew = _dev(edge_weights) if edge_weights is not None else e0
    msg = torch.zeros(n_dir, b, cv, h, w, l, device="cuda") if msg_init is None else _dev(msg_init)
    cost = torch.full((b, cv, l, h, w) if cost_labels_first else (b, cv, h, w, l), float("nan"), device="cuda")
    mi = torch.zeros(n_iter, n_dir, b, cv, h, w, l, dtype=torch.uint8, device="cuda") if training else e8
    ni = torch.zeros(n_iter, n_dir, b, cv, h, w, dtype=torch.uint8, device="cuda") if training else e8
    lab = torch.zeros(n_iter, b, cv, h, w, dtype=torch.uint8, device="cuda") if save_labels else e8
    if mode == "TRWP":
        TRWP.forward(rho, n_iter, int(enable_min_a_dir), u, c, ew, msg, cost, mi, ni, e0, lab,
                     context_window=context_window, cost_labels_first=cost_labels_first)
    else:
        mu = torch.zeros_like(msg)
        ISGMR.forward(int(enable_sgm), rho, n_iter, int(enable_min_a_dir), u, c, ew, msg, cost, mi, ni,
                      e0, mu, lab, context_window=context_window, cost_labels_first=cost_labels_first)
    torch.cuda.synchronize()
    return dict(cost=cost.cpu().numpy(), msg=msg.cpu().numpy(),
                min_idx=mi.cpu().numpy() if training else None,
                norm_idx=ni.cpu().numpy() if training else None,
                label_all=lab.cpu().numpy() if save_labels else None)


def backward(mode, ctx, edge_weights, dcost, min_idx, norm_idx, rho=None, enable_sgm=False,
             keep_diag=False, context_window=0, cost_labels_first=False):
    """`dcost` is [B,cv,L,H,W] with cost_labels_first, else [B,cv,H,W,L]; dunary always [B,cv,H,W,L]."""
    if rho is None:
        rho = 0.5 if mode == "TRWP" else 1.0
    g = _dev(dcost)
    c = _dev(ctx)
    mi = _dev(min_idx, torch.uint8)
    ni = _dev(norm_idx, torch.uint8)
    n_iter, n_dir = mi.shape[:2]
    e0 = torch.empty(0, device="cuda")
    ew = _dev(edge_weights) if edge_weights is not None else e0
    shape = tuple(mi.shape[2:])
    dunary = torch.full(shape, float("nan"), device="cuda")
    dctx = torch.zeros_like(c)
    dew = torch.zeros_like(ew)
    # scratch is deliberately filled with garbage: the library must not rely on its contents
    dmsg = torch.full((n_dir,) + shape, float("nan"), device="cuda")
    if mode == "TRWP":
        TRWP.backward(rho, c, ew, g, mi, ni, dunary, dctx, dew, dmsg, e0, keep_diag=keep_diag,
                      context_window=context_window, cost_labels_first=cost_labels_first)
    else:
        dmu = torch.full_like(dmsg, float("nan"))
        ISGMR.backward(int(enable_sgm), rho, c, ew, g, mi, ni, dunary, dctx, dew, dmsg, e0, dmu,
                       keep_diag=keep_diag, context_window=context_window, cost_labels_first=cost_labels_first)
    torch.cuda.synchronize()
    return dict(dunary=dunary.cpu().numpy(), dctx=dctx.cpu().numpy(),
                dew=dew.cpu().numpy() if edge_weights is not None else None)


def forward_soft(unary, ctx, edge_weights, n_dir, n_iter, rho=0.5, training=True, save_labels=False):
    u = _dev(unary)
    b, cv, h, w, l = u.shape
    c = _dev(ctx)
    e0 = torch.empty(0, device="cuda")
    e8 = torch.empty(0, dtype=torch.uint8, device="cuda")
    ew = _dev(edge_weights) if edge_weights is not None else e0
    msg = torch.zeros(n_dir, b, cv, h, w, l, device="cuda")
    cost = torch.full((b, cv, h, w, l), float("nan"), device="cuda")
    el = torch.zeros(n_iter, n_dir, b, cv, h, w, l, l, device="cuda") if training else e0
    ni = torch.zeros(n_iter, n_dir, b, cv, h, w, dtype=torch.uint8, device="cuda") if training else e8
    lab = torch.zeros(n_iter, b, cv, h, w, dtype=torch.uint8, device="cuda") if save_labels else e8
    TRWP.forward_soft(rho, n_iter, u, c, ew, msg, el, ni, cost, e0, lab)
    torch.cuda.synchronize()
    return dict(cost=cost.cpu().numpy(), msg=msg.cpu().numpy(),
                edge_label=el.cpu().numpy() if training else None,
                norm_idx=ni.cpu().numpy() if training else None,
                label_all=lab.cpu().numpy() if save_labels else None)


def backward_soft(ctx, edge_weights, dcost, edge_label, norm_idx, rho=0.5):
    g = _dev(dcost)
    c = _dev(ctx)
    el = _dev(edge_label)
    ni = _dev(norm_idx, torch.uint8)
    n_dir = ni.shape[1]
    e0 = torch.empty(0, device="cuda")
    ew = _dev(edge_weights) if edge_weights is not None else e0
    dunary = torch.full_like(g, float("nan"))
    dctx = torch.zeros_like(c)
    dew = torch.zeros_like(ew)
    dmsg = torch.full((n_dir,) + tuple(g.shape), float("nan"), device="cuda")
    TRWP.backward_soft(rho, g, c, ew, el, ni, dunary, dctx, dew, dmsg, e0)
    torch.cuda.synchronize()
    return dict(dunary=dunary.cpu().numpy(), dctx=dctx.cpu().numpy(),
                dew=dew.cpu().numpy() if edge_weights is not None else None)
