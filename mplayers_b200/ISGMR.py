"""Drop-in for the reference's `ISGMR` extension module (lib_stereo.ISGMR / lib_seg.ISGMR):
`forward` / `backward` with the reference's positional signatures
(MPLayers/ISGMR/ISGMR.cpp:300-313,344-356,399-404).  See TRWP.py for the visible differences; in
addition `msg` / `msg_update` (and `dmsg` / `dmsg_update`) are used alternately instead of being
copied every iteration, so on return `msg` holds the final messages and `msg_update` those of the
iteration before.
"""
import ctypes

import torch

from . import _lib
from .TRWP import _problem


def forward(enable_sgm, rho, n_iter, enable_min_a_dir, unary, context, edge_weights, msg, cost_final,
            msg_min_index, msg_norm_index, unary_update, msg_update, label_all, context_window=0,
            cost_labels_first=False):
    dev = unary.device
    for t, n in ((unary, "unary"), (context, "context"), (edge_weights, "edge_weights"), (msg, "msg"),
                 (cost_final, "cost_final"), (msg_update, "msg_update")):
        _lib.require(t, n, torch.float32, dev)
    for t, n in ((msg_min_index, "msg_min_index"), (msg_norm_index, "msg_norm_index"),
                 (label_all, "label_all")):
        _lib.require(t, n, torch.uint8, dev)
    if msg.dim() != 6 or tuple(unary.shape) != tuple(msg.shape[1:]) or msg.shape != msg_update.shape:
        raise RuntimeError("msg and msg_update must be [D,B,cv,H,W,L] matching unary [B,cv,H,W,L]")
    prob = _problem(n_iter, tuple(msg.shape), context, rho, enable_min_a_dir, enable_sgm,
                    context_window=context_window, cost_labels_first=cost_labels_first)
    with torch.cuda.device(dev):
        nbytes = _lib.lib().mpl_forward_workspace_bytes(ctypes.byref(prob))
        ws = _lib.workspace(nbytes, dev)
        _lib.check(_lib.lib().mpl_isgmr_forward(
            ctypes.byref(prob), _lib.ptr(unary), _lib.ptr(context), _lib.ptr(edge_weights),
            _lib.ptr(msg), _lib.ptr(msg_update), _lib.ptr(cost_final), _lib.ptr(msg_min_index),
            _lib.ptr(msg_norm_index), _lib.ptr(label_all), _lib.ptr(ws), nbytes,
            _lib.stream_ptr(dev)))
        _lib.check_status(ws, "ISGMR.forward")


def backward(enable_sgm, rho, context, edge_weights, dcost_final, msg_min_index, msg_norm_index,
             dunary, dcontext, dedge_weights, dmsg, dunary_update, dmsg_update, keep_diag=False, context_window=0,
             cost_labels_first=False):
    dev = dcost_final.device
    for t, n in ((context, "context"), (edge_weights, "edge_weights"), (dcost_final, "dcost_final"),
                 (dunary, "dunary"), (dcontext, "dcontext"), (dedge_weights, "dedge_weights"),
                 (dmsg, "dmsg"), (dmsg_update, "dmsg_update")):
        _lib.require(t, n, torch.float32, dev)
    for t, n in ((msg_min_index, "msg_min_index"), (msg_norm_index, "msg_norm_index")):
        _lib.require(t, n, torch.uint8, dev)
    if msg_min_index.dim() != 7:
        raise RuntimeError("msg_min_index must be [I,D,B,cv,H,W,L]")
    prob = _problem(msg_min_index.size(0), tuple(msg_min_index.shape[1:]), context, rho,
                    enable_sgm=enable_sgm, keep_diag_=keep_diag, context_window=max(int(context_window), 0),
                    cost_labels_first=cost_labels_first)
    with torch.cuda.device(dev):
        nbytes = _lib.lib().mpl_backward_workspace_bytes(ctypes.byref(prob))
        ws = _lib.workspace(nbytes, dev)
        _lib.check(_lib.lib().mpl_isgmr_backward(
            ctypes.byref(prob), _lib.ptr(context), _lib.ptr(edge_weights), _lib.ptr(dcost_final),
            _lib.ptr(msg_min_index), _lib.ptr(msg_norm_index), _lib.ptr(dunary), _lib.ptr(dcontext),
            _lib.ptr(dedge_weights), _lib.ptr(dmsg), _lib.ptr(dmsg_update), _lib.ptr(ws), nbytes,
            _lib.stream_ptr(dev)))
        _lib.check_status(ws, "ISGMR.backward")
