"""Drop-in for the reference's `TRWP` extension module (lib_stereo.TRWP / lib_seg.TRWP, and the hard
branch of TRWP_hard_soft): `forward` / `backward` with the reference's positional signatures
(MPLayers/TRWP/TRWP.cpp:245-256,285-295,323-326), writing into caller-allocated tensors.

Differences a caller can see: errors raise RuntimeError instead of printing; the kernels run on
the current CUDA stream of the tensors' device; the `unary_update` / `dunary_update` scratch
tensors are accepted and ignored; the context convention follows the tensor rank instead of
`n_disp == 21`; there is no CPU path.
"""
import ctypes

import torch

from . import _lib

keep_diag = False  # TRWP_hard_soft accumulates dcontext on the diagonal, the TRWP lib does not


def _problem(n_iter, msg_shape, context, rho, enable_min_a_dir=0, enable_sgm=0, keep_diag_=0,
             context_window=0, cost_labels_first=False):
    n_dir, batch, n_cv, h, w, n_disp = msg_shape
    return _lib.Problem(int(n_iter), n_dir, batch, n_cv, h, w, n_disp,
                        _lib.context_rank(context, n_disp), int(enable_min_a_dir), int(enable_sgm),
                        int(keep_diag_), float(rho), int(context_window), 0, 0, int(bool(cost_labels_first)))


def forward(rho, n_iter, enable_min_a_dir, unary, context, edge_weights, msg, cost_final,
            msg_min_index, msg_norm_index, unary_update, label_all, context_window=0, cost_labels_first=False):
    """`context_window` (keyword, not in the reference's signature): see mpl_problem::context_window;
    0 lets the library find out by itself, which makes an inference call with a rank-1 context and
    more than 32 labels wait for the stream once.  `cost_labels_first` (keyword): cost_final is
    [B,cv,L,H,W] instead of [B,cv,H,W,L] (mpl_problem::cost_labels_first)."""
    dev = unary.device
    for t, n in ((unary, "unary"), (context, "context"), (edge_weights, "edge_weights"), (msg, "msg"),
                 (cost_final, "cost_final")):
        _lib.require(t, n, torch.float32, dev)
    for t, n in ((msg_min_index, "msg_min_index"), (msg_norm_index, "msg_norm_index"),
                 (label_all, "label_all")):
        _lib.require(t, n, torch.uint8, dev)
    if msg.dim() != 6 or tuple(unary.shape) != tuple(msg.shape[1:]):
        raise RuntimeError("msg must be [D,B,cv,H,W,L] matching unary [B,cv,H,W,L]")
    prob = _problem(n_iter, tuple(msg.shape), context, rho, enable_min_a_dir, context_window=context_window,
                    cost_labels_first=cost_labels_first)
    with torch.cuda.device(dev):
        nbytes = _lib.lib().mpl_forward_workspace_bytes(ctypes.byref(prob))
        ws = _lib.workspace(nbytes, dev)
        _lib.check(_lib.lib().mpl_trwp_forward(
            ctypes.byref(prob), _lib.ptr(unary), _lib.ptr(context), _lib.ptr(edge_weights),
            _lib.ptr(msg), _lib.ptr(cost_final), _lib.ptr(msg_min_index), _lib.ptr(msg_norm_index),
            _lib.ptr(label_all), _lib.ptr(ws), nbytes, _lib.stream_ptr(dev)))
        _lib.check_status(ws, "TRWP.forward")


def backward(rho, context, edge_weights, dcost_final, msg_min_index, msg_norm_index, dunary,
             dcontext, dedge_weights, dmsg, dunary_update, keep_diag=None, context_window=0,
             cost_labels_first=False):
    """`context_window` (keyword, not in the reference's signature): in the backward pass only a hint
    for how the scatter of a rank-1 context with more than 32 labels is split; any value gives the
    same sums."""
    dev = dcost_final.device
    for t, n in ((context, "context"), (edge_weights, "edge_weights"), (dcost_final, "dcost_final"),
                 (dunary, "dunary"), (dcontext, "dcontext"), (dedge_weights, "dedge_weights"),
                 (dmsg, "dmsg")):
        _lib.require(t, n, torch.float32, dev)
    for t, n in ((msg_min_index, "msg_min_index"), (msg_norm_index, "msg_norm_index")):
        _lib.require(t, n, torch.uint8, dev)
    if msg_min_index.dim() != 7:
        raise RuntimeError("msg_min_index must be [I,D,B,cv,H,W,L]")
    kd = globals()["keep_diag"] if keep_diag is None else keep_diag
    prob = _problem(msg_min_index.size(0), tuple(msg_min_index.shape[1:]), context, rho,
                    keep_diag_=kd, context_window=max(int(context_window), 0),
                    cost_labels_first=cost_labels_first)
    with torch.cuda.device(dev):
        nbytes = _lib.lib().mpl_backward_workspace_bytes(ctypes.byref(prob))
        ws = _lib.workspace(nbytes, dev)
        _lib.check(_lib.lib().mpl_trwp_backward(
            ctypes.byref(prob), _lib.ptr(context), _lib.ptr(edge_weights), _lib.ptr(dcost_final),
            _lib.ptr(msg_min_index), _lib.ptr(msg_norm_index), _lib.ptr(dunary), _lib.ptr(dcontext),
            _lib.ptr(dedge_weights), _lib.ptr(dmsg), _lib.ptr(ws), nbytes, _lib.stream_ptr(dev)))
        _lib.check_status(ws, "TRWP.backward")


def forward_soft(rho, n_iter, unary, context, edge_weights, msg, msg_edge_label, msg_norm_index,
                 cost_final, unary_update, label_all):
    """TRWP_hard_soft.forward_soft of the reference (MPLayers/TRWP_hard_soft/TRWP.cpp:433; argument
    order of pytorch/MP_module_hard_soft.py:44-46).  msg_edge_label [I,D,B,cv,H,W,L,L] and
    msg_norm_index [I,D,B,cv,H,W] are empty tensors in inference."""
    dev = unary.device
    for t, n in ((unary, "unary"), (context, "context"), (edge_weights, "edge_weights"), (msg, "msg"),
                 (cost_final, "cost_final"), (msg_edge_label, "msg_edge_label")):
        _lib.require(t, n, torch.float32, dev)
    for t, n in ((msg_norm_index, "msg_norm_index"), (label_all, "label_all")):
        _lib.require(t, n, torch.uint8, dev)
    if msg.dim() != 6 or tuple(unary.shape) != tuple(msg.shape[1:]):
        raise RuntimeError("msg must be [D,B,cv,H,W,L] matching unary [B,cv,H,W,L]")
    prob = _problem(n_iter, tuple(msg.shape), context, rho)
    with torch.cuda.device(dev):
        nbytes = _lib.lib().mpl_forward_workspace_bytes(ctypes.byref(prob))
        ws = _lib.workspace(nbytes, dev)
        _lib.check(_lib.lib().mpl_trwp_soft_forward(
            ctypes.byref(prob), _lib.ptr(unary), _lib.ptr(context), _lib.ptr(edge_weights), _lib.ptr(msg),
            _lib.ptr(cost_final), _lib.ptr(msg_edge_label), _lib.ptr(msg_norm_index), _lib.ptr(label_all),
            _lib.ptr(ws), nbytes, _lib.stream_ptr(dev)))
        _lib.check_status(ws, "TRWP.forward_soft")


def backward_soft(rho, dcost_final, context, edge_weights, msg_edge_label, msg_norm_index, dunary,
                  dcontext, dedge_weights, dmsg, dunary_update):
    """TRWP_hard_soft.backward_soft (MPLayers/TRWP_hard_soft/TRWP.cpp:434; argument order of
    pytorch/MP_module_hard_soft.py:95-97)."""
    dev = dcost_final.device
    for t, n in ((context, "context"), (edge_weights, "edge_weights"), (dcost_final, "dcost_final"),
                 (msg_edge_label, "msg_edge_label"), (dunary, "dunary"), (dcontext, "dcontext"),
                 (dedge_weights, "dedge_weights"), (dmsg, "dmsg")):
        _lib.require(t, n, torch.float32, dev)
    _lib.require(msg_norm_index, "msg_norm_index", torch.uint8, dev)
    if msg_norm_index.dim() != 6 or msg_edge_label.dim() != 8:
        raise RuntimeError("msg_norm_index must be [I,D,B,cv,H,W] and msg_edge_label [I,D,B,cv,H,W,L,L]")
    n_iter = msg_norm_index.size(0)
    shape = tuple(msg_norm_index.shape[1:]) + (msg_edge_label.size(-1),)
    prob = _problem(n_iter, shape, context, rho)
    with torch.cuda.device(dev):
        nbytes = _lib.lib().mpl_backward_workspace_bytes(ctypes.byref(prob))
        ws = _lib.workspace(nbytes, dev)
        _lib.check(_lib.lib().mpl_trwp_soft_backward(
            ctypes.byref(prob), _lib.ptr(context), _lib.ptr(edge_weights), _lib.ptr(dcost_final),
            _lib.ptr(msg_edge_label), _lib.ptr(msg_norm_index), _lib.ptr(dunary), _lib.ptr(dcontext),
            _lib.ptr(dedge_weights), _lib.ptr(dmsg), _lib.ptr(ws), nbytes, _lib.stream_ptr(dev)))
        _lib.check_status(ws, "TRWP.backward_soft")


def soft_weighted_message(message, message_soft_sum_norm, message_soft_sum_min_ind):
    """TRWP_hard_soft.soft_weighted_message (MPLayers/TRWP_hard_soft/TRWP.cpp:382-397; call of
    pytorch/unittest_mp.py:126).  message [T,L,L] (front, current); writes the normalised
    soft-weighted column sums [T,L] and the index of each table's minimum [T,1] (uint8)."""
    dev = message.device
    _lib.require(message, "message", torch.float32, dev)
    _lib.require(message_soft_sum_norm, "message_soft_sum_norm", torch.float32, dev)
    _lib.require(message_soft_sum_min_ind, "message_soft_sum_min_ind", torch.uint8, dev)
    if message.dim() != 3 or message.size(1) != message.size(2):
        raise RuntimeError("message must be [T,L,L], got %s" % (tuple(message.shape),))
    t, l = message.size(0), message.size(1)
    if message_soft_sum_norm.numel() != t * l or message_soft_sum_min_ind.numel() != t:
        raise RuntimeError("outputs must hold T*L values and T indices")
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().mpl_soft_weighted_message(
            _lib.ptr(message), t, l, _lib.ptr(message_soft_sum_norm), _lib.ptr(message_soft_sum_min_ind),
            _lib.stream_ptr(dev)))


def soft_weighted_message_back(dmessage_soft_sum_norm, message, message_soft_sum_min_ind, dmessage):
    """TRWP_hard_soft.soft_weighted_message_back (TRWP.cpp:399-419): writes dmessage [T,L,L]."""
    dev = message.device
    for x, n in ((dmessage_soft_sum_norm, "dmessage_soft_sum_norm"), (message, "message"), (dmessage, "dmessage")):
        _lib.require(x, n, torch.float32, dev)
    _lib.require(message_soft_sum_min_ind, "message_soft_sum_min_ind", torch.uint8, dev)
    if message.dim() != 3 or message.size(1) != message.size(2) or dmessage.shape != message.shape:
        raise RuntimeError("message and dmessage must be [T,L,L]")
    t, l = message.size(0), message.size(1)
    if dmessage_soft_sum_norm.numel() != t * l or message_soft_sum_min_ind.numel() != t:
        raise RuntimeError("dmessage_soft_sum_norm must hold T*L values and message_soft_sum_min_ind T indices")
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().mpl_soft_weighted_message_backward(
            _lib.ptr(dmessage_soft_sum_norm), _lib.ptr(message), _lib.ptr(message_soft_sum_min_ind), t, l,
            _lib.ptr(dmessage), _lib.stream_ptr(dev)))
