"""Energy of labellings on the grid MRF the layers minimise (evaluation helper).

With `enable_saving_label` a forward call returns the labelling after every iteration
(`label_all`); the reference turns those into energy-versus-iteration curves with a MATLAB script
(tools/matlab/MRF/calEnergy.m, fed by MPLayers/main.py:322-333).  `labeling_energy` computes the
same two sums on the GPU for any number of labellings at once."""
import ctypes

import torch

from . import _lib


def labeling_energy(unary, label_context, edge_weights, labels, n_dir):
    """unary [B,cv,H,W,L] f32; label_context [L] or [L,L]; edge_weights [D,B,cv,H,W] or None;
    labels [I,B,cv,H,W] (or [B,cv,H,W]) u8.  Returns a float64 tensor [I,2] on the device:
    (unary energy, pairwise energy) of each labelling; their sum is the MRF energy."""
    dev = unary.device
    if labels.dim() == 4:
        labels = labels.unsqueeze(0)
    _lib.require(unary, "unary", torch.float32, dev)
    _lib.require(label_context, "label_context", torch.float32, dev)
    _lib.require(labels, "labels", torch.uint8, dev)
    if edge_weights is not None:
        _lib.require(edge_weights, "edge_weights", torch.float32, dev)
    b, cv, h, w, l = unary.shape
    if tuple(labels.shape[1:]) != (b, cv, h, w):
        raise RuntimeError("labels must be [I,B,cv,H,W] matching unary [B,cv,H,W,L]")
    prob = _lib.Problem(0, int(n_dir), b, cv, h, w, l, _lib.context_rank(label_context, l), 0, 0, 0, 1.0)
    out = torch.zeros(labels.size(0), 2, dtype=torch.float64, device=dev)
    with torch.cuda.device(dev):
        n = _lib.lib().mpl_energy_workspace_bytes(ctypes.byref(prob))
        ws = _lib.workspace(n, dev)
        _lib.check(_lib.lib().mpl_labeling_energy(
            ctypes.byref(prob), _lib.ptr(unary), _lib.ptr(label_context), _lib.ptr(edge_weights),
            _lib.ptr(labels), int(labels.size(0)), _lib.ptr(out), _lib.ptr(ws), n, _lib.stream_ptr(dev)))
    return out


def save_energy_mat(file_path, unary, label_context, label_all, n_iter, n_dir, rho, p_func, p_weight, trunct,
                    min_a_dir=False):
    """Writes the `.mat` file the reference's driver hands to its MATLAB energy script
    (MPLayers/main.py:322-333): the run's parameters, `unary` [H,W,L], `label_context` [L,L,D] and
    the per-iteration labellings `seg_all` [H,W,I] (uint8).  unary [B=1,cv=1,H,W,L] or [H,W,L];
    label_context [D,L,L] or [L,L]; label_all [I,1,1,H,W] or [I,H,W].  Needs scipy."""
    import numpy as np
    import scipy.io as scio
    u = unary.detach().reshape(unary.shape[-3:]).cpu().numpy()
    ctx = label_context.detach().cpu()
    ctx = ctx.unsqueeze(0).repeat(int(n_dir), 1, 1) if ctx.dim() == 2 else ctx
    seg = label_all.detach().reshape(label_all.size(0), *label_all.shape[-2:]).permute(1, 2, 0).cpu().numpy()
    scio.savemat(file_path, {'n_iter': n_iter, 'n_dir': n_dir, 'rho': rho, 'p_func': p_func,
                             'n_disp': u.shape[-1], 'p_weight': p_weight, 'trunct': trunct,
                             'min_a_dir': int(min_a_dir), 'unary': u,
                             'label_context': ctx.permute(1, 2, 0).numpy(),
                             'seg_all': seg.astype(np.uint8)})
