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
