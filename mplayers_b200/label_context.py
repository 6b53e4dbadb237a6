"""Builder of the pairwise `label_context` parameter, import-compatible with the reference's
utils/label_context.py:6-90 (same arguments, same three return values).

2-D [L,L] for 21 classes (only the upper triangle is ever read by the layers), 1-D [L] otherwise;
modes Potts / TL / TQ / NPotts, optional truncation, scaled by `mpnet_term_weight`.
"""
import numpy as np
import torch
import torch.nn as nn


def create_label_context(args, enable_seg=None, enable_symmetric=False):
    n = args.n_classes
    if enable_seg is None:
        enable_seg = (n == 21)
    mode = args.mpnet_smoothness_mode
    trunc_v = args.mpnet_smoothness_trunct_value
    trunc_loc = args.mpnet_smoothness_trunct_loc

    if enable_seg:
        gap = np.arange(n)[None, :] - np.arange(n)[:, None]          # right - left
        if enable_symmetric:
            gap = np.abs(gap)
        lc = np.zeros((n, n), dtype=np.float32)
        pos = gap > 0
        if mode in ("Potts", "potts"):
            if args.mpnet_smoothness_train != "sigmoid":
                lc[pos] = 1
        elif mode == "TL":
            lc[pos] = gap[pos]
        elif mode == "TQ":
            lc[pos] = gap[pos].astype(np.float32) ** 2
        elif mode == "NPotts":
            lc[np.arange(n), np.arange(n)] = -1
        if trunc_v >= 0:
            if trunc_loc >= 0:
                # the reference compares the gap of the LAST (left, right) pair visited by its
                # construction loop, i.e. a constant, against the truncation location
                # (utils/label_context.py:40-48); reproduced as is.
                last_gap = gap[n - 1, n - 1]
                if last_gap >= trunc_loc:
                    lc = np.minimum(lc, trunc_v)
            else:
                lc = np.minimum(lc, trunc_v)
    else:
        d = np.arange(n, dtype=np.float32)
        lc = np.zeros((n,), dtype=np.float32)
        if mode in ("Potts", "potts"):
            if args.mpnet_smoothness_train != "sigmoid":
                lc[1:] = 1
        elif mode == "TL":
            lc = d.copy()
        elif mode == "TQ":
            lc = d ** 2
        elif mode == "NPotts":
            lc[0] = -1
        if trunc_v >= 0:
            if trunc_loc >= 0:
                sel = d >= trunc_loc
                lc[sel] = np.minimum(lc[sel], trunc_v)
            else:
                lc = np.minimum(lc, trunc_v)

    label_context = torch.from_numpy(np.ascontiguousarray(lc, dtype=np.float32)) * args.mpnet_term_weight
    if getattr(args, "enable_cuda", False) and not label_context.is_cuda:
        label_context = label_context.cuda()
    enable_grad = args.mpnet_smoothness_train in {"softmax", "sigmoid", "on"}
    label_context = nn.Parameter(label_context, requires_grad=enable_grad)

    if label_context.dim() == 2:
        label_context_loc = np.triu_indices(n, k=1)
        label_context_diag_loc = [range(n), range(n)]
    else:
        label_context_loc = range(1, n)
        label_context_diag_loc = range(1)
    return label_context, label_context_loc, label_context_diag_loc
