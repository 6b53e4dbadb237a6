"""Loader for the reference's own C++ CPU extensions built by `oracle/build.py --ref` into
oracle/_ref/ (TRWP.so, ISGMR.so).  TEST INFRASTRUCTURE / CPU BASELINE ONLY.

The reference CPU path (MPLayers/TRWP/TRWP.cpp:172-243, MPLayers/ISGMR/ISGMR.cpp:190-298) is
forward only, ignores edge weights, saves no indices, reads the context as a [D,L,L] stack
(matrix `dir` for direction `dir`; upper-triangle read when L == 21, first row as a 1-D function
otherwise) and runs OpenMP with a fixed 16 threads (tools/cpp/utils.h:17).
"""
import importlib.util
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_mods = {}


def available():
    return all(os.path.exists(os.path.join(_HERE, "_ref", n + ".so")) for n in ("TRWP", "ISGMR"))


def _load(name):
    if name not in _mods:
        import torch  # noqa: F401  (the extension links against libtorch)
        path = os.path.join(_HERE, "_ref", name + ".so")
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mods[name] = mod
    return _mods[name]


def context_stack(ctx, n_dir):
    """[D,L,L] tensor the reference CPU path expects, from a [L] function or [L,L] matrix."""
    ctx = np.asarray(ctx, np.float32)
    L = ctx.shape[-1]
    if ctx.ndim == 1:
        mat = np.zeros((L, L), np.float32)
        mat[0] = ctx          # the non-21-label path reads context[|c-f|] = row 0
    else:
        mat = ctx
    return np.ascontiguousarray(np.broadcast_to(mat, (n_dir, L, L)))


def forward(mode, unary, ctx, n_dir, n_iter, save_labels=False):
    """Runs the reference CPU forward.  Returns dict(cost, msg, label_all)."""
    import torch
    u = torch.from_numpy(np.ascontiguousarray(unary, np.float32))
    b, cv, h, w, l = u.shape
    c = torch.from_numpy(context_stack(ctx, n_dir))
    ew = torch.ones(n_dir, b, cv, h, w)
    msg = torch.zeros(n_dir, b, cv, h, w, l)
    cost = torch.zeros(b, cv, h, w, l)
    e8 = torch.empty(0, dtype=torch.uint8)
    lab = torch.zeros(n_iter, b, cv, h, w, dtype=torch.uint8) if save_labels else e8
    uu = torch.zeros(b, cv, h, w, l)
    if mode == "TRWP":
        _load("TRWP").forward(0.5, int(n_iter), 0, u, c, ew, msg, cost, e8, e8, uu, lab)
    else:
        mu = torch.zeros(n_dir, b, cv, h, w, l)
        _load("ISGMR").forward(0, 1.0, int(n_iter), 0, u, c, ew, msg, cost, e8, e8, uu, mu, lab)
    return dict(cost=cost.numpy(), msg=msg.numpy(), label_all=lab.numpy() if save_labels else None)
