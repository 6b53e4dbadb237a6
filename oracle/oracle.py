"""numpy front end of the CPU oracle (oracle/mp_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the bench's CPU-baseline legs import this module; the
shipped package never does.  Layouts are the reference extension's:
unary/cost [B,cv,H,W,L], messages [D,B,cv,H,W,L], edge weights [D,B,cv,H,W],
msg_min_index [I,D,B,cv,H,W,L] u8, msg_norm_index [I,D,B,cv,H,W] u8.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


class _Problem(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("mode", "enable_sgm", "enable_min_a_dir", "keep_diag", "ctx_rank", "n_iter",
                 "n_dir", "batch", "n_cv", "height", "width", "n_disp")] + \
               [("rho", ctypes.c_float), ("n_threads", ctypes.c_int)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "libmp_oracle.so")
        src = os.path.join(_HERE, "mp_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            import importlib.util
            spec = importlib.util.spec_from_file_location("_mpo_build", os.path.join(_HERE, "build.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_oracle(force=True)
        _lib = ctypes.CDLL(path)
        _lib.mpo_forward.restype = ctypes.c_int
        _lib.mpo_backward.restype = ctypes.c_int
        _lib.mpo_max_threads.restype = ctypes.c_int
        _lib.mpo_forward_soft.restype = ctypes.c_int
        _lib.mpo_backward_soft.restype = ctypes.c_int
    return _lib


def _p(a, typ):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(typ))


def _problem(mode, unary, n_dir, n_iter, ctx, rho, enable_sgm, enable_min_a_dir, keep_diag, n_threads):
    b, cv, h, w, l = unary.shape
    assert ctx.ndim in (1, 2) and ctx.shape[-1] == l
    if rho is None:
        rho = 0.5 if mode == "TRWP" else 1.0
    if n_threads is None:
        n_threads = lib().mpo_max_threads()
    return _Problem({"TRWP": 0, "ISGMR": 1}[mode], int(enable_sgm), int(enable_min_a_dir),
                    int(keep_diag), ctx.ndim, n_iter, n_dir, b, cv, h, w, l, float(rho), n_threads)


def forward(mode, unary, ctx, edge_weights, n_dir, n_iter, rho=None, training=True,
            save_labels=False, enable_sgm=False, enable_min_a_dir=False, n_threads=None, msg_init=None):
    """Returns dict(cost, msg, min_idx, norm_idx, label_all).  msg_init: messages to start from
    (default zeros, as the reference allocates them)."""
    unary = np.ascontiguousarray(unary, np.float32)
    ctx = np.ascontiguousarray(ctx, np.float32)
    b, cv, h, w, l = unary.shape
    if edge_weights is None:
        edge_weights = np.ones((n_dir, b, cv, h, w), np.float32)
    edge_weights = np.ascontiguousarray(edge_weights, np.float32)
    assert edge_weights.shape == (n_dir, b, cv, h, w)
    prob = _problem(mode, unary, n_dir, n_iter, ctx, rho, enable_sgm, enable_min_a_dir, 0, n_threads)
    msg = np.zeros((n_dir, b, cv, h, w, l), np.float32)
    if msg_init is not None:
        msg[...] = msg_init
    cost = np.zeros_like(unary)
    mi = np.zeros((n_iter, n_dir, b, cv, h, w, l), np.uint8) if training else None
    ni = np.zeros((n_iter, n_dir, b, cv, h, w), np.uint8) if training else None
    lab = np.zeros((n_iter, b, cv, h, w), np.uint8) if save_labels else None
    rc = lib().mpo_forward(ctypes.byref(prob), _p(unary, ctypes.c_float), _p(ctx, ctypes.c_float),
                           _p(edge_weights, ctypes.c_float), _p(msg, ctypes.c_float),
                           _p(cost, ctypes.c_float), _p(mi, ctypes.c_uint8), _p(ni, ctypes.c_uint8),
                           _p(lab, ctypes.c_uint8))
    if rc:
        raise RuntimeError("mpo_forward failed with code %d" % rc)
    return dict(cost=cost, msg=msg, min_idx=mi, norm_idx=ni, label_all=lab)


def audit_ties(mode, unary, ctx, edge_weights, n_dir, n_iter, alt_min_idx, rho=None, n_threads=None):
    """Tie audit of another implementation's saved argmin indices (layout of min_idx).  Runs the
    forward pass and, wherever `alt_min_idx` differs from the index computed here, compares the value
    of that candidate with the minimum bit for bit.  Returns (differing entries, differing entries
    that are NOT exact ties); the second number must be 0."""
    unary = np.ascontiguousarray(unary, np.float32)
    ctx = np.ascontiguousarray(ctx, np.float32)
    b, cv, h, w, l = unary.shape
    if edge_weights is None:
        edge_weights = np.ones((n_dir, b, cv, h, w), np.float32)
    edge_weights = np.ascontiguousarray(edge_weights, np.float32)
    alt = np.ascontiguousarray(alt_min_idx, np.uint8)
    assert alt.shape == (n_iter, n_dir, b, cv, h, w, l)
    prob = _problem(mode, unary, n_dir, n_iter, ctx, rho, 0, 0, 0, n_threads)
    msg = np.zeros((n_dir, b, cv, h, w, l), np.float32)
    cost = np.zeros_like(unary)
    mi = np.zeros(alt.shape, np.uint8)
    ni = np.zeros(alt.shape[:-1], np.uint8)
    out = (ctypes.c_longlong * 2)()
    lib().mpo_forward_audit.restype = ctypes.c_int
    rc = lib().mpo_forward_audit(ctypes.byref(prob), _p(unary, ctypes.c_float), _p(ctx, ctypes.c_float),
                                 _p(edge_weights, ctypes.c_float), _p(msg, ctypes.c_float),
                                 _p(cost, ctypes.c_float), _p(mi, ctypes.c_uint8), _p(ni, ctypes.c_uint8),
                                 _p(alt, ctypes.c_uint8), out)
    if rc:
        raise RuntimeError("mpo_forward_audit failed with code %d" % rc)
    return int(out[0]), int(out[1])


def backward(mode, ctx, edge_weights, dcost, min_idx, norm_idx, rho=None, enable_sgm=False,
             keep_diag=False, n_threads=None):
    """Returns dict(dunary, dctx, dew)."""
    dcost = np.ascontiguousarray(dcost, np.float32)
    ctx = np.ascontiguousarray(ctx, np.float32)
    n_iter, n_dir = min_idx.shape[:2]
    b, cv, h, w, l = dcost.shape
    if edge_weights is None:
        edge_weights = np.ones((n_dir, b, cv, h, w), np.float32)
    edge_weights = np.ascontiguousarray(edge_weights, np.float32)
    prob = _problem(mode, dcost, n_dir, n_iter, ctx, rho, enable_sgm, 0, keep_diag, n_threads)
    dunary = np.zeros_like(dcost)
    dctx = np.zeros_like(ctx)
    dew = np.zeros_like(edge_weights)
    rc = lib().mpo_backward(ctypes.byref(prob), _p(ctx, ctypes.c_float),
                            _p(edge_weights, ctypes.c_float), _p(dcost, ctypes.c_float),
                            _p(np.ascontiguousarray(min_idx), ctypes.c_uint8),
                            _p(np.ascontiguousarray(norm_idx), ctypes.c_uint8),
                            _p(dunary, ctypes.c_float), _p(dctx, ctypes.c_float),
                            _p(dew, ctypes.c_float))
    if rc:
        raise RuntimeError("mpo_backward failed with code %d" % rc)
    return dict(dunary=dunary, dctx=dctx, dew=dew)


def forward_soft(unary, ctx, edge_weights, n_dir, n_iter, rho=0.5, training=True, save_labels=False,
                 n_threads=None):
    """Soft (expected-value) TRWP.  Returns dict(cost, msg, edge_label, norm_idx, label_all);
    edge_label [I,D,B,cv,H,W,L,L] holds entry [f][c] for even directions and [c][f] for odd ones."""
    unary = np.ascontiguousarray(unary, np.float32)
    ctx = np.ascontiguousarray(ctx, np.float32)
    b, cv, h, w, l = unary.shape
    if edge_weights is None:
        edge_weights = np.ones((n_dir, b, cv, h, w), np.float32)
    edge_weights = np.ascontiguousarray(edge_weights, np.float32)
    prob = _problem("TRWP", unary, n_dir, n_iter, ctx, rho, 0, 0, 1, n_threads)
    msg = np.zeros((n_dir, b, cv, h, w, l), np.float32)
    cost = np.zeros_like(unary)
    el = np.zeros((n_iter, n_dir, b, cv, h, w, l, l), np.float32) if training else None
    ni = np.zeros((n_iter, n_dir, b, cv, h, w), np.uint8) if training else None
    lab = np.zeros((n_iter, b, cv, h, w), np.uint8) if save_labels else None
    rc = lib().mpo_forward_soft(ctypes.byref(prob), _p(unary, ctypes.c_float), _p(ctx, ctypes.c_float),
                                _p(edge_weights, ctypes.c_float), _p(msg, ctypes.c_float),
                                _p(cost, ctypes.c_float), _p(el, ctypes.c_float), _p(ni, ctypes.c_uint8),
                                _p(lab, ctypes.c_uint8))
    if rc:
        raise RuntimeError("mpo_forward_soft failed with code %d" % rc)
    return dict(cost=cost, msg=msg, edge_label=el, norm_idx=ni, label_all=lab)


def backward_soft(ctx, edge_weights, dcost, edge_label, norm_idx, rho=0.5, n_threads=None):
    """Returns dict(dunary, dctx, dew); dctx includes the diagonal (c == f)."""
    dcost = np.ascontiguousarray(dcost, np.float32)
    ctx = np.ascontiguousarray(ctx, np.float32)
    n_iter, n_dir = norm_idx.shape[:2]
    b, cv, h, w, l = dcost.shape
    if edge_weights is None:
        edge_weights = np.ones((n_dir, b, cv, h, w), np.float32)
    edge_weights = np.ascontiguousarray(edge_weights, np.float32)
    prob = _problem("TRWP", dcost, n_dir, n_iter, ctx, rho, 0, 0, 1, n_threads)
    dunary = np.zeros_like(dcost)
    dctx = np.zeros_like(ctx)
    dew = np.zeros_like(edge_weights)
    rc = lib().mpo_backward_soft(ctypes.byref(prob), _p(ctx, ctypes.c_float), _p(edge_weights, ctypes.c_float),
                                 _p(dcost, ctypes.c_float), _p(np.ascontiguousarray(edge_label), ctypes.c_float),
                                 _p(np.ascontiguousarray(norm_idx), ctypes.c_uint8), _p(dunary, ctypes.c_float),
                                 _p(dctx, ctypes.c_float), _p(dew, ctypes.c_float))
    if rc:
        raise RuntimeError("mpo_backward_soft failed with code %d" % rc)
    return dict(dunary=dunary, dctx=dctx, dew=dew)


def max_threads():
    return lib().mpo_max_threads()
