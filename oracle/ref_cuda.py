"""Loader for the reference's own CUDA extensions, recompiled unmodified for sm_100a by
`oracle/build.py --ref-cuda` into oracle/_ref/cuda/ (TRWP.so, ISGMR.so).
TEST INFRASTRUCTURE / SIDE-BY-SIDE BASELINE ONLY: the GPU implementation this library replaces,
run on the same device for parity at sizes no CPU checker reaches and for a like-for-like time.

The call sequence mirrors what the reference's autograd functions do around the extension
(pytorch/MP_module.py:17-86 for TRWP, :89-161 for ISGMR): every tensor is allocated by the
caller, zero-initialised where the kernels accumulate, and passed positionally.  The reference
reads the context as an [L, L] upper triangle exactly when L == 21 and as a 1-D function of
|c - f| otherwise (MPLayers/TRWP/TRWP_forward.cu:132-135), so only those two forms are offered.
Its kernels address with 32-bit offsets: callers keep I*D*B*cv*H*W*L below 2**32.
"""
import importlib.util
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_DIR = os.path.join(_HERE, "_ref", "cuda")
_mods = {}


def available(mode="TRWP"):
    return os.path.exists(os.path.join(_DIR, mode + ".so"))


def _load(name):
    if name not in _mods:
        import torch  # noqa: F401  (the extension links against libtorch)
        spec = importlib.util.spec_from_file_location(name, os.path.join(_DIR, name + ".so"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mods[name] = mod
    return _mods[name]


def expressible(n_disp, ctx_ndim, n_iter, n_dir, n_pix):
    """True when the reference kernels can run this problem as stated (see the module text)."""
    if (n_disp == 21) != (ctx_ndim == 2):
        return False
    return n_iter * n_dir * n_pix * n_disp < 2 ** 32


def forward(mode, unary, ctx, edge_weights, n_dir, n_iter, rho, training=True, save_labels=False,
            enable_min_a_dir=False, enable_sgm=False):
    """unary [B,cv,H,W,L], ctx [L,L] (L == 21) or [L], edge_weights [D,B,cv,H,W] or None: CUDA
    tensors.  Returns dict(cost, msg, min_idx, norm_idx, label_all) of CUDA tensors."""
    import torch
    b, cv, h, w, l = unary.shape
    if not expressible(l, ctx.dim(), n_iter, n_dir, b * cv * h * w):
        raise ValueError("the reference CUDA kernels cannot express this problem")
    msg = unary.new_zeros(n_dir, b, cv, h, w, l)
    cost = unary.new_zeros(b, cv, h, w, l)
    uu = unary.new_zeros(b, cv, h, w, l)
    e8 = torch.empty(0, dtype=torch.uint8)
    if training:
        mi = unary.new_zeros(n_iter, n_dir, b, cv, h, w, l, dtype=torch.uint8)
        ni = unary.new_zeros(n_iter, n_dir, b, cv, h, w, dtype=torch.uint8)
    else:
        mi, ni = e8, e8
    lab = unary.new_zeros(n_iter, b, cv, h, w, dtype=torch.uint8) if save_labels else e8
    ew = edge_weights if edge_weights is not None else unary.new_ones(n_dir, b, cv, h, w)
    if mode == "TRWP":
        _load("TRWP").forward(float(rho), int(n_iter), int(enable_min_a_dir), unary, ctx, ew, msg,
                              cost, mi, ni, uu, lab)
    else:
        mu = unary.new_zeros(n_dir, b, cv, h, w, l)
        _load("ISGMR").forward(int(enable_sgm), float(rho), int(n_iter), int(enable_min_a_dir),
                               unary, ctx, ew, msg, cost, mi, ni, uu, mu, lab)
    return dict(cost=cost, msg=msg, min_idx=mi, norm_idx=ni, label_all=lab, edge_weights=ew)


def backward(mode, ctx, edge_weights, dcost, min_idx, norm_idx, rho, enable_sgm=False):
    """Returns (dunary, dcontext, dedge_weights) CUDA tensors; edge_weights as given to forward
    (the all-ones tensor forward() made when there were none)."""
    n_iter, n_dir, b, cv, h, w, l = min_idx.shape
    dcost = dcost.contiguous()
    dun = dcost.new_zeros(b, cv, h, w, l)
    dmsg = dcost.new_zeros(n_dir, b, cv, h, w, l)
    duu = dcost.new_zeros(b, cv, h, w, l)
    dew = dcost.new_zeros(n_dir, b, cv, h, w)
    dctx = dcost.new_zeros(l, l) if l == 21 else dcost.new_zeros(l)
    if mode == "TRWP":
        _load("TRWP").backward(float(rho), ctx, edge_weights, dcost, min_idx, norm_idx, dun, dctx,
                               dew, dmsg, duu)
    else:
        dmu = dcost.new_zeros(n_dir, b, cv, h, w, l)
        _load("ISGMR").backward(int(enable_sgm), float(rho), ctx, edge_weights, dcost, min_idx,
                                norm_idx, dun, dctx, dew, dmsg, duu, dmu)
    return dun, dctx, dew
