"""Pure-Python stand-in for `direction_sharding.CudaBackend` on CPU tensors, for tiny cases only.
TEST INFRASTRUCTURE: it lets the host logic of the direction-sharded ISGMR (who owns which
directions, what is summed and all-reduced when) run as gloo ranks without a GPU, checked against
the CPU oracle's monolithic ISGMR.  One ISGMR sweep per direction restated from
MPLayers/ISGMR/ISGMR_forward.cu:101-217 (forward) and MPLayers/ISGMR/ISGMR_backward.cu:39-130
(backward), with the chain enumeration of the library's host-side mpl_chain_geometry."""
import ctypes
import types

import numpy as np
import torch

from mplayers_b200 import _lib


def _chains(d, h, w):
    L = _lib.lib()
    L.mpl_chain_count.restype = ctypes.c_int32
    L.mpl_chain_count.argtypes = [ctypes.c_int32] * 3
    L.mpl_chain_geometry.restype = ctypes.c_int32
    L.mpl_chain_geometry.argtypes = [ctypes.c_int32] * 4 + [ctypes.POINTER(ctypes.c_int32)]
    out = []
    buf = (ctypes.c_int32 * 5)()
    for c in range(L.mpl_chain_count(d, h, w)):
        assert L.mpl_chain_geometry(d, h, w, c, buf) == 0
        out.append(tuple(buf))
    return out


def _ctx_matrix(context):
    c = context.numpy()
    l = c.shape[-1]
    if c.ndim == 1:
        return np.array([[c[abs(a - b)] for b in range(l)] for a in range(l)], np.float64)
    return np.array([[c[min(a, b), max(a, b)] for b in range(l)] for a in range(l)], np.float64)


def _owned_chains(d, p):
    """(b, v, h0, w0, n, hs, ws) of the chains of direction d that part p.part of p.parts covers: the
    even direction's chains in library order, images outermost, cut into p.parts contiguous runs;
    the odd direction walks the same lines from their other end (what the kernels do)."""
    base = _chains(d & ~1, p.h, p.w)
    total = len(base) * p.b * p.cv
    lo, hi = (0, total) if p.parts <= 1 else (total * p.part // p.parts, total * (p.part + 1) // p.parts)
    out = []
    for g in range(lo, hi):
        img, t = divmod(g, len(base))
        b, v = divmod(img, p.cv)
        h0, w0, n, hs, ws = base[t]
        if d & 1:
            h0, w0, hs, ws = h0 + (n - 1) * hs, w0 + (n - 1) * ws, -hs, -ws
        out.append((b, v, h0, w0, n, hs, ws))
    return out


class CpuBackend:
    """Per-direction tensors hold the owned slices only ([dc, ...]), indexed by d - d0."""

    def problem(self, unary, n_iter, n_dir, context, rho, enable_sgm, keep_diag=0, part=0, parts=1):
        b, cv, h, w, l = unary.shape
        return types.SimpleNamespace(n_iter=n_iter, n_dir=n_dir, b=b, cv=cv, h=h, w=w, l=l, rho=float(rho),
                                     rank=context.dim(), keep_diag=keep_diag, part=part, parts=parts)

    def forward_directions(self, p, d0, dc, aggregate, context, ew, msg_read, msg_write, min_idx, norm_idx):
        cm = _ctx_matrix(context)
        A, R, Wr = aggregate.numpy(), msg_read.numpy(), msg_write.numpy()
        for d in range(d0, d0 + dc):
            o, oi = d - d0, (d ^ 1) - d0
            for (b, v, h0, w0, n, hs, ws) in _owned_chains(d, p):
                r = np.zeros(p.l)
                for k in range(1, n):
                    fy, fx = h0 + (k - 1) * hs, w0 + (k - 1) * ws
                    y, x = h0 + k * hs, w0 + k * ws
                    uu = (A[b, v, fy, fx].astype(np.float64) - R[o, b, v, fy, fx]) * p.rho - R[oi, b, v, fy, fx]
                    e = 1.0 if ew is None else float(ew[d, b, v, y, x])
                    val = e * cm + (uu + p.rho * r)[None, :]        # [c, f]
                    best = val.min(1)
                    if min_idx is not None:
                        min_idx[o, b, v, y, x] = torch.from_numpy(
                            (p.l - 1 - np.argmin(val[:, ::-1], 1)).astype(np.uint8))   # highest index on ties
                        norm_idx[o, b, v, y, x] = int(p.l - 1 - np.argmin(best[::-1]))
                    r = best - best.min()
                    Wr[o, b, v, y, x] = r.astype(np.float32)

    def sum_directions(self, p, d0, dc, fields, out, first=0, count=None, base=None):
        flat = out.view(-1)
        count = flat.numel() - first if count is None else count
        acc = torch.zeros(count) if base is None else base.reshape(-1)[first:first + count].clone()
        for o in range(dc):
            acc += fields[o].reshape(-1)[first:first + count]
        flat[first:first + count] = acc
        return out

    def backward_workspace(self, p, dev):
        return torch.zeros(p.l, p.l, dtype=torch.float64)

    def backward_directions(self, p, d0, dc, context, ew, x, min_idx, norm_idx, scatter, dew, ws, clear):
        if clear:
            ws.zero_()
        cm = _ctx_matrix(context)
        X, Y, T = x.numpy(), scatter.numpy(), ws.numpy()
        for d in range(d0, d0 + dc):
            o = d - d0
            for (b, v, h0, w0, n, hs, wst) in _owned_chains(d, p):
                q = np.zeros(p.l)
                for k in range(n - 1, 0, -1):
                    y, xx = h0 + k * hs, w0 + k * wst
                    Y[o, b, v, y, xx] = q.astype(np.float32)
                    t = X[o, b, v, y, xx].astype(np.float64) + p.rho * q
                    t[int(norm_idx[o, b, v, y, xx])] -= t.sum()
                    idx = min_idx[o, b, v, y, xx].numpy().astype(int)
                    e = 1.0 if ew is None else float(ew[d, b, v, y, xx])
                    q = np.zeros(p.l)
                    for c in range(p.l):
                        q[idx[c]] += t[c]
                        if c != idx[c] or p.keep_diag:
                            T[c, idx[c]] += e * t[c]
                        if dew is not None:
                            dew[o, b, v, y, xx] += float(cm[c, idx[c]] * t[c])
                Y[o, b, v, h0, w0] = q.astype(np.float32)

    def combine(self, p, d0, dc, q_total, scatter, x, dunary):
        rq = p.rho * q_total
        if dunary is not None:
            dunary.add_(rq)
        for o in range(dc):
            x[o] = rq - p.rho * scatter[o] - scatter[o ^ 1]   # the partner of slice d is d ^ 1: d0 is even

    def context_finish(self, p, ws, dcontext):
        t = ws.numpy()
        out = np.zeros(tuple(dcontext.shape), np.float64)
        for c in range(p.l):
            for f in range(p.l):
                if dcontext.dim() == 2:
                    out[min(c, f), max(c, f)] += t[c, f]
                else:
                    out[abs(c - f)] += t[c, f]
        dcontext.add_(torch.from_numpy(out.astype(np.float32)))
