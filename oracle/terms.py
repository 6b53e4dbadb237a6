"""CPU restatement (numpy) of the reference's input builders -- test infrastructure, never
imported by the product.

  stereo_data_cost   computeDSI, MPLayers/aux/aux.cpp:6-91
  gradient_cues      computeCues, aux.cpp:93-158 (+ the compaction of auxPy.cpp:86-99)
  smoothness_context computeSmoothnessContext, aux.cpp:160-214 (float CostType, as setup.py builds it)
  edge_weights       getEdgeShift, utils/edge_weights.py:45-111, and the threshold/penalty rule of
                     MPLayers/extra_exp_edge_weights.py:115-121 ("cue_penalty")

Pinned by tests/golden/terms_*.npz: outputs of the reference's own aux.cpp (compiled unmodified by
oracle/build.py --ref-terms around a stand-in image container) and of its utils/edge_weights.py
imported as is, on seeded synthetic images (tests/golden/make_terms_golden.py).
"""
import numpy as np

STEPS = [(0, 1), (0, -1), (1, 0), (-1, 0), (1, 1), (-1, -1), (1, -1), (-1, 1), (1, 2), (-1, -2),
         (2, 1), (-2, -1), (2, -1), (-2, 1), (1, -2), (-1, 2)]
REDUCING = ("superpixel_edge", "kernel_cue_real", "kernel_cue_binary", "threshold", "cue_penalty")


def _logf(x):
    """Single-precision log of the C library, element by element (numpy's own float32 log rounds
    differently in the last place for some arguments)."""
    import ctypes
    import ctypes.util
    libm = ctypes.CDLL(ctypes.util.find_library("m") or "libm.so.6")
    libm.logf.restype = ctypes.c_float
    libm.logf.argtypes = [ctypes.c_float]
    return np.array([libm.logf(float(v)) for v in x.ravel()], dtype=np.float32).reshape(x.shape)


def _half_sample(im):
    """centre, min and max over {centre, (centre+left)/2, (centre+right)/2}, integer division."""
    c = im
    l = c.copy()
    r = c.copy()
    l[:, 1:] = (c[:, 1:] + c[:, :-1]) // 2
    r[:, :-1] = (c[:, :-1] + c[:, 1:]) // 2
    return c, np.minimum(c, np.minimum(l, r)), np.maximum(c, np.maximum(l, r))


def stereo_data_cost(left, right, n_labels, birchfield=1, squared=0, trunc=255):
    """left, right uint8 [H,W,C]; returns float32 [H,W,n_labels]."""
    H, W, nB = left.shape
    nc = min(3, nB)
    worst = nc * (255 * 255 if squared else 255)
    maxsum = trunc * trunc if squared else nc * abs(trunc)
    bad = min(worst, maxsum)
    a = left[:, :, :nc].astype(np.int64)
    b = right[:, :, :nc].astype(np.int64)
    ac, alo, ahi = _half_sample(a)
    bc, blo, bhi = _half_sample(b)
    out = np.full((H, W, n_labels), bad, dtype=np.int64)
    for d in range(min(n_labels, W)):
        s1 = slice(d, W)
        s2 = slice(0, W - d)
        if birchfield:
            di1 = np.maximum(0, np.maximum(ac[:, s1] - bhi[:, s2], blo[:, s2] - ac[:, s1]))
            di2 = np.maximum(0, np.maximum(bc[:, s2] - ahi[:, s1], alo[:, s1] - bc[:, s2]))
            diff = np.minimum(di1, di2)
        else:
            diff = np.abs(ac[:, s1] - bc[:, s2])
        if squared:
            diff = diff * diff
        out[:, d:, d] = np.minimum(diff.sum(axis=2), maxsum)
    return out.astype(np.float32)


def gradient_cues(img, grad_thresh, grad_penalty, compact=False):
    H, W, nB = img.shape
    nc = min(3, nB)
    thr = grad_thresh * nc * grad_thresh
    a = img[:, :, :nc].astype(np.int64)
    right = np.concatenate([a[:, 1:], a[:, -1:]], axis=1)
    down = np.concatenate([a[1:], a[-1:]], axis=0)
    sx = ((a - right) ** 2).sum(axis=2)
    sy = ((a - down) ** 2).sum(axis=2)
    hc = np.where(sx < thr, grad_penalty, 1).astype(np.float32)
    vc = np.where(sy < thr, grad_penalty, 1).astype(np.float32)
    if not compact:
        return hc, vc
    return hc[:, :W - 1].reshape(1, -1).copy(), vc[:H - 1].T.reshape(1, -1).copy()


def smoothness_context(n_labels, method, smoothness_max):
    f = np.float32
    smax = f(smoothness_max)
    idx = np.arange(n_labels, dtype=np.float32)
    value = (idx[:, None] - idx[None, :]).astype(np.float32)
    if method == "L":
        return np.abs(value)
    if method == "Q":
        return value * value
    if method == "TL":
        return np.minimum(np.abs(value), smax)
    if method == "TQ":
        return np.minimum(value * value, smax * smax)
    if method == "Cauchy":
        t = (value.astype(np.float64) / np.float64(smax)).astype(np.float32)
        lg = _logf((f(1) + t * t).astype(np.float32))   # std::log(float) of the C library
        return (0.5 * np.float64(smax) * np.float64(smax) * lg.astype(np.float64)).astype(np.float32)
    if method == "Huber":
        return np.where(np.abs(value) <= smax, value * value,
                        f(2) * smax * np.abs(value) - smax * smax).astype(np.float32)
    raise ValueError(method)


def edge_weights(edge_mode, image, n_dirs, sigma=10.0, threshold=0.0, penalty=0.0):
    """image float32 [B,C,H,W]; returns [n_dirs,B,Cout,H,W], Cout = 1 for the REDUCING modes."""
    f = np.float32
    B, C, H, W = image.shape
    reduced = edge_mode in REDUCING
    out = np.zeros((n_dirs, B, 1 if reduced else C, H, W), dtype=np.float32)
    for d in range(n_dirs):
        hs, ws = STEPS[d]
        if abs(hs) >= H or abs(ws) >= W:
            continue
        th = slice(max(hs, 0), H + min(hs, 0))
        tw = slice(max(ws, 0), W + min(ws, 0))
        sh = slice(max(-hs, 0), H - max(hs, 0))
        sw = slice(max(-ws, 0), W - max(ws, 0))
        cur = image[:, :, th, tw]
        front = image[:, :, sh, sw]
        diff = np.abs(cur - front).astype(np.float32)
        if edge_mode == "gt_edge":
            diff = np.where(cur == 255, f(1), diff)
            g = (diff == 0).astype(np.float32)
        elif edge_mode == "canny":
            diff = np.where(cur == 1, f(1), diff)
            g = f(1) - diff
        elif edge_mode in ("sobel", "edge_net_sigmoid"):
            g = f(1) - diff
        elif edge_mode == "edge_net":
            g = np.exp(-diff).astype(np.float32)
        elif edge_mode == "superpixel_edge":
            g = (diff.sum(axis=1, keepdims=True) == 0).astype(np.float32)
        elif reduced:
            acc = np.zeros_like(diff[:, 0])
            for c in range(C):
                acc = acc + diff[:, c] * diff[:, c]
            mean = (acc / f(C))[:, None]
            if edge_mode == "threshold":
                g = (mean < f(threshold)).astype(np.float32) * f(penalty)
            elif edge_mode == "cue_penalty":
                g = np.where(mean < f(threshold), f(penalty), f(1)).astype(np.float32)
            else:
                g = np.exp(mean / f(-2.0 * sigma * sigma)).astype(np.float32)
                if edge_mode == "kernel_cue_binary":
                    cut = f(0.8) * f(g.astype(np.float64).mean())
                    g = (g >= cut).astype(np.float32)
        else:
            g = front
        out[d, :, :, th, tw] = g
    return out


def soft_weighted_message(message):
    """Stand-alone soft-weighted message op (MPLayers/TRWP_hard_soft/TRWP_swbp.cu:135-186), in
    float64.  message [T,L(front),L(current)] -> (norm [T,L], min_ind [T] uint8, soft [T,L]).
    The same quantity is written with torch ops in pytorch/unittest_mp.py:131-139."""
    m = np.asarray(message, np.float64)
    e = np.exp(-(m - m.min(axis=1, keepdims=True)))
    prob = e / e.sum(axis=1, keepdims=True)
    soft = (prob * m).sum(axis=1)
    L = m.shape[1]
    ind = (L - 1 - np.argmin(soft[:, ::-1], axis=1)).astype(np.uint8)   # highest index among equal minima
    return soft - np.take_along_axis(soft, ind[:, None].astype(np.int64), 1), ind, soft


def soft_weighted_message_back(dnorm, message, min_ind):
    """TRWP_swbp.cu:188-245: dmessage[t,f,c] = d[t,c] * prob[t,f,c] * (1 - message[t,f,c] + soft[t,c])
    with d = dnorm, minus sum_c dnorm at c = min_ind[t]."""
    m = np.asarray(message, np.float64)
    d = np.asarray(dnorm, np.float64).copy()
    e = np.exp(-(m - m.min(axis=1, keepdims=True)))
    prob = e / e.sum(axis=1, keepdims=True)
    soft = (prob * m).sum(axis=1)
    d[np.arange(m.shape[0]), np.asarray(min_ind).reshape(-1).astype(np.int64)] -= d.sum(axis=1)
    return d[:, None, :] * prob * (1.0 - m + soft[:, None, :])
