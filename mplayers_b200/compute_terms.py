"""Stereo MRF terms on the GPU: matching cost volume, gradient cues, pairwise table.

Counterpart of the reference's `compute_terms` extension (MPLayers/aux/auxPy.cpp:9-112, driven by
MPLayers/test_compute_terms.py:13-56).  `compute_terms_py(param)` keeps the reference's call
(paths in, (data_cost, RGB, smoothness_context, param) out); `compute_all_terms` is the same work
on images that are already tensors.  The cost volume comes out as [H,W,L], which is the layers'
unary [B=1,cv=1,H,W,L] without a permute.
"""
import torch

from . import _lib


class MRFParams():
    """MPLayers/test_compute_terms.py:13-26."""

    def __init__(self, left_img_path, right_img_path, context, n_disp, grad_thresh, grad_penalty, truncated):
        self.left_img_path = left_img_path
        self.right_img_path = right_img_path
        self.context = context
        self.grad_thresh = grad_thresh
        self.grad_penalty = grad_penalty
        self.truncated = truncated
        self.n_disp = n_disp
        self.height = 0
        self.width = 0
        self.n_channels = 0
        self.data_type = torch.float32


def _u8_image(t, name):
    _lib.require(t, name, torch.uint8)
    if t.dim() == 2:
        t = t.unsqueeze(2)
    if t.dim() != 3:
        raise RuntimeError("%s must be [H,W] or [H,W,C] uint8, got %s" % (name, tuple(t.shape)))
    return t


def stereo_data_cost(left, right, n_disp, birchfield=1, squared_diffs=0, trunc_diffs=255):
    """computeDSI (MPLayers/aux/aux.cpp:6-91).  left, right: CUDA uint8 [H,W,C] (or [H,W]).
    Returns float32 [H,W,n_disp]."""
    left, right = _u8_image(left, "left"), _u8_image(right, "right")
    if left.shape != right.shape:
        raise RuntimeError("image shapes don't match: %s, %s" % (tuple(left.shape), tuple(right.shape)))
    h, w, c = left.shape
    dev = left.device
    out = torch.empty(h, w, int(n_disp), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().mpl_stereo_data_cost(_lib.ptr(left), _lib.ptr(right), h, w, c, int(n_disp),
                                                   int(birchfield), int(squared_diffs), int(trunc_diffs),
                                                   _lib.ptr(out), _lib.stream_ptr(dev)))
    return out


def gradient_cues(image, grad_thresh, grad_penalty, compact=False):
    """computeCues (aux.cpp:93-158).  Returns (h_cue, v_cue): [H,W] each, or with compact=True the
    vectors the reference hands to Python, [1,H*(W-1)] and [1,(H-1)*W] (auxPy.cpp:86-99)."""
    image = _u8_image(image, "image")
    h, w, c = image.shape
    dev = image.device
    if compact:
        hc = torch.zeros(1, h * (w - 1), dtype=torch.float32, device=dev)
        vc = torch.zeros(1, (h - 1) * w, dtype=torch.float32, device=dev)
    else:
        hc = torch.empty(h, w, dtype=torch.float32, device=dev)
        vc = torch.empty(h, w, dtype=torch.float32, device=dev)
    if compact and (h < 2 or w < 2):
        raise RuntimeError("compact cues need an image of at least 2x2")
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().mpl_gradient_cues(_lib.ptr(image), h, w, c, int(grad_thresh), int(grad_penalty),
                                                int(bool(compact)), _lib.ptr(hc), _lib.ptr(vc),
                                                _lib.stream_ptr(dev)))
    return hc, vc


def smoothness_context(n_disp, method, smoothness_max, device="cuda"):
    """computeSmoothnessContext (aux.cpp:160-214): [n_disp,n_disp] table for "L", "Q", "TL", "TQ",
    "Cauchy" or "Huber"."""
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("smoothness_context builds on a CUDA device: this library has no CPU path")
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    out = torch.empty(int(n_disp), int(n_disp), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().mpl_smoothness_context(int(n_disp), str(method).encode(), float(smoothness_max),
                                                     _lib.ptr(out), _lib.stream_ptr(dev)))
    return out


def compute_all_terms(left, right, context, grad_thresh, grad_penalty, truncated, n_disp):
    """ComputerAllTerms (auxPy.cpp:9-112) on device images: returns (data_cost [H,W,L],
    RGB [H,W,C] float32 copy of `left`, h_cue [1,H*(W-1)], v_cue [1,(H-1)*W],
    smoothness_context [L,L]); Birchfield-Tomasi, absolute differences, truncation 255 as there."""
    left = _u8_image(left, "left")
    data_cost = stereo_data_cost(left, right, n_disp, birchfield=1, squared_diffs=0, trunc_diffs=255)
    h_cue, v_cue = gradient_cues(left, grad_thresh, grad_penalty, compact=True)
    ctx = smoothness_context(n_disp, context, truncated, device=left.device)
    return data_cost, left.float(), h_cue, v_cue, ctx


def _read_image(path):
    """uint8 [H,W] or [H,W,C] in the channel order OpenCV's imread gives (the reference build reads
    with it, auxPy.cpp:30)."""
    import numpy as np
    try:
        import cv2
        img = cv2.imread(path, cv2.IMREAD_UNCHANGED)
        if img is None:
            raise RuntimeError("cannot read image " + path)
    except ImportError:
        from PIL import Image
        img = np.asarray(Image.open(path))
        if img.ndim == 3:
            img = img[:, :, ::-1]
    if img.dtype != np.uint8:
        raise RuntimeError("%s: 8-bit images only" % path)
    return torch.from_numpy(np.ascontiguousarray(img))


def compute_terms_py(param, device="cuda"):
    """MPLayers/test_compute_terms.py:29-56: reads the two images of `param`, fills
    param.height/width/n_channels and returns (data_cost [H,W,L], RGB [H,W,C], smoothness_context,
    param) as CUDA tensors."""
    left = _read_image(param.left_img_path).to(device)
    right = _read_image(param.right_img_path).to(device)
    if left.dim() == 2:
        param.height, param.width = left.shape
        param.n_channels = 1
    else:
        param.height, param.width, param.n_channels = left.shape
    data_cost, rgb, _, _, ctx = compute_all_terms(left, right, param.context, param.grad_thresh,
                                                  param.grad_penalty, param.truncated, param.n_disp)
    return data_cost, rgb, ctx, param
