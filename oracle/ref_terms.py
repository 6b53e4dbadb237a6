"""ctypes loader of oracle/_ref/libref_terms.so: the reference's own aux.cpp (computeDSI,
computeCues, computeSmoothnessContext) compiled unmodified by `python oracle/build.py --ref-terms`.
Test infrastructure only."""
import ctypes
import os

import numpy as np

LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libref_terms.so")
_lib = None


def available():
    return os.path.exists(LIB)


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB)
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def stereo_data_cost(left, right, n_labels, birchfield=1, squared=0, trunc=255):
    left, right = np.ascontiguousarray(left), np.ascontiguousarray(right)
    H, W, C = left.shape
    out = np.empty((H, W, n_labels), dtype=np.float32)
    _load().ref_compute_dsi(_p(left), _p(right), H, W, C, n_labels, birchfield, squared, trunc, _p(out))
    return out


def gradient_cues(img, grad_thresh, grad_penalty):
    img = np.ascontiguousarray(img)
    H, W, C = img.shape
    hc, vc = np.empty((H, W), dtype=np.float32), np.empty((H, W), dtype=np.float32)
    _load().ref_compute_cues(_p(img), H, W, C, grad_thresh, grad_penalty, _p(hc), _p(vc))
    return hc, vc


def smoothness_context(n_labels, method, smoothness_max):
    out = np.zeros((n_labels, n_labels), dtype=np.float32)
    _load().ref_smoothness_context(n_labels, method.encode(), ctypes.c_float(smoothness_max), _p(out))
    return out
