"""ctypes binding of libmplayers_b200.so (the C ABI declared in include/mplayers_b200.h).

There is no CPU implementation behind these calls: if the library has not been built, loading
fails with an ImportError that says how to build it, and the compute entry points fail on a
machine without a CUDA device.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmplayers_b200.so")

MPL_OK = 0


class Problem(ctypes.Structure):
    """struct mpl_problem of include/mplayers_b200.h"""
    _fields_ = [(n, ctypes.c_int32) for n in
                ("n_iter", "n_dir", "batch", "n_cv", "height", "width", "n_disp", "context_rank",
                 "enable_min_a_dir", "enable_sgm", "keep_diag")] + [("rho", ctypes.c_float)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "libmplayers_b200.so is not built; run `python -m mplayers_b200.build` "
                "(needs nvcc; the kernels target sm_100a).  There is no CPU fallback.")
        L = ctypes.CDLL(LIB_PATH)
        vp, sz = ctypes.c_void_p, ctypes.c_size_t
        pp = ctypes.POINTER(Problem)
        L.mpl_forward_workspace_bytes.restype = sz
        L.mpl_forward_workspace_bytes.argtypes = [pp]
        L.mpl_backward_workspace_bytes.restype = sz
        L.mpl_backward_workspace_bytes.argtypes = [pp]
        L.mpl_trwp_forward.restype = ctypes.c_int
        L.mpl_trwp_forward.argtypes = [pp] + [vp] * 9 + [sz, vp]
        L.mpl_trwp_backward.restype = ctypes.c_int
        L.mpl_trwp_backward.argtypes = [pp] + [vp] * 10 + [sz, vp]
        L.mpl_isgmr_forward.restype = ctypes.c_int
        L.mpl_isgmr_forward.argtypes = [pp] + [vp] * 10 + [sz, vp]
        L.mpl_isgmr_backward.restype = ctypes.c_int
        L.mpl_isgmr_backward.argtypes = [pp] + [vp] * 11 + [sz, vp]
        i32 = ctypes.c_int32
        L.mpl_isgmr_forward_directions.restype = ctypes.c_int
        L.mpl_isgmr_forward_directions.argtypes = [pp, i32, i32] + [vp] * 8 + [sz, vp]
        L.mpl_sum_directions.restype = ctypes.c_int
        L.mpl_sum_directions.argtypes = [pp, i32, i32, vp, ctypes.c_float, vp, vp, vp]
        L.mpl_isgmr_backward_directions.restype = ctypes.c_int
        L.mpl_isgmr_backward_directions.argtypes = [pp, i32, i32] + [vp] * 8 + [sz, i32, vp]
        L.mpl_isgmr_backward_combine.restype = ctypes.c_int
        L.mpl_isgmr_backward_combine.argtypes = [pp, i32, i32] + [vp] * 5
        L.mpl_backward_context_finish.restype = ctypes.c_int
        L.mpl_backward_context_finish.argtypes = [pp, vp, sz, vp, vp]
        L.mpl_trwp_soft_forward.restype = ctypes.c_int
        L.mpl_trwp_soft_forward.argtypes = [pp] + [vp] * 9 + [sz, vp]
        L.mpl_trwp_soft_backward.restype = ctypes.c_int
        L.mpl_trwp_soft_backward.argtypes = [pp] + [vp] * 10 + [sz, vp]
        L.mpl_scores_to_costs.restype = ctypes.c_int
        L.mpl_scores_to_costs.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp]
        L.mpl_scores_to_costs_backward.restype = ctypes.c_int
        L.mpl_scores_to_costs_backward.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp]
        L.mpl_negate_lhw_to_hwl.restype = ctypes.c_int
        L.mpl_negate_lhw_to_hwl.argtypes = [vp, vp, i32, i32, i32, i32, vp]
        L.mpl_negate_hwl_to_lhw.restype = ctypes.c_int
        L.mpl_negate_hwl_to_lhw.argtypes = [vp, vp, i32, i32, i32, i32, vp]
        for name in ("mpl_permute_lhw_to_hwl", "mpl_permute_hwl_to_lhw"):
            getattr(L, name).restype = ctypes.c_int
            getattr(L, name).argtypes = [vp, vp, i32, i32, i32, i32, vp]
        L.mpl_energy_workspace_bytes.restype = sz
        L.mpl_energy_workspace_bytes.argtypes = [pp]
        L.mpl_labeling_energy.restype = ctypes.c_int
        L.mpl_labeling_energy.argtypes = [pp] + [vp] * 4 + [ctypes.c_int32, vp, vp, sz, vp]
        f32 = ctypes.c_float
        L.mpl_soft_weighted_message.restype = ctypes.c_int
        L.mpl_soft_weighted_message.argtypes = [vp, ctypes.c_int64, i32, vp, vp, vp]
        L.mpl_soft_weighted_message_backward.restype = ctypes.c_int
        L.mpl_soft_weighted_message_backward.argtypes = [vp, vp, vp, ctypes.c_int64, i32, vp, vp]
        L.mpl_stereo_data_cost.restype = ctypes.c_int
        L.mpl_stereo_data_cost.argtypes = [vp, vp] + [i32] * 7 + [vp, vp]
        L.mpl_gradient_cues.restype = ctypes.c_int
        L.mpl_gradient_cues.argtypes = [vp] + [i32] * 6 + [vp, vp, vp]
        L.mpl_smoothness_context.restype = ctypes.c_int
        L.mpl_smoothness_context.argtypes = [i32, ctypes.c_char_p, f32, vp, vp]
        L.mpl_edge_mode.restype = i32
        L.mpl_edge_mode.argtypes = [ctypes.c_char_p]
        L.mpl_edge_mode_channels.restype = i32
        L.mpl_edge_mode_channels.argtypes = [i32, i32]
        L.mpl_edge_weights.restype = ctypes.c_int
        L.mpl_edge_weights.argtypes = [i32, vp] + [i32] * 5 + [f32] * 3 + [vp, vp, sz, vp]
        L.mpl_trwp_backward_static.restype = ctypes.c_int
        L.mpl_trwp_backward_static.argtypes = [pp] + [vp] * 10
        L.mpl_static_scratch_bytes.restype = sz
        L.mpl_forward_status.restype = ctypes.c_int
        L.mpl_forward_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int32)]
        L.mpl_last_error.restype = ctypes.c_char_p
        L.mpl_kernel_launches.restype = ctypes.c_int64
        L.mpl_version.restype = ctypes.c_int32
        _lib = L
    return _lib


def kernel_launches():
    return int(lib().mpl_kernel_launches())


def check(rc):
    if rc != MPL_OK:
        raise RuntimeError("mplayers_b200: " + lib().mpl_last_error().decode())


def check_status(ws):
    """With MPL_CHECK_STATUS=1 in the environment: wait for the forward call that used workspace
    `ws` and raise if a kernel recorded that one of its bounded waits gave up.  Off by default
    because it synchronises."""
    if os.environ.get("MPL_CHECK_STATUS") != "1":
        return
    st = ctypes.c_int32(0)
    check(lib().mpl_forward_status(ctypes.c_void_p(ws.data_ptr()), ctypes.byref(st)))
    if st.value != 0:
        raise RuntimeError("mplayers_b200: device status %d (a staging wait timed out)" % st.value)


def ptr(t):
    """Device pointer of a tensor; None and empty tensors map to NULL."""
    if t is None or t.numel() == 0:
        return None
    return ctypes.c_void_p(t.data_ptr())


def require(t, name, dtype, device=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError("%s must be a torch.Tensor" % name)
    if t.numel() == 0:
        return
    if t.dtype != dtype:
        raise RuntimeError("%s must be %s, got %s" % (name, dtype, t.dtype))
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)  # tools/cuda/cudaUtils.hpp:10
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor: this library has no CPU path" % name)
    if device is not None and t.device != device:
        raise RuntimeError("%s is on %s, expected %s" % (name, t.device, device))


def context_rank(context, n_disp):
    """Context convention from the tensor rank.

    [L] -> rank 1 (ctx[|c-f|]); [L,L] -> rank 2 (upper-triangle read).  A [D,L,L] stack, which the
    reference's energy-minimisation driver passes (MPLayers/main.py:178), is read the way the
    reference CUDA kernels read it: its first L floats as a 1-D function, or its first matrix when
    L == 21 (MPLayers/TRWP/TRWP_forward.cu:101,132-135).
    """
    if context.dim() == 1:
        rank = 1
    elif context.dim() == 2:
        rank = 2
    elif context.dim() == 3:
        rank = 2 if n_disp == 21 else 1
    else:
        raise RuntimeError("context must have 1, 2 or 3 dimensions")
    need = n_disp * n_disp if rank == 2 else n_disp
    if context.numel() < need or context.size(-1) != n_disp:
        raise RuntimeError("context shape %s does not match n_disp=%d" % (tuple(context.shape), n_disp))
    return rank


def workspace(nbytes, device):
    return torch.empty(int(nbytes), dtype=torch.uint8, device=device)


def stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
