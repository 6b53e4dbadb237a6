"""ctypes binding of libmplayers_b200.so (the C ABI declared in include/mplayers_b200.h).

There is no CPU implementation behind these calls: if the library has not been built, loading
fails with an ImportError that says how to build it, and the compute entry points fail on a
machine without a CUDA device.
"""
import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmplayers_b200.so")

MPL_OK = 0


class Problem(ctypes.Structure):
    """struct mpl_problem of include/mplayers_b200.h"""
    _fields_ = [(n, ctypes.c_int32) for n in
                ("n_iter", "n_dir", "batch", "n_cv", "height", "width", "n_disp", "context_rank",
                 "enable_min_a_dir", "enable_sgm", "keep_diag")] + [("rho", ctypes.c_float),
                                                                   ("context_window", ctypes.c_int32),
                                                                   ("chain_part", ctypes.c_int32),
                                                                   ("chain_parts", ctypes.c_int32),
                                                                   ("cost_labels_first", ctypes.c_int32)]


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
        L.mpl_analyze_context.restype = ctypes.c_int
        L.mpl_analyze_context.argtypes = [pp, vp, vp, ctypes.POINTER(ctypes.c_int32), vp, sz, vp]
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
        L.mpl_sum_directions_range.restype = ctypes.c_int
        L.mpl_sum_directions_range.argtypes = [pp, i32, i32, vp, ctypes.c_float, vp, vp, ctypes.c_int64,
                                               ctypes.c_int64, vp]
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
        L.mpl_workspace_status.restype = ctypes.c_int
        L.mpl_workspace_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int32)]
        L.mpl_static_scratch_status.restype = ctypes.c_int
        L.mpl_static_scratch_status.argtypes = [ctypes.POINTER(ctypes.c_int32)]
        L.mpl_workspace_status_offset.restype = sz
        L.mpl_selftest_bounded_wait.restype = ctypes.c_int
        L.mpl_selftest_bounded_wait.argtypes = [vp, sz, ctypes.c_int64, vp]
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


class DeviceStatusError(RuntimeError):
    """A kernel recorded that one of its bounded waits gave up; the outputs of that call are invalid."""


_STATUS_WHAT = {101: "forward staging", 102: "forward staging", 111: "forward staging", 112: "forward staging",
                121: "forward staging", 122: "forward staging", 131: "forward staging", 132: "forward staging",
                141: "backward staging", 151: "backward staging", 201: "backward staging", 202: "backward staging",
                901: "self-test wait"}


def _raise_status(code, what):
    raise DeviceStatusError("mplayers_b200: device status %d after %s (%s: a bounded wait timed out; the "
                            "outputs of that call are invalid)" % (code, what, _STATUS_WHAT.get(code, "unknown")))


class _StatusWatch:
    """Deferred check of the device status words.  After every call the word is copied to pinned
    host memory on the call's stream, without waiting; the copies that have completed are inspected
    at the next library call (and by `poll_status`), so a wait that gave up surfaces as an exception
    one call later instead of passing silently, and no call synchronises for it."""
    SLOTS = 64

    def __init__(self):
        self.host = None
        self.pending = []   # (slot, event, what)
        self.free = list(range(self.SLOTS))
        self.lock = threading.Lock()   # ranks may be threads of one process

    def watch(self, ws, what):
        with self.lock:
            self._watch(ws, what)

    def poll(self, wait=False, wait_oldest=False):
        with self.lock:
            self._poll(wait, wait_oldest)

    def _watch(self, ws, what):
        if self.host is None:
            self.host = torch.zeros(self.SLOTS, dtype=torch.int32).pin_memory()
        self._poll()
        if not self.free:           # every slot in flight: wait for the oldest
            self._poll(wait_oldest=True)
        slot = self.free.pop()
        off = int(lib().mpl_workspace_status_offset())
        self.host[slot:slot + 1].copy_(ws[off:off + 4].view(torch.int32), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(ws.device))
        self.pending.append((slot, ev, what))

    def _poll(self, wait=False, wait_oldest=False):
        keep, bad = [], None
        for i, (slot, ev, what) in enumerate(self.pending):
            if wait or (wait_oldest and i == 0):
                ev.synchronize()
            if ev.query():
                code = int(self.host[slot])
                self.free.append(slot)
                if code != 0 and bad is None:
                    bad = (code, what)
            else:
                keep.append((slot, ev, what))
        self.pending = keep
        if bad is not None:
            _raise_status(*bad)


_watch = _StatusWatch()


def poll_status(wait=False):
    """Raises DeviceStatusError if an earlier call's kernels recorded a wait that gave up.  With
    wait=True it first waits for every call watched so far (a natural place: where the training
    loop synchronises anyway, e.g. when it reads the loss)."""
    _watch.poll(wait=wait)


def check_status(ws, what="a forward call"):
    """Status word of the call that just used workspace `ws`.  MPL_CHECK_STATUS=1: wait for the call
    and raise at once if a bounded wait gave up (synchronises; what the tests run with).
    MPL_CHECK_STATUS=0: no check.  Default: deferred check, see _StatusWatch."""
    mode = os.environ.get("MPL_CHECK_STATUS", "")
    if mode == "0":
        return
    if mode == "1":
        st = ctypes.c_int32(0)
        check(lib().mpl_workspace_status(ctypes.c_void_p(ws.data_ptr()), ctypes.byref(st)))
        if st.value != 0:
            _raise_status(st.value, what)
        return
    if torch.cuda.is_current_stream_capturing():
        return  # a captured call cannot be watched from the host; read the word after the replay
    _watch.watch(ws, what)


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


def analyze_context(context, edge_weights=None, n_pixels=0, n_dir=2):
    """mpl_problem::context_window for a rank-1 context [L] (and, optionally, edge weights
    [D,B,cv,H,W]): R > 0 if the windowed evaluation is exact, else -1.  Waits for the device."""
    if context.dim() != 1:
        return -1
    dev = context.device
    L = context.numel()
    if edge_weights is not None and edge_weights.numel():
        n_dir, b, cv, h, w = edge_weights.shape
    else:
        edge_weights, b, cv, h, w = None, 1, 1, 1, max(int(n_pixels), 1)
    prob = Problem(1, int(n_dir), b, cv, h, w, L, 1, 0, 0, 0, 1.0, 0)
    out = ctypes.c_int32(-1)
    with torch.cuda.device(dev):
        n = lib().mpl_forward_workspace_bytes(ctypes.byref(prob))
        ws = workspace(n, dev)
        check(lib().mpl_analyze_context(ctypes.byref(prob), ptr(context.contiguous()), ptr(edge_weights),
                                        ctypes.byref(out), ptr(ws), n, stream_ptr(dev)))
    return int(out.value)


def workspace(nbytes, device):
    return torch.empty(int(nbytes), dtype=torch.uint8, device=device)


def stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
