"""Failure detection of the staged kernels, exercised without faulting, trapping or hanging the GPU:
every device-side wait is bounded and reports through the status word of the call's workspace.
A self-test kernel waits (with a limit of a fraction of a millisecond) on an mbarrier that nothing
arrives at; it must return, the status word must carry its code, the host must turn it into an
exception -- at once in the synchronous mode the tests run in, one call later in the default
deferred mode -- and the context must stay usable.  Needs a GPU."""
import ctypes
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _selftest(ws, cycles=200_000):
    from mplayers_b200 import _lib
    rc = _lib.lib().mpl_selftest_bounded_wait(ctypes.c_void_p(ws.data_ptr()), ws.numel(), cycles,
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _lib.lib().mpl_last_error().decode()


def test_bounded_wait_gives_up_and_reports(monkeypatch):
    from mplayers_b200 import _lib
    ws = _lib.workspace(256, torch.device("cuda"))
    t0 = time.perf_counter()
    _selftest(ws)
    torch.cuda.synchronize()                      # the kernel RETURNS (no trap, no endless spin)
    assert time.perf_counter() - t0 < 5.0
    st = ctypes.c_int32(-1)
    assert _lib.lib().mpl_workspace_status(ctypes.c_void_p(ws.data_ptr()), ctypes.byref(st)) == 0
    assert st.value == 901
    # synchronous mode: the wrapper's check raises right after the call
    monkeypatch.setenv("MPL_CHECK_STATUS", "1")
    with pytest.raises(_lib.DeviceStatusError, match="901"):
        _lib.check_status(ws, "the self-test")
    # the context is intact: a real layer call still gives the oracle's result
    import gpu_runner as g
    from oracle import oracle
    rng = np.random.default_rng(0)
    unary = rng.standard_normal((1, 1, 9, 12, 21)).astype(np.float32)
    ctx = (1.0 - np.eye(21)).astype(np.float32)
    got = g.forward("TRWP", unary, ctx, None, 4, 2)
    want = oracle.forward("TRWP", unary, ctx, None, 4, 2)
    assert np.array_equal(got["cost"], want["cost"])


def test_deferred_check_raises_one_call_later(monkeypatch):
    from mplayers_b200 import _lib
    monkeypatch.delenv("MPL_CHECK_STATUS", raising=False)
    _lib.poll_status(wait=True)                   # nothing pending from earlier tests
    ws = _lib.workspace(256, torch.device("cuda"))
    _selftest(ws)
    _lib.check_status(ws, "the self-test")        # default mode: no wait, no exception yet
    with pytest.raises(_lib.DeviceStatusError, match="self-test"):
        _lib.poll_status(wait=True)
    _lib.poll_status(wait=True)                   # reported once
    # a clean call leaves nothing to report
    clean = _lib.workspace(256, torch.device("cuda"))
    clean.zero_()
    _lib.check_status(clean, "a clean call")
    _lib.poll_status(wait=True)
    monkeypatch.setenv("MPL_CHECK_STATUS", "0")
    _selftest(ws)
    _lib.check_status(ws, "unchecked")            # checking switched off
    _lib.poll_status(wait=True)


def test_backward_status_word_is_read(monkeypatch):
    """The backward's status word sits at the same offset of its workspace as the forward's and is
    checked after every backward call; here the word of a finished call is read back directly."""
    from mplayers_b200 import TRWP, _lib
    monkeypatch.setenv("MPL_CHECK_STATUS", "1")
    lib = _lib.lib()
    B, H, W, L, D, I = 1, 16, 24, 21, 4, 2
    g = torch.Generator().manual_seed(0)
    prob = _lib.Problem(I, D, B, 1, H, W, L, 2, 0, 0, 0, 0.5)
    n = lib.mpl_backward_workspace_bytes(ctypes.byref(prob))
    assert n >= 256 + L * L * 4
    ws = torch.full((n,), 0xFF, dtype=torch.uint8, device="cuda")   # garbage: the call must clear what it uses
    ctx = torch.rand(L, L, generator=g).cuda()
    ew = torch.rand(D, B, 1, H, W, generator=g).cuda()
    dcost = torch.rand(B, 1, H, W, L, generator=g).cuda()
    mi = torch.zeros(I, D, B, 1, H, W, L, dtype=torch.uint8, device="cuda")
    ni = torch.zeros(I, D, B, 1, H, W, dtype=torch.uint8, device="cuda")
    du, dc, de = torch.empty_like(dcost), torch.zeros_like(ctx), torch.zeros_like(ew)
    dmsg = torch.empty(D, B, 1, H, W, L, device="cuda")
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.mpl_trwp_backward(ctypes.byref(prob), vp(ctx), vp(ew), vp(dcost), vp(mi), vp(ni), vp(du), vp(dc),
                               vp(de), vp(dmsg), vp(ws), n, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.mpl_last_error().decode()
    st = ctypes.c_int32(-1)
    assert lib.mpl_workspace_status(vp(ws), ctypes.byref(st)) == 0
    assert st.value == 0
    assert torch.isfinite(du).all() and torch.isfinite(dc).all()
