"""The allocation-free TRWP backward entry point (mpl_trwp_backward_static) against the regular
one.  Some hosts of this library may not allocate device memory when they call it (a fully
reserved memory pool, a latency-critical section, a plugin sandbox); for them the scratch is a
fixed array inside the library.  Collected last on purpose: a failure here must not hide the
results of the other tests in a run that stops at the first failure."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(_lib, n_iter, D, B, H, W, L, rank):
    return _lib.Problem(n_iter, D, B, 1, H, W, L, rank, 0, 0, 0, 0.5)


def _run_both(seed, B, H, W, L, D, I):
    from mplayers_b200 import TRWP, _lib
    lib = _lib.lib()
    g = torch.Generator().manual_seed(seed)
    unary = torch.randn(B, 1, H, W, L, generator=g).cuda()
    a = torch.triu(2 * torch.rand(L, L, generator=g), 1)
    ctx = (a + a.t()).cuda()
    ew = (0.2 + 0.8 * torch.rand(D, B, 1, H, W, generator=g)).cuda()
    dcost = torch.rand(B, 1, H, W, L, generator=g).cuda()
    msg = torch.zeros(D, B, 1, H, W, L, device="cuda")
    cost = torch.empty_like(unary)
    mi = torch.zeros(I, D, B, 1, H, W, L, dtype=torch.uint8, device="cuda")
    ni = torch.zeros(I, D, B, 1, H, W, dtype=torch.uint8, device="cuda")
    e0 = torch.empty(0, device="cuda")
    e8 = torch.empty(0, dtype=torch.uint8, device="cuda")
    TRWP.forward(0.5, I, 0, unary, ctx, ew, msg, cost, mi, ni, e0, e8)

    # regular entry point (caller-provided workspace, allocated here by torch)
    du_a, dc_a, de_a = torch.empty_like(dcost), torch.zeros_like(ctx), torch.zeros_like(ew)
    dmsg = torch.empty(D, B, 1, H, W, L, device="cuda")
    TRWP.backward(0.5, ctx, ew, dcost, mi, ni, du_a, dc_a, de_a, dmsg, e0)

    # allocation-free entry point: every buffer is created BEFORE the call, nothing inside it
    du_b, dc_b, de_b = torch.empty_like(dcost), torch.zeros_like(ctx), torch.zeros_like(ew)
    dmsg_b = torch.empty(D, B, 1, H, W, L, device="cuda")
    prob = _problem(_lib, I, D, B, H, W, L, 2)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(du, dc, de, dm):
        rc = lib.mpl_trwp_backward_static(ctypes.byref(prob), vp(ctx), vp(ew), vp(dcost), vp(mi), vp(ni), vp(du),
                                          vp(dc), vp(de), vp(dm), stream)
        assert rc == 0, lib.mpl_last_error().decode()

    # Warm-up call: loads the kernels' code and looks the scratch array's address up.  What follows
    # must not change the device's free memory as the DRIVER counts it (torch's own counter would
    # not see an allocation made inside the library).
    call(torch.empty_like(dcost), torch.zeros_like(ctx), torch.zeros_like(ew), torch.empty_like(dmsg))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    torch_before = torch.cuda.memory_allocated()
    launches_before = lib.mpl_kernel_launches()
    call(du_b, dc_b, de_b, dmsg_b)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_allocated() == torch_before
    assert lib.mpl_kernel_launches() > launches_before      # kernels ran: not a silent no-op
    st = ctypes.c_int32(-1)
    assert lib.mpl_static_scratch_status(ctypes.byref(st)) == 0 and st.value == 0

    # ... and against the CPU oracle directly, not only against the regular entry point
    from oracle import oracle
    want = oracle.backward("TRWP", ctx.cpu().numpy(), ew.cpu().numpy(), dcost.cpu().numpy(), mi.cpu().numpy(),
                           ni.cpu().numpy())
    from helpers import assert_grad_close
    assert_grad_close(du_b.cpu().numpy(), want["dunary"], "dunary (static scratch)")
    assert_grad_close(dc_b.cpu().numpy(), want["dctx"], "dctx (static scratch)")
    assert_grad_close(de_b.cpu().numpy(), want["dew"], "dew (static scratch)")
    return (du_a, dc_a, de_a), (du_b, dc_b, de_b)


def _close(a, b, rtol=1e-4):
    a, b = a.cpu().numpy().astype(np.float64), b.cpu().numpy().astype(np.float64)
    return np.abs(a - b).max() <= rtol * max(np.abs(b).max(), 1e-30)


def test_static_scratch_backward_matches_regular_twice_in_a_row():
    # two different problems back to back: the second call finds the first call's leftovers in
    # the shared scratch and must clear what it uses
    for seed, shape in ((1, (2, 24, 32, 21, 4, 3)), (2, (1, 17, 20, 21, 8, 2))):
        ref, got = _run_both(seed, *shape)
        for r, g in zip(ref, got):
            assert _close(g, r)


def test_static_scratch_rejects_oversized_problems():
    from mplayers_b200 import _lib
    lib = _lib.lib()
    assert lib.mpl_static_scratch_bytes() == 8 << 20
    prob = _problem(_lib, 1, 4, 4, 2048, 2048, 256, 2)   # 4096 chains x 256 x 256 floats of tables
    one = ctypes.c_void_p(256)                           # never dereferenced: the size check comes first
    rc = lib.mpl_trwp_backward_static(ctypes.byref(prob), one, None, one, one, one, one, one, None, one, None)
    assert rc == 2
    msg = lib.mpl_last_error().decode()
    assert "scratch" in msg and str(8 << 20) in msg
