"""The large ISGMR configuration (8 directions, 64 labels, dense 64 x 64 context) on its own
generator: forward and backward against the CPU oracle on a 256 x 256 image (chains of up to 256
pixels in every direction class, two-labels-per-lane kernels, scatter-field bookkeeping), and a case
with more chains in one launch than 4096, where every chain must still own its partial
label-context table so that the gradient is run-to-run identical.  Needs a GPU."""
import numpy as np
import pytest

from helpers import assert_grad_close
from oracle import oracle

pytestmark = pytest.mark.gpu


def _numpy_case(cfg):
    u = cfg["unary"].permute(0, 1, 3, 4, 2).contiguous().numpy()
    e = cfg["edge_weights"].unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous().numpy()
    return u, cfg["label_context"].numpy().astype(np.float32), e


def test_large_isgmr_generator_256_vs_oracle():
    import gpu_runner as g
    from mplayers_b200 import synthetic
    cfg = synthetic.config5_large(H=256, W=256, n_iter=2)
    assert cfg["n_dir"] == 8 and cfg["unary"].shape[2] == 64 and cfg["label_context"].shape == (64, 64)
    u, ctx, e = _numpy_case(cfg)
    want = oracle.forward("ISGMR", u, ctx, e, 8, 2)
    got = g.forward("ISGMR", u, ctx, e, 8, 2)
    for key in ("cost", "msg", "norm_idx", "min_idx"):
        assert np.array_equal(got[key], want[key]), key
    rng = np.random.default_rng(9)
    dcost = rng.uniform(0, 1, size=u.shape).astype(np.float32)
    wb = oracle.backward("ISGMR", ctx, e, dcost, want["min_idx"], want["norm_idx"])
    gb = g.backward("ISGMR", ctx, e, dcost, got["min_idx"], got["norm_idx"])
    assert_grad_close(gb["dunary"], wb["dunary"], "dunary")
    assert_grad_close(gb["dctx"], wb["dctx"], "dctx")
    assert_grad_close(gb["dew"], wb["dew"], "dew")
    # the same with TRWP's sequential directions (C + P bookkeeping of the two-labels-per-lane kernel)
    want_t = oracle.forward("TRWP", u, ctx, e, 8, 1)
    got_t = g.forward("TRWP", u, ctx, e, 8, 1)
    for key in ("cost", "min_idx", "norm_idx"):
        assert np.array_equal(got_t[key], want_t[key]), key
    wt = oracle.backward("TRWP", ctx, e, dcost, want_t["min_idx"], want_t["norm_idx"])
    gt = g.backward("TRWP", ctx, e, dcost, got_t["min_idx"], got_t["norm_idx"])
    assert_grad_close(gt["dunary"], wt["dunary"], "dunary (TRWP)")
    assert_grad_close(gt["dctx"], wt["dctx"], "dctx (TRWP)")
    assert_grad_close(gt["dew"], wt["dew"], "dew (TRWP)")


def test_more_chains_than_4096_in_one_launch():
    """ISGMR backward runs all directions of an iteration in ONE launch: 400 x 400 pixels and 8
    directions are 4 x 400 + 4 x 799 = 4796 chains.  Each owns a partial table (the workspace is
    sized for it), so the label-context gradient equals the oracle's and repeats bit for bit."""
    import ctypes

    import gpu_runner as g
    from mplayers_b200 import _lib
    rng = np.random.default_rng(21)
    H = W = 400
    L, D, I = 36, 8, 1
    prob = _lib.Problem(I, D, 1, 1, H, W, L, 2, 0, 0, 0, 1.0)
    n = _lib.lib().mpl_backward_workspace_bytes(ctypes.byref(prob))
    assert n == 256 + 4796 * L * L * 4          # one table per chain of the launch
    unary = rng.standard_normal((1, 1, H, W, L)).astype(np.float32)
    a = np.triu(rng.uniform(0, 2, (L, L)), 1)
    ctx = (a + a.T).astype(np.float32)
    ew = rng.uniform(0.2, 1.0, size=(D, 1, 1, H, W)).astype(np.float32)
    dcost = rng.uniform(0, 1, size=unary.shape).astype(np.float32)
    want = oracle.forward("ISGMR", unary, ctx, ew, D, I)
    got = g.forward("ISGMR", unary, ctx, ew, D, I)
    assert np.array_equal(got["min_idx"], want["min_idx"])
    wb = oracle.backward("ISGMR", ctx, ew, dcost, want["min_idx"], want["norm_idx"])
    b1 = g.backward("ISGMR", ctx, ew, dcost, got["min_idx"], got["norm_idx"])
    b2 = g.backward("ISGMR", ctx, ew, dcost, got["min_idx"], got["norm_idx"])
    assert_grad_close(b1["dctx"], wb["dctx"], "dctx")
    assert_grad_close(b1["dunary"], wb["dunary"], "dunary")
    assert_grad_close(b1["dew"], wb["dew"], "dew")
    for key in ("dctx", "dunary", "dew"):
        assert np.array_equal(b1[key], b2[key]), key
