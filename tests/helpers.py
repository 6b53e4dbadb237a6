"""Comparison helpers shared by the parity tests."""
import numpy as np

COST_RTOL = 1e-5   # forward costs: relative to the largest |cost| of the case
GRAD_RTOL = 1e-4   # gradients: relative to the largest |gradient| of the tensor


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    scale = max(np.abs(b).max(), 1e-30)
    return np.abs(a - b).max() / scale


def ctx_matrix(ctx):
    """Dense [L,L] view of either context convention (symmetric read of the upper triangle)."""
    ctx = np.asarray(ctx)
    L = ctx.shape[-1]
    if ctx.ndim == 1:
        k = np.abs(np.arange(L)[:, None] - np.arange(L)[None, :])
        return ctx[k]
    up = np.triu(ctx)
    return up + np.triu(ctx, 1).T


CELL_RTOL = 2e-3   # gradients, entry by entry, on entries above CELL_FLOOR of the tensor's largest
CELL_FLOOR = 1e-2


def assert_grad_close(got, want, name="gradient", rtol=GRAD_RTOL, cell_rtol=CELL_RTOL, cell_floor=CELL_FLOOR):
    """Max-norm check (the stated gradient tolerance) plus a relative check entry by entry on the entries
    that are not small: the label-context gradient spans orders of magnitude between cells, and a
    max-norm alone would not see a wrong small cell."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    assert np.isfinite(got).all(), name + ": non-finite entries"
    scale = max(np.abs(want).max(), 1e-30)
    err = np.abs(got - want)
    assert err.max() / scale < rtol, "%s: max-norm error %.3g" % (name, err.max() / scale)
    big = np.abs(want) >= cell_floor * scale
    if big.any():
        per = err[big] / np.abs(want[big])
        assert per.max() < cell_rtol, "%s: entry-wise relative error %.3g" % (name, per.max())


def audit_index_ties(mode, unary, ctx, ew, n_dir, n_iter, got_idx, want_idx, rho=None):
    """Every saved argmin index that differs from the oracle's must be an exact tie: the oracle
    re-runs the forward pass and compares, at each differing entry, the value of the other index's
    candidate with the minimum bit for bit (oracle.audit_ties).  Returns the number of differing
    entries (all of them audited)."""
    from oracle import oracle
    n_diff = int((np.asarray(got_idx) != np.asarray(want_idx)).sum())
    if n_diff == 0:
        return 0
    seen, not_ties = oracle.audit_ties(mode, unary, ctx, ew, n_dir, n_iter, got_idx, rho=rho)
    assert seen == n_diff, "audit saw %d differing indices, the comparison %d" % (seen, n_diff)
    assert not_ties == 0, "%d of %d differing argmin indices are not exact ties" % (not_ties, n_diff)
    return n_diff
