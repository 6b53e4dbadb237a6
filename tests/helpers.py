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


def audit_index_mismatches(min_a, min_b, unary_like_values=None):
    """Fraction of differing saved indices (used where an exact-tie audit is done elsewhere)."""
    return float((min_a != min_b).mean())
