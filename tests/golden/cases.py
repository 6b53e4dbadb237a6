"""Seeded inputs of the golden-vector cases (shared by make_golden.py and the tests).

Inputs are regenerated from the seed; only the reference's OUTPUTS are stored in the .npz
fixtures next to this file.
"""
import numpy as np

# name -> (mode, D, B, H, W, L, I, ctx_kind, seed)
CASES = {
    "trwp_d4_small":   ("TRWP", 4, 2, 7, 9, 5, 3, "sym2d", 11),
    "isgmr_d4_small":  ("ISGMR", 4, 2, 7, 9, 5, 3, "sym2d", 12),
    "trwp_d8_small":   ("TRWP", 8, 1, 6, 8, 6, 2, "sym2d", 13),
    "isgmr_d8_small":  ("ISGMR", 8, 1, 6, 8, 6, 2, "sym2d", 14),
    "trwp_d16_small":  ("TRWP", 16, 1, 7, 8, 4, 2, "sym2d", 15),
    "isgmr_d16_small": ("ISGMR", 16, 1, 7, 8, 4, 2, "sym2d", 16),
    "trwp_d4_tl1d":    ("TRWP", 4, 1, 6, 10, 12, 2, "tl1d", 17),
    "isgmr_d8_tq1d":   ("ISGMR", 8, 1, 6, 7, 40, 2, "tq1d", 18),
    # the reference's CPU-runnable configuration: B1 D4 64x64 L21 I5, Potts, E~U[0.5,1], seed 0
    "trwp_config1":    ("TRWP", 4, 1, 64, 64, 21, 5, "potts2d", 0),
    "isgmr_config1":   ("ISGMR", 4, 1, 64, 64, 21, 5, "potts2d", 0),
    # soft (expected-value) TRWP: names start with "trwp_soft"
    "trwp_soft_d4_small":  ("TRWP", 4, 2, 7, 9, 5, 3, "sym2d", 21),
    "trwp_soft_d8_small":  ("TRWP", 8, 1, 6, 8, 6, 2, "sym2d", 22),
    "trwp_soft_d4_tl1d":   ("TRWP", 4, 1, 6, 10, 12, 2, "tl1d", 23),
}


def is_soft(name):
    return name.startswith("trwp_soft")


def make_context(kind, L, rng):
    if kind == "potts2d":
        return (1.0 - np.eye(L)).astype(np.float32)
    if kind == "sym2d":
        a = rng.uniform(0.0, 2.0, size=(L, L))
        a = np.triu(a, 1)
        return (a + a.T).astype(np.float32)
    k = np.arange(L, dtype=np.float64)
    if kind == "tl1d":   # truncated linear, slope 1, truncation 2
        return np.minimum(k, 2.0).astype(np.float32)
    if kind == "tq1d":   # truncated quadratic
        return (0.05 * np.minimum(k * k, 30.0)).astype(np.float32)
    raise ValueError(kind)


def make_inputs(name):
    """unary [B,1,H,W,L], ctx ([L,L] symmetric or [L]), edge_weights [D,B,1,H,W], dcost [B,1,H,W,L]."""
    mode, D, B, H, W, L, I, kind, seed = CASES[name]
    rng = np.random.default_rng(seed)
    unary = rng.standard_normal((B, 1, H, W, L)).astype(np.float32)
    ctx = make_context(kind, L, rng)
    if name.endswith("config1"):
        ew = rng.uniform(0.5, 1.0, size=(D, B, 1, H, W)).astype(np.float32)
    else:
        ew = rng.uniform(0.5, 1.5, size=(D, B, 1, H, W)).astype(np.float32)
    dcost = rng.uniform(0.0, 1.0, size=(B, 1, H, W, L)).astype(np.float32)
    return dict(mode=mode, n_dir=D, n_iter=I, unary=unary, ctx=ctx, ew=ew, dcost=dcost)
