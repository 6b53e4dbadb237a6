"""Pins the CPU oracle to the reference's own C++ CPU forward (compiled from the reference
sources by `python oracle/build.py --ref`).  Skipped where that build is absent.  The reference
CPU path ignores edge weights, so these cases use weight 1."""
import numpy as np
import pytest

from helpers import COST_RTOL, rel_err
from oracle import oracle, ref_cpu

pytestmark = pytest.mark.skipif(not ref_cpu.available(), reason="oracle/_ref not built")

CASES = [
    # mode, D, B, H, W, L, I, ctx kind
    ("TRWP", 4, 1, 16, 20, 21, 3, "sym2d"),
    ("ISGMR", 4, 2, 12, 14, 21, 3, "sym2d"),
    ("TRWP", 8, 1, 12, 15, 21, 2, "potts2d"),
    ("ISGMR", 8, 1, 12, 15, 21, 2, "potts2d"),
    ("TRWP", 16, 1, 11, 13, 21, 2, "sym2d"),
    ("ISGMR", 16, 1, 11, 13, 21, 2, "sym2d"),
    ("TRWP", 4, 1, 9, 17, 48, 2, "tl1d"),
    ("ISGMR", 8, 1, 9, 11, 64, 2, "tq1d"),
    ("TRWP", 16, 1, 9, 11, 16, 2, "tl1d"),
]


def _ctx(kind, L, rng):
    import cases
    return cases.make_context(kind, L, rng)


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_forward_matches_reference_cpu(case):
    mode, D, B, H, W, L, I, kind = case
    rng = np.random.default_rng(1000 + CASES.index(case))
    unary = rng.standard_normal((B, 1, H, W, L)).astype(np.float32)
    ctx = _ctx(kind, L, rng)
    ref = ref_cpu.forward(mode, unary, ctx, D, I, save_labels=True)
    got = oracle.forward(mode, unary, ctx, None, D, I, training=False, save_labels=True)
    assert rel_err(got["cost"], ref["cost"]) < COST_RTOL
    assert rel_err(got["msg"], ref["msg"]) < COST_RTOL
    # labels: equal except where the two best costs are within fp32 rounding of each other
    diff = got["label_all"] != ref["label_all"]
    assert diff.mean() < 1e-3
