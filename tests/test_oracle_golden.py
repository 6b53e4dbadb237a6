"""Pins the CPU oracle (oracle/mp_oracle.c) to golden vectors produced by the reference's own
pure-PyTorch autograd implementation (tests/golden/make_golden.py).  CPU only."""
import os

import numpy as np
import pytest

import cases
from helpers import COST_RTOL, GRAD_RTOL, rel_err
from oracle import oracle

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", [n for n in cases.CASES if cases.is_soft(n)])
def test_soft_oracle_matches_reference_golden(name):
    """Soft (expected-value) TRWP: costs, the saved edge values and normalisation indices, and the
    three gradients against the reference's PyTorch implementation with enable_soft_weight."""
    inp = cases.make_inputs(name)
    gold = np.load(os.path.join(GOLD, name + ".npz"))
    fwd = oracle.forward_soft(inp["unary"], inp["ctx"], inp["ew"], inp["n_dir"], inp["n_iter"])
    assert rel_err(fwd["cost"], gold["cost"]) < COST_RTOL
    assert np.array_equal(fwd["norm_idx"], gold["norm_idx"])
    # edge values of pixels without a predecessor are never written by the extension
    visited = gold["edge_label"] != 0
    assert np.abs(fwd["edge_label"] - gold["edge_label"])[visited].max() < COST_RTOL * np.abs(gold["edge_label"]).max()
    bwd = oracle.backward_soft(inp["ctx"], inp["ew"], inp["dcost"], fwd["edge_label"], fwd["norm_idx"])
    assert rel_err(bwd["dunary"], gold["dunary"]) < GRAD_RTOL
    assert rel_err(bwd["dew"], gold["dew"]) < GRAD_RTOL
    assert rel_err(bwd["dctx"], gold["dctx"]) < GRAD_RTOL


@pytest.mark.parametrize("name", [n for n in cases.CASES if not cases.is_soft(n)])
def test_oracle_matches_reference_golden(name):
    inp = cases.make_inputs(name)
    gold = np.load(os.path.join(GOLD, name + ".npz"))
    fwd = oracle.forward(inp["mode"], inp["unary"], inp["ctx"], inp["ew"], inp["n_dir"],
                         inp["n_iter"], training=True)
    assert rel_err(fwd["cost"], gold["cost"]) < COST_RTOL
    if "min_idx" in gold.files:
        # float64 reference vs float32 oracle: identical indices except where two candidates
        # are closer than fp32 resolution; the seeded small cases have none.
        assert np.array_equal(fwd["norm_idx"], gold["norm_idx"])
        assert np.array_equal(fwd["min_idx"], gold["min_idx"])
    for keep_diag in (False, True):
        bwd = oracle.backward(inp["mode"], inp["ctx"], inp["ew"], inp["dcost"], fwd["min_idx"],
                              fwd["norm_idx"], keep_diag=keep_diag)
        assert rel_err(bwd["dunary"], gold["dunary"]) < GRAD_RTOL
        assert rel_err(bwd["dew"], gold["dew"]) < GRAD_RTOL
        want = gold["dctx"].copy()
        if keep_diag:
            if want.ndim == 2:
                want[np.diag_indices_from(want)] = gold["dctx_diag"]
            else:
                want[0] = gold["dctx_diag"][0]
        assert rel_err(bwd["dctx"], want) < GRAD_RTOL


def test_tie_audit_counts_only_non_ties():
    """oracle.audit_ties: an index that differs from the oracle's is accepted only when its
    candidate has exactly the minimum's value.  Integer-valued inputs make exact ties frequent."""
    rng = np.random.default_rng(0)
    L = 8
    unary = rng.integers(0, 3, size=(1, 1, 6, 7, L)).astype(np.float32)
    ctx = np.minimum(np.arange(L), 2).astype(np.float32)
    fwd = oracle.forward("TRWP", unary, ctx, None, 4, 2)
    assert oracle.audit_ties("TRWP", unary, ctx, None, 4, 2, fwd["min_idx"]) == (0, 0)
    # an arbitrary other index is counted, and reported as a non-tie unless its value happens to tie
    wrong = fwd["min_idx"].copy()
    wrong[0, 0, 0, 0, 2, 3, 1] = (wrong[0, 0, 0, 0, 2, 3, 1] + 1) % L
    seen, bad = oracle.audit_ties("TRWP", unary, ctx, None, 4, 2, wrong)
    assert seen == 1 and bad in (0, 1)
    # a constant unary makes every candidate of the first step equal: any index is a tie there
    flat = np.zeros((1, 1, 3, 4, 4), np.float32)
    f2 = oracle.forward("ISGMR", flat, np.zeros(4, np.float32), None, 4, 1)
    alt = np.zeros_like(f2["min_idx"])          # lowest index everywhere
    seen, bad = oracle.audit_ties("ISGMR", flat, np.zeros(4, np.float32), None, 4, 1, alt)
    assert bad == 0 and seen == int((alt != f2["min_idx"]).sum()) and seen > 0
