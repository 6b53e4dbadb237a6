"""Parity of the CUDA path (called through the C ABI) with the CPU oracle and with the golden
vectors of the reference implementation.  Needs a GPU."""
import os

import numpy as np
import pytest

import cases
from helpers import COST_RTOL, GRAD_RTOL, assert_grad_close, audit_index_ties, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _gpu():
    import gpu_runner
    return gpu_runner


def _check_backward(mode, ctx, ew, dcost, fwd, **kw):
    g = _gpu()
    for keep_diag in (False, True):
        want = oracle.backward(mode, ctx, ew, dcost, fwd["min_idx"], fwd["norm_idx"], keep_diag=keep_diag, **kw)
        got = g.backward(mode, ctx, ew, dcost, fwd["min_idx"], fwd["norm_idx"], keep_diag=keep_diag, **kw)
        assert_grad_close(got["dunary"], want["dunary"], "dunary")
        assert_grad_close(got["dctx"], want["dctx"], "dctx")   # entry by entry as well as in max-norm
        if ew is not None:
            assert_grad_close(got["dew"], want["dew"], "dew")
    return got


@pytest.mark.parametrize("name", [n for n in cases.CASES if not cases.is_soft(n)])
def test_golden_cases(name):
    """CUDA vs golden vectors of the reference's PyTorch implementation, and vs the oracle."""
    g = _gpu()
    inp = cases.make_inputs(name)
    gold = np.load(os.path.join(GOLD, name + ".npz"))
    got = g.forward(inp["mode"], inp["unary"], inp["ctx"], inp["ew"], inp["n_dir"], inp["n_iter"])
    want = oracle.forward(inp["mode"], inp["unary"], inp["ctx"], inp["ew"], inp["n_dir"], inp["n_iter"])
    assert rel_err(got["cost"], gold["cost"]) < COST_RTOL
    # same arithmetic order as the oracle: bit-identical values, identical indices
    assert np.array_equal(got["cost"], want["cost"])
    assert np.array_equal(got["msg"], want["msg"])
    assert np.array_equal(got["norm_idx"], want["norm_idx"])
    assert np.array_equal(got["min_idx"], want["min_idx"])
    if "min_idx" in gold.files:
        assert np.array_equal(got["min_idx"], gold["min_idx"])
        assert np.array_equal(got["norm_idx"], gold["norm_idx"])
    bwd = g.backward(inp["mode"], inp["ctx"], inp["ew"], inp["dcost"], got["min_idx"], got["norm_idx"])
    assert rel_err(bwd["dunary"], gold["dunary"]) < GRAD_RTOL
    assert rel_err(bwd["dew"], gold["dew"]) < GRAD_RTOL
    assert rel_err(bwd["dctx"], gold["dctx"]) < GRAD_RTOL
    kd = g.backward(inp["mode"], inp["ctx"], inp["ew"], inp["dcost"], got["min_idx"], got["norm_idx"],
                    keep_diag=True)
    wantkd = gold["dctx"].copy()
    if wantkd.ndim == 2:
        wantkd[np.diag_indices_from(wantkd)] = gold["dctx_diag"]
    else:
        wantkd[0] = gold["dctx_diag"][0]
    assert rel_err(kd["dctx"], wantkd) < GRAD_RTOL


def _rand_case(seed, mode, D, B, CV, H, W, L, I, kind, ew_kind="pos"):
    rng = np.random.default_rng(seed)
    unary = rng.standard_normal((B, CV, H, W, L)).astype(np.float32)
    if kind == "nonmono1d":       # 1-D function that is not non-decreasing: dense evaluation
        ctx = rng.uniform(0, 2, size=(L,)).astype(np.float32)
        ctx[0] = 0
    elif kind == "neg1d":         # saturating but with a value above the plateau
        ctx = np.minimum(np.arange(L), 3).astype(np.float32)
        if L > 2:
            ctx[1] = 5.0
    else:
        ctx = cases.make_context(kind, L, rng)
    if ew_kind == "none":
        ew = None
    elif ew_kind == "neg":        # a negative weight forces the dense path for rank-1 contexts
        ew = rng.uniform(-0.5, 1.5, size=(D, B, CV, H, W)).astype(np.float32)
    else:
        ew = rng.uniform(0.2, 1.0, size=(D, B, CV, H, W)).astype(np.float32)
    dcost = rng.uniform(0, 1, size=(B, CV, H, W, L)).astype(np.float32)
    return unary, ctx, ew, dcost


# (mode, D, B, CV, H, W, L, I, ctx kind, edge-weight kind)
SHAPES = [
    ("TRWP", 4, 1, 1, 1, 1, 1, 2, "sym2d", "pos"),        # single pixel, single label
    ("TRWP", 4, 1, 1, 1, 9, 2, 2, "sym2d", "pos"),        # one row
    ("ISGMR", 8, 1, 1, 9, 1, 3, 2, "sym2d", "pos"),       # one column
    ("TRWP", 16, 2, 1, 2, 3, 5, 2, "sym2d", "pos"),       # image smaller than the largest step
    ("ISGMR", 16, 1, 2, 3, 2, 4, 3, "sym2d", "none"),
    ("TRWP", 4, 2, 2, 13, 17, 21, 3, "sym2d", "pos"),     # cv axis > 1
    ("ISGMR", 8, 2, 1, 12, 11, 21, 2, "potts2d", "pos"),
    ("TRWP", 8, 1, 1, 9, 14, 32, 2, "sym2d", "pos"),      # full warp
    ("ISGMR", 4, 1, 1, 8, 9, 31, 2, "tl1d", "pos"),       # rank-1 context, warp kernel
    ("TRWP", 4, 1, 1, 8, 9, 33, 2, "sym2d", "pos"),       # first CTA-kernel size
    ("ISGMR", 8, 1, 1, 10, 9, 64, 2, "sym2d", "pos"),     # config-5 style dense 64x64
    ("TRWP", 4, 1, 1, 7, 8, 65, 2, "sym2d", "pos"),       # rank-2 beyond the register-row kernel
    ("TRWP", 4, 1, 1, 6, 7, 130, 1, "sym2d", "none"),     # rank-2 beyond the shared-memory table
    ("ISGMR", 4, 1, 1, 5, 6, 256, 2, "sym2d", "pos"),     # maximum label count
    ("TRWP", 4, 1, 1, 9, 12, 192, 2, "tl1d", "pos"),      # config-2 style windowed
    ("ISGMR", 4, 1, 1, 8, 9, 256, 2, "tq1d", "none"),     # config-3 style windowed
    ("TRWP", 8, 2, 1, 9, 10, 48, 2, "tl1d", "neg"),       # negative weight -> dense rank-1
    ("ISGMR", 4, 1, 1, 9, 10, 40, 2, "nonmono1d", "pos"),  # non-monotone rank-1
    ("TRWP", 4, 1, 1, 9, 10, 40, 2, "neg1d", "pos"),      # value above the plateau -> dense
    ("ISGMR", 16, 1, 1, 9, 10, 70, 1, "tq1d", "pos"),
    # two-labels-per-lane kernels (32 < L <= 64, L % 4 == 0): chains longer than the staging ring,
    # partly filled warps, both gradient schemes, every direction class
    ("ISGMR", 8, 1, 1, 45, 37, 64, 1, "sym2d", "pos"),
    ("TRWP", 4, 2, 1, 11, 53, 36, 2, "sym2d", "pos"),
    ("TRWP", 16, 1, 1, 21, 19, 64, 1, "sym2d", "pos"),
    ("ISGMR", 16, 1, 1, 18, 35, 52, 2, "sym2d", "none"),
    ("TRWP", 8, 1, 2, 33, 17, 44, 1, "nonmono1d", "pos"),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "-".join(map(str, s)))
def test_forward_backward_vs_oracle(shape):
    g = _gpu()
    mode, D, B, CV, H, W, L, I, kind, ewk = shape
    unary, ctx, ew, dcost = _rand_case(SHAPES.index(shape) + 100, mode, D, B, CV, H, W, L, I, kind, ewk)
    got = g.forward(mode, unary, ctx, ew, D, I, save_labels=True)
    want = oracle.forward(mode, unary, ctx, ew, D, I, save_labels=True)
    assert np.array_equal(got["cost"], want["cost"])
    assert np.array_equal(got["msg"], want["msg"])
    assert np.array_equal(got["norm_idx"], want["norm_idx"])
    assert np.array_equal(got["label_all"], want["label_all"])
    mism = got["min_idx"] != want["min_idx"]
    windowed = kind in ("tl1d", "tq1d") and L > 32 and ewk != "neg"
    if windowed:
        # the windowed evaluation may pick another index only among candidates of EQUAL value
        # (MPLayers/TRWP/TRWP_forward.cu:126-152 fixes the index up to exact ties): every differing
        # entry is audited by recomputing both candidates in the oracle and comparing their bits
        audit_index_ties(mode, unary, ctx, ew, D, I, got["min_idx"], want["min_idx"])
        assert mism.mean() < 2e-3
    else:
        assert not mism.any()
    # inference mode gives the same costs without saving anything
    ev = g.forward(mode, unary, ctx, ew, D, I, training=False)
    assert np.array_equal(ev["cost"], want["cost"])
    _check_backward(mode, ctx, ew, dcost, want)


@pytest.mark.parametrize("mode", ["TRWP", "ISGMR"])
def test_options(mode):
    g = _gpu()
    unary, ctx, ew, dcost = _rand_case(7, mode, 4, 1, 1, 10, 12, 21, 1, "sym2d")
    got = g.forward(mode, unary, ctx, ew, 4, 2, enable_min_a_dir=True, save_labels=True)
    want = oracle.forward(mode, unary, ctx, ew, 4, 2, enable_min_a_dir=True, save_labels=True)
    assert np.array_equal(got["cost"], want["cost"])
    assert np.array_equal(got["label_all"], want["label_all"])
    if mode == "ISGMR":   # SGM: one iteration, unary counted n_dir times
        got = g.forward(mode, unary, ctx, ew, 4, 1, enable_sgm=True)
        want = oracle.forward(mode, unary, ctx, ew, 4, 1, enable_sgm=True)
        assert np.array_equal(got["cost"], want["cost"])
        a = g.backward(mode, ctx, ew, dcost, want["min_idx"], want["norm_idx"], enable_sgm=True)
        b = oracle.backward(mode, ctx, ew, dcost, want["min_idx"], want["norm_idx"], enable_sgm=True)
        assert rel_err(a["dunary"], b["dunary"]) < GRAD_RTOL
    # arbitrary rho
    got = g.forward(mode, unary, ctx, ew, 4, 2, rho=0.7)
    want = oracle.forward(mode, unary, ctx, ew, 4, 2, rho=0.7)
    assert np.array_equal(got["cost"], want["cost"])
    a = g.backward(mode, ctx, ew, dcost, want["min_idx"], want["norm_idx"], rho=0.7)
    b = oracle.backward(mode, ctx, ew, dcost, want["min_idx"], want["norm_idx"], rho=0.7)
    assert rel_err(a["dunary"], b["dunary"]) < GRAD_RTOL
    assert rel_err(a["dew"], b["dew"]) < GRAD_RTOL
    assert rel_err(a["dctx"], b["dctx"]) < GRAD_RTOL


def test_run_to_run_identical():
    g = _gpu()
    unary, ctx, ew, dcost = _rand_case(3, "TRWP", 4, 2, 1, 33, 47, 21, 3, "sym2d")
    a = g.forward("TRWP", unary, ctx, ew, 4, 3)
    b = g.forward("TRWP", unary, ctx, ew, 4, 3)
    for k in ("cost", "msg", "min_idx", "norm_idx"):
        assert np.array_equal(a[k], b[k])
    ga = g.backward("TRWP", ctx, ew, dcost, a["min_idx"], a["norm_idx"])
    gb = g.backward("TRWP", ctx, ew, dcost, a["min_idx"], a["norm_idx"])
    for k in ("dunary", "dctx", "dew"):
        assert np.array_equal(ga[k], gb[k])


@pytest.mark.parametrize("mode,D,H,W,L,kind", [
    ("TRWP", 4, 37, 64, 21, "sym2d"),    # horizontal + vertical bulk-copy kernels, ragged last stage vertically
    ("TRWP", 4, 16, 20, 21, "potts2d"),  # width with a 4-pixel tail stage
    ("ISGMR", 8, 19, 32, 21, "sym2d"),   # directions 0-3 bulk-copy, 4-7 generic kernel in one call
    ("TRWP", 4, 33, 48, 32, "sym2d"),    # full warp of labels
    ("ISGMR", 4, 18, 36, 7, "tl1d"),     # few labels, rank-1 context
    ("TRWP", 4, 9, 30, 21, "sym2d"),     # width not a multiple of 4: generic kernel only
])
def test_bulk_copy_kernel_shapes(mode, D, H, W, L, kind):
    """Shapes that do / do not meet the 16-byte alignment rules of the bulk-copy staged kernel."""
    g = _gpu()
    for B, ewk in ((3, "pos"), (1, "none")):
        unary, ctx, ew, dcost = _rand_case(500 + H + W + L, mode, D, B, 1, H, W, L, 3, kind, ewk)
        got = g.forward(mode, unary, ctx, ew, D, 3, save_labels=True)
        want = oracle.forward(mode, unary, ctx, ew, D, 3, save_labels=True)
        for k in ("cost", "msg", "norm_idx", "min_idx", "label_all"):
            assert np.array_equal(got[k], want[k]), k
        ev = g.forward(mode, unary, ctx, ew, D, 3, training=False)
        assert np.array_equal(ev["cost"], want["cost"])


@pytest.mark.parametrize("mode,D,H,W,L,kind,ewk", [
    ("TRWP", 4, 11, 23, 192, "tl1d", "none"),    # config-2 style: 6 labels per lane, window 2
    ("ISGMR", 4, 9, 10, 256, "tq1d", "none"),    # config-3 style: 8 labels per lane, window 16
    ("ISGMR", 8, 10, 9, 64, "tl1d", "pos"),      # 2 labels per lane, diagonals, edge weights
    ("TRWP", 16, 9, 8, 100, "tq1d", "pos"),      # L not a multiple of the lane block
    ("TRWP", 4, 7, 19, 36, "tl1d", "pos"),       # just above one label per lane
    ("ISGMR", 4, 8, 9, 128, "potts1d", "none"),  # Potts as a rank-1 function (window 1)
])
def test_wide_inference_kernel(mode, D, H, W, L, kind, ewk):
    """Inference with a windowed rank-1 context and L % 4 == 0: warp-per-chain kernel with several
    labels per lane.  Costs and messages must equal the dense evaluation bit for bit."""
    g = _gpu()
    rng = np.random.default_rng(900 + L + D)
    unary = rng.standard_normal((2, 1, H, W, L)).astype(np.float32)
    if kind == "potts1d":
        ctx = np.ones(L, np.float32)
        ctx[0] = 0
    else:
        ctx = cases.make_context(kind, L, rng)
    ew = None if ewk == "none" else rng.uniform(0.2, 1.0, size=(D, 2, 1, H, W)).astype(np.float32)
    got = g.forward(mode, unary, ctx, ew, D, 3, training=False, save_labels=True)
    want = oracle.forward(mode, unary, ctx, ew, D, 3, training=False, save_labels=True)
    assert np.array_equal(got["cost"], want["cost"])
    assert np.array_equal(got["msg"], want["msg"])
    assert np.array_equal(got["label_all"], want["label_all"])


@pytest.mark.parametrize("mode,D,H,W,L,kind,ewk,quant", [
    ("TRWP", 4, 11, 23, 192, "tl1d", "none", False),   # 6 labels per lane, window 2
    ("ISGMR", 4, 9, 10, 256, "tq1d", "none", False),   # 8 labels per lane, window 16, aggregate mode
    ("TRWP", 16, 9, 8, 100, "tq1d", "pos", False),     # L not a multiple of the lane block, diagonals
    ("ISGMR", 8, 10, 9, 128, "tl1d", "pos", False),
    ("ISGMR", 4, 8, 9, 128, "potts1d", "none", False),
    ("TRWP", 4, 9, 21, 192, "tl1d", "none", True),     # quantised costs: exact ties everywhere
    ("ISGMR", 8, 8, 9, 96, "tq1d", "pos", True),
    ("TRWP", 4, 8, 9, 128, "potts1d", "none", True),
    ("TRWP", 4, 10, 840, 192, "tl1d", "pos", False),   # many short chains: shallow staging
    ("ISGMR", 8, 10, 9, 64, "tl1d", "pos", True),      # 2 labels per lane (33..64 labels, narrow window)
    ("TRWP", 4, 7, 19, 36, "tq1d", "pos", False),      # window 6 on 36 labels
    ("ISGMR", 4, 64, 70, 192, "tl1d", "pos", True),    # chains longer than several stages, ties
])
def test_wide_training_kernel(mode, D, H, W, L, kind, ewk, quant):
    """Training with a windowed rank-1 context runs the warp-per-chain kernel too (above 64 labels, and
    from 33 labels for windows up to 8).  Its saved indices follow the reference's rule among equal candidates
    (MPLayers/TRWP/TRWP_forward.cu:126-152: the highest index wins), so they must EQUAL the dense
    evaluation's, also where costs quantised to quarters make most minima tie; the backward pass
    replays them."""
    g = _gpu()
    rng = np.random.default_rng(1300 + L + D + (7 if quant else 0))
    unary = rng.standard_normal((2, 1, H, W, L)).astype(np.float32)
    if quant:
        unary = np.round(unary * 2) / 2
    if kind == "potts1d":
        ctx = np.ones(L, np.float32)
        ctx[0] = 0
    else:
        ctx = cases.make_context(kind, L, rng)
        if quant:
            ctx = np.round(ctx * 4) / 4
    ew = None if ewk == "none" else rng.uniform(0.2, 1.0, size=(D, 2, 1, H, W)).astype(np.float32)
    if quant and ew is not None:
        ew = np.round(ew * 4 + 1) / 4
    dcost = rng.uniform(0, 1, size=unary.shape).astype(np.float32)
    got = g.forward(mode, unary, ctx, ew, D, 2, save_labels=True)
    want = oracle.forward(mode, unary, ctx, ew, D, 2, save_labels=True)
    for k in ("cost", "msg", "norm_idx", "min_idx", "label_all"):
        assert np.array_equal(got[k], want[k]), k
    _check_backward(mode, ctx, ew, dcost, want)


@pytest.mark.parametrize("mode,D,H,W,L,kind,ewk", [
    ("TRWP", 4, 19, 37, 192, "tl1d", "pos"),       # 6 labels per lane; chains longer than two stages
    ("ISGMR", 4, 9, 21, 256, "tq1d", "none"),      # 8 labels per lane, scatter-field scheme
    ("TRWP", 16, 9, 8, 100, "tq1d", "pos"),        # 4 labels per lane, a partly filled lane, diagonals
    ("ISGMR", 8, 11, 9, 136, "tl1d", "pos"),       # 6 labels per lane with a partly filled lane
    ("TRWP", 4, 8, 19, 128, "nonmono1d", "pos"),   # context that does not saturate: many far targets per step
    ("ISGMR", 4, 8, 9, 68, "nonmono1d", "none"),
    ("TRWP", 4, 9, 13, 96, "potts1d", "none"),
    ("TRWP", 4, 10, 840, 192, "tl1d", "pos"),      # 1680 vertical chains in a launch: shallow stages (4 steps)
    ("ISGMR", 8, 10, 9, 64, "tl1d", "pos"),        # 2 labels per lane
    ("TRWP", 4, 7, 19, 36, "tq1d", "pos"),         # 2 labels per lane, half of the lanes without labels
    ("ISGMR", 4, 6, 700, 128, "tq1d", "none"),     # 2800 chains in the one launch of an ISGMR iteration
])
def test_wide_backward_kernel(mode, D, H, W, L, kind, ewk):
    """Backward pass for a rank-1 context with 32 < L <= 256, L % 4 == 0: warp-per-chain kernel with
    several labels per lane.  The split of the scatter into near and far indices is a tuning
    parameter (the window hint): every width, and no hint, must give the oracle's gradients."""
    g = _gpu()
    rng = np.random.default_rng(1700 + L + D)
    unary = rng.standard_normal((2, 1, H, W, L)).astype(np.float32)
    if kind == "potts1d":
        ctx = np.ones(L, np.float32)
        ctx[0] = 0
    elif kind == "nonmono1d":
        ctx = rng.uniform(0, 2, size=(L,)).astype(np.float32)
        ctx[0] = 0
    else:
        ctx = cases.make_context(kind, L, rng)
    ew = None if ewk == "none" else rng.uniform(0.2, 1.0, size=(D, 2, 1, H, W)).astype(np.float32)
    dcost = rng.uniform(0, 1, size=unary.shape).astype(np.float32)
    fwd = oracle.forward(mode, unary, ctx, ew, D, 2)
    for keep_diag in (False, True):
        want = oracle.backward(mode, ctx, ew, dcost, fwd["min_idx"], fwd["norm_idx"], keep_diag=keep_diag)
        for window in (0, 1, 3, 6, 16):
            got = g.backward(mode, ctx, ew, dcost, fwd["min_idx"], fwd["norm_idx"], keep_diag=keep_diag,
                             context_window=window)
            assert_grad_close(got["dunary"], want["dunary"], "dunary w%d" % window)
            assert_grad_close(got["dctx"], want["dctx"], "dctx w%d" % window)
            if ew is not None:
                assert_grad_close(got["dew"], want["dew"], "dew w%d" % window)


@pytest.mark.parametrize("mode,D,L,I", [
    ("ISGMR", 8, 64, 2), ("ISGMR", 8, 64, 3),   # aggregate path (many labels / directions), even and odd iteration counts
    ("ISGMR", 4, 21, 2), ("ISGMR", 4, 21, 3),   # every slice staged
    ("TRWP", 4, 21, 2), ("TRWP", 8, 40, 1),
])
def test_warm_start_from_given_messages(mode, D, L, I):
    """The iterations start from the messages the caller passes in `msg` (MPLayers/TRWP/TRWP_forward.cu:
    440-518 and MPLayers/ISGMR/ISGMR_forward.cu:506-622 read them as they are), on every kernel path
    and for both parities of the iteration count."""
    g = _gpu()
    unary, ctx, ew, dcost = _rand_case(77 + L + I, mode, D, 1, 1, 12, 16, L, I, "sym2d")
    first = oracle.forward(mode, unary, ctx, ew, D, 2)
    want = oracle.forward(mode, unary, ctx, ew, D, I, msg_init=first["msg"])
    got = g.forward(mode, unary, ctx, ew, D, I, msg_init=first["msg"])
    for k in ("cost", "msg", "min_idx", "norm_idx"):
        assert np.array_equal(got[k], want[k]), k
    # and it equals running the iterations in one go (ISGMR and TRWP are stationary iterations)
    whole = oracle.forward(mode, unary, ctx, ew, D, 2 + I)
    assert np.array_equal(got["msg"], whole["msg"])


@pytest.mark.parametrize("mode,D,H,W,L,I", [
    ("TRWP", 4, 13, 37, 21, 2),      # 37 pixels per row: a ragged last tile of 32
    ("ISGMR", 8, 9, 10, 64, 2),
    ("TRWP", 4, 5, 7, 100, 1),
])
def test_cost_with_labels_first(mode, D, H, W, L, I):
    """mpl_problem::cost_labels_first: the forward writes cost_final, and the backward reads its
    gradient, as [B,cv,L,H,W] (what pytorch/MP_module.py:232 produces with a permute); values are
    those of the labels-last call, bit for bit."""
    g = _gpu()
    unary, ctx, ew, dcost = _rand_case(500 + L, mode, D, 2, 2, H, W, L, I, "sym2d")
    plain = g.forward(mode, unary, ctx, ew, D, I)
    first = g.forward(mode, unary, ctx, ew, D, I, cost_labels_first=True)
    assert first["cost"].shape == (2, 2, L, H, W)
    assert np.array_equal(first["cost"], plain["cost"].transpose(0, 1, 4, 2, 3))
    for k in ("msg", "min_idx", "norm_idx"):
        assert np.array_equal(first[k], plain[k]), k
    b0 = g.backward(mode, ctx, ew, dcost, plain["min_idx"], plain["norm_idx"])
    b1 = g.backward(mode, ctx, ew, np.ascontiguousarray(dcost.transpose(0, 1, 4, 2, 3)), plain["min_idx"],
                    plain["norm_idx"], cost_labels_first=True)
    for k in ("dunary", "dctx", "dew"):
        assert np.array_equal(b0[k], b1[k]), k


def test_context_window_statement_and_analysis():
    """Inference with a rank-1 context and more than 32 labels: the caller's statement about the
    context (mpl_problem::context_window) selects the same kernels as the library's own analysis, and
    -1 the evaluation of all candidates; all three give the oracle's bits."""
    import torch
    from mplayers_b200 import _lib
    g = _gpu()
    rng = np.random.default_rng(4)
    L, D = 96, 4
    unary = rng.standard_normal((1, 1, 10, 12, L)).astype(np.float32)
    ctx = cases.make_context("tl1d", L, rng)
    want = oracle.forward("TRWP", unary, ctx, None, D, 2, training=False)
    assert _lib.analyze_context(torch.from_numpy(ctx).cuda()) == 2
    assert _lib.analyze_context(torch.from_numpy(rng.uniform(0, 1, L).astype(np.float32)).cuda()) == -1
    neg = torch.full((D, 1, 1, 10, 12), -0.5, device="cuda")
    assert _lib.analyze_context(torch.from_numpy(ctx).cuda(), neg) == -1
    for window in (0, 2, -1):
        got = g.forward("TRWP", unary, ctx, None, D, 2, training=False, context_window=window)
        assert np.array_equal(got["cost"], want["cost"]), window
