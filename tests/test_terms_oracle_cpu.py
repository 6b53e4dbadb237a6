"""The CPU restatement of the input builders (oracle/terms.py) against the fixtures generated from
the reference's own code (tests/golden/make_terms_golden.py), and -- where the reference build is
present -- against that build directly on further seeded inputs.  Also the argument checks of the
builders' C entry points, which run before any CUDA call."""
import ctypes
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

import terms_cases  # noqa: E402
from oracle import ref_terms, terms  # noqa: E402

GOLD = np.load(os.path.join(ROOT, "tests", "golden", "terms_golden.npz"))
EXP_RTOL = 1e-6   # modes that go through exp(): the libraries' exp differ in the last place


@pytest.mark.parametrize("name", sorted(terms_cases.STEREO))
def test_stereo_cost_and_cues_match_reference_fixtures(name):
    H, W, C, L, bf, sq, tr, gt, gp = terms_cases.STEREO[name]
    left, right = terms_cases.stereo_pair(name)
    assert np.array_equal(terms.stereo_data_cost(left, right, L, bf, sq, tr), GOLD["dsi/" + name])
    hc, vc = terms.gradient_cues(left, gt, gp)
    assert np.array_equal(hc, GOLD["hcue/" + name]) and np.array_equal(vc, GOLD["vcue/" + name])
    hcc, vcc = terms.gradient_cues(left, gt, gp, compact=True)
    # auxPy.cpp:86-99: h_cue[h*(W-1)+w], v_cue[w*(H-1)+h]
    assert hcc.shape == (1, H * (W - 1)) and vcc.shape == (1, (H - 1) * W)
    assert hcc[0, 3 * (W - 1) + 5] == hc[3, 5] and vcc[0, 5 * (H - 1) + 3] == vc[3, 5]


@pytest.mark.parametrize("method,L,smax", terms_cases.CONTEXT)
def test_smoothness_context_matches_reference_fixtures(method, L, smax):
    assert np.array_equal(terms.smoothness_context(L, method, smax), GOLD["ctx/" + method])


@pytest.mark.parametrize("name", sorted(terms_cases.EDGE))
def test_edge_weights_match_reference_fixtures(name):
    mode, B, C, H, W, D, kw, kind = terms_cases.EDGE[name]
    ours = terms.edge_weights(mode if mode != "anything_else" else "shifted", terms_cases.edge_image(name), D, **kw)
    ref = GOLD["edge/" + name]
    if ours.shape[2] != C:
        ours = np.repeat(ours, C, axis=2)   # the reference broadcasts the reduced value over channels
    if mode in ("edge_net", "kernel_cue_real"):
        assert np.abs(ours - ref).max() <= EXP_RTOL
    else:
        assert np.array_equal(ours, ref)


@pytest.mark.skipif(not ref_terms.available(), reason="reference term builders not built "
                    "(python oracle/build.py --ref-terms)")
def test_restatement_against_reference_build_on_more_inputs():
    rng = np.random.default_rng(5)
    for _ in range(12):
        H, W, C = int(rng.integers(1, 9)), int(rng.integers(2, 60)), int(rng.choice([1, 3, 4]))
        L = int(rng.integers(1, 48))
        bf, sq = int(rng.integers(0, 2)), int(rng.integers(0, 2))
        tr = int(rng.choice([255, 40, 7]))
        left = rng.integers(0, 256, (H, W, C)).astype(np.uint8)
        right = np.clip(np.roll(left.astype(int), -3, axis=1) + rng.integers(-9, 10, left.shape), 0, 255).astype(np.uint8)
        assert np.array_equal(terms.stereo_data_cost(left, right, L, bf, sq, tr),
                              ref_terms.stereo_data_cost(left, right, L, bf, sq, tr))
        a, b = terms.gradient_cues(left, 12, 3), ref_terms.gradient_cues(left, 12, 3)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_builder_entry_points_validate_before_cuda():
    from mplayers_b200 import _lib
    lib = _lib.lib()
    one = ctypes.c_void_p(16)   # never dereferenced
    assert lib.mpl_stereo_data_cost(None, one, 4, 4, 3, 8, 1, 0, 255, one, None) == 1
    assert lib.mpl_stereo_data_cost(one, one, 4, 4, 3, 300, 1, 0, 255, one, None) == 2
    assert "n_disp" in lib.mpl_last_error().decode()
    assert lib.mpl_stereo_data_cost(one, one, 0, 4, 3, 8, 1, 0, 255, one, None) == 1
    assert lib.mpl_gradient_cues(one, 4, 4, 0, 10, 2, 0, one, one, None) == 1
    assert lib.mpl_smoothness_context(16, b"XYZ", 2.0, one, None) == 2
    assert "XYZ" in lib.mpl_last_error().decode()
    assert lib.mpl_edge_mode(b"kernel_cue_real") == 5 and lib.mpl_edge_mode(b"nope") == -1
    assert lib.mpl_edge_mode(b"edge_net_sigmoid") == lib.mpl_edge_mode(b"sobel")
    assert lib.mpl_edge_mode_channels(lib.mpl_edge_mode(b"threshold"), 3) == 1
    assert lib.mpl_edge_mode_channels(lib.mpl_edge_mode(b"gt_edge"), 3) == 3
    assert lib.mpl_edge_weights(6, one, 1, 3, 4, 4, 4, 10.0, 0.0, 0.0, one, None, 0, None) == 1
    assert "workspace" in lib.mpl_last_error().decode()
    assert lib.mpl_edge_weights(3, one, 1, 3, 4, 4, 17, 10.0, 0.0, 0.0, one, None, 0, None) == 2
    assert lib.mpl_edge_weights(5, one, 1, 3, 4, 4, 4, 0.0, 0.0, 0.0, one, None, 0, None) == 1


def test_host_mirrors_refuse_cpu_tensors():
    import torch
    from mplayers_b200 import compute_terms, edge_weights
    with pytest.raises(RuntimeError, match="no CPU path"):
        edge_weights.getEdgeShift("sobel", torch.rand(1, 1, 4, 4), 4)
    with pytest.raises(RuntimeError, match="no CPU path"):
        compute_terms.stereo_data_cost(torch.zeros(4, 4, 3, dtype=torch.uint8), torch.zeros(4, 4, 3, dtype=torch.uint8), 8)
    assert edge_weights.get_steps(9) == (-1, -2)
