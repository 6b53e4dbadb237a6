"""Input builders on the GPU (stereo cost volume, gradient cues, pairwise tables, edge weights)
through the host mirrors, which call the C ABI: against the fixtures made from the reference's own
code, against the CPU restatement on further shapes, and at the full size of the stereo and
segmentation configurations.  Integer-valued outputs must be bit-exact; outputs that go through
exp()/log() within 1e-6."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

import terms_cases  # noqa: E402
from oracle import terms as oracle_terms  # noqa: E402

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(ROOT, "tests", "golden", "terms_golden.npz"))
EXP_TOL = 1e-6


def _cuda(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("name", sorted(terms_cases.STEREO))
def test_stereo_terms_match_reference_fixtures(name):
    from mplayers_b200 import compute_terms
    H, W, C, L, bf, sq, tr, gt, gp = terms_cases.STEREO[name]
    left, right = terms_cases.stereo_pair(name)
    got = compute_terms.stereo_data_cost(_cuda(left), _cuda(right), L, bf, sq, tr)
    assert np.array_equal(got.cpu().numpy(), GOLD["dsi/" + name])
    hc, vc = compute_terms.gradient_cues(_cuda(left), gt, gp)
    assert np.array_equal(hc.cpu().numpy(), GOLD["hcue/" + name])
    assert np.array_equal(vc.cpu().numpy(), GOLD["vcue/" + name])
    hcc, vcc = compute_terms.gradient_cues(_cuda(left), gt, gp, compact=True)
    eh, ev = oracle_terms.gradient_cues(left, gt, gp, compact=True)
    assert np.array_equal(hcc.cpu().numpy(), eh) and np.array_equal(vcc.cpu().numpy(), ev)


@pytest.mark.parametrize("method,L,smax", terms_cases.CONTEXT)
def test_smoothness_context_matches_reference_fixtures(method, L, smax):
    from mplayers_b200 import compute_terms
    got = compute_terms.smoothness_context(L, method, smax).cpu().numpy()
    ref = GOLD["ctx/" + method]
    if method == "Cauchy":   # goes through logf
        assert np.abs(got - ref).max() <= EXP_TOL * np.abs(ref).max()
    else:
        assert np.array_equal(got, ref)


def _edge_check(mode, got, ref):
    if mode in ("edge_net", "kernel_cue_real"):
        assert np.abs(got - ref).max() <= EXP_TOL
    elif mode == "kernel_cue_binary":
        assert (got != ref).mean() <= 1e-3   # a weight within rounding of the cut may flip
    else:
        assert np.array_equal(got, ref)


@pytest.mark.parametrize("name", sorted(terms_cases.EDGE))
def test_edge_weights_match_reference_fixtures(name):
    from mplayers_b200 import edge_weights
    mode, B, C, H, W, D, kw, kind = terms_cases.EDGE[name]
    got = edge_weights.getEdgeShift(mode, _cuda(terms_cases.edge_image(name)), D, **kw)
    ref = GOLD["edge/" + name]
    assert tuple(got.shape) == ref.shape
    _edge_check(mode, got.cpu().numpy(), ref)


def test_edge_weight_shape_conventions():
    import torch
    from mplayers_b200 import edge_weights
    img = torch.rand(3, 6, 7, device="cuda")
    assert tuple(edge_weights.getEdgeShift("sobel", img, 4).shape) == (4, 3, 6, 7)
    assert tuple(edge_weights.getEdgeShift("sobel", img[0], 8).shape) == (8, 6, 7)
    assert tuple(edge_weights.getEdgeShift("kernel_cue_real", img, 4).shape) == (4, 3, 6, 7)
    assert tuple(edge_weights.edge_weights_native("kernel_cue_real", img[None], 4).shape) == (4, 1, 1, 6, 7)
    with pytest.raises(RuntimeError, match="broadcasts"):
        edge_weights.getEdgeShift("threshold", torch.rand(2, 3, 6, 7, device="cuda"), 4)
    out = edge_weights.multi_edge_weights("kernel_cue_real", img * 255, 4, scale_list=[1, 0.5], sigma=10)
    assert [tuple(o.shape) for o in out] == [(4, 3, 6, 7), (4, 3, 3, 3)]   # as the reference: channels kept
    exp = oracle_terms.edge_weights("kernel_cue_real", (img * 255)[None].cpu().numpy(), 4, sigma=10)[:, 0, 0]
    assert np.abs(out[0][:, 0].cpu().numpy() - exp).max() <= EXP_TOL


def test_builders_against_restatement_on_random_shapes():
    from mplayers_b200 import compute_terms, edge_weights
    rng = np.random.default_rng(11)
    for _ in range(25):
        H, W, C = int(rng.integers(1, 12)), int(rng.integers(1, 150)), int(rng.choice([1, 2, 3, 4]))
        L = int(rng.choice([1, 3, 16, 21, 64, 100, 192, 256]))
        bf, sq = int(rng.integers(0, 2)), int(rng.integers(0, 2))
        tr = int(rng.choice([255, 40, 7, -12]))
        left = rng.integers(0, 256, (H, W, C)).astype(np.uint8)
        right = np.clip(np.roll(left.astype(int), -2, axis=1) + rng.integers(-9, 10, left.shape), 0, 255).astype(np.uint8)
        got = compute_terms.stereo_data_cost(_cuda(left), _cuda(right), L, bf, sq, tr).cpu().numpy()
        assert np.array_equal(got, oracle_terms.stereo_data_cost(left, right, L, bf, sq, tr)), (H, W, C, L, bf, sq, tr)
        hc, vc = compute_terms.gradient_cues(_cuda(left), 9, 2)
        eh, ev = oracle_terms.gradient_cues(left, 9, 2)
        assert np.array_equal(hc.cpu().numpy(), eh) and np.array_equal(vc.cpu().numpy(), ev)
    modes = ["gt_edge", "superpixel_edge", "canny", "sobel", "edge_net", "kernel_cue_real", "kernel_cue_binary",
             "threshold", "shifted", "cue_penalty"]
    for i in range(30):
        mode = modes[i % len(modes)]
        B, C, H, W = int(rng.integers(1, 4)), int(rng.integers(1, 4)), int(rng.integers(1, 40)), int(rng.integers(1, 70))
        D = int(rng.choice([1, 4, 8, 16]))
        img = np.floor(rng.random((B, C, H, W)) * 4).astype(np.float32) if mode in ("gt_edge", "superpixel_edge", "canny") \
            else (rng.random((B, C, H, W)) * 255).astype(np.float32)
        kw = dict(sigma=35.0, threshold=4000.0, penalty=3.0)
        got = edge_weights.edge_weights_native(mode, _cuda(img), D, **kw).cpu().numpy()
        _edge_check(mode, got, oracle_terms.edge_weights(mode, img, D, **kw))


def _time_ms(fn, n=5):
    import torch
    fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def test_stereo_cost_volume_full_size_feeds_the_layer():
    """375 x 1242 pixels, 192 disparities: bit-exact against the restatement, and the volume goes
    into the layer as its unary without a permute."""
    import torch
    import mplayers_b200
    from mplayers_b200 import compute_terms, synthetic
    H, W, C, L = 375, 1242, 3, 192
    rng = np.random.default_rng(3)
    scene = rng.integers(0, 256, (H, W + 2 * L, C))
    left = np.clip(scene[:, L:L + W] + rng.integers(-5, 6, (H, W, C)), 0, 255).astype(np.uint8)
    right = np.clip(scene[:, L + 37:L + 37 + W] + rng.integers(-5, 6, (H, W, C)), 0, 255).astype(np.uint8)
    dl, dr = _cuda(left), _cuda(right)
    got = compute_terms.stereo_data_cost(dl, dr, L)
    assert np.array_equal(got.cpu().numpy(), oracle_terms.stereo_data_cost(left, right, L))
    ms = _time_ms(lambda: compute_terms.stereo_data_cost(dl, dr, L))
    print("\n[terms] stereo cost volume %dx%dx%d: %.3f ms, %.0f GB/s written" % (H, W, L, ms, H * W * L * 4 / ms / 1e6))
    data_cost, rgb, h_cue, v_cue, ctx = compute_terms.compute_all_terms(dl, dr, "TL", 10, 3, 2, L)
    assert np.array_equal(rgb.cpu().numpy(), left.astype(np.float32))
    assert np.array_equal(ctx.cpu().numpy(), oracle_terms.smoothness_context(L, "TL", 2))
    args = synthetic.make_args(dict(unary=torch.empty(1, 1, L, 1, 1), mode="TRWP", n_iter=1, n_dir=4))
    layer = mplayers_b200.MPModule(args).eval()
    layer.set_label_context((ctx[0] * 10.0).contiguous(), None, None)
    cost, _ = layer.forward_native(data_cost.view(1, 1, H, W, L))
    disp = cost.view(H, W, L).argmin(dim=2)
    good = ((disp[:, 250:] - 37).abs() <= 1).float().mean().item()
    assert good > 0.9, good   # the scene is a fronto-parallel plane at disparity 37


def test_edge_weights_full_size():
    from mplayers_b200 import edge_weights
    rng = np.random.default_rng(4)
    img = (rng.random((2, 3, 512, 512)) * 255).astype(np.float32)
    d = _cuda(img)
    for mode, D in (("kernel_cue_real", 16), ("sobel", 8), ("cue_penalty", 4)):
        kw = dict(sigma=30.0, threshold=5000.0, penalty=2.0)
        got = edge_weights.edge_weights_native(mode, d, D, **kw)
        _edge_check(mode, got.cpu().numpy(), oracle_terms.edge_weights(mode, img, D, **kw))
        ms = _time_ms(lambda: edge_weights.edge_weights_native(mode, d, D, **kw))
        print("\n[terms] edge weights %s D=%d 2x3x512x512: %.3f ms" % (mode, D, ms))


def test_compute_terms_py_reads_image_files(tmp_path):
    from mplayers_b200 import compute_terms
    try:
        import cv2
    except ImportError:
        pytest.skip("OpenCV's Python module is needed to write the test images")
    left, right = terms_cases.stereo_pair("bt_rgb")
    lp, rp = str(tmp_path / "l.png"), str(tmp_path / "r.png")
    cv2.imwrite(lp, left)
    cv2.imwrite(rp, right)
    param = compute_terms.MRFParams(lp, rp, "TL", 24, 10, 3, 5)
    data_cost, rgb, ctx, param = compute_terms.compute_terms_py(param)
    assert (param.height, param.width, param.n_channels) == left.shape
    assert np.array_equal(data_cost.cpu().numpy(), GOLD["dsi/bt_rgb"])
    assert np.array_equal(rgb.cpu().numpy(), left.astype(np.float32))
    assert np.array_equal(ctx.cpu().numpy(), oracle_terms.smoothness_context(24, "TL", 5))
