"""Seeded inputs of the input-builder fixtures (shared by make_terms_golden.py and the tests).
Synthetic images only: a random piecewise-smooth scene, its copy shifted by a per-row disparity
for the right view, plus noise -- no item of any stereo or segmentation dataset."""
import numpy as np

# name: (H, W, channels, n_disp, birchfield, squared_diffs, trunc_diffs, grad_thresh, grad_penalty)
STEREO = {
    "bt_rgb": (12, 70, 3, 24, 1, 0, 255, 10, 3),
    "bt_gray_squared": (9, 45, 1, 16, 1, 1, 20, 8, 2),
    "abs_rgb_trunc": (8, 37, 3, 40, 0, 0, 15, 10, 2),
    "bt_four_channels": (6, 33, 4, 12, 1, 0, 255, 5, 4),
    "abs_squared_wide_labels": (5, 19, 3, 32, 0, 1, 30, 10, 3),   # n_disp > width
}

CONTEXT = [("L", 16, 0.0), ("Q", 16, 0.0), ("TL", 24, 5.0), ("TQ", 24, 4.0), ("Cauchy", 20, 7.0), ("Huber", 20, 6.0)]

# name: (mode, B, C, H, W, n_dirs, kwargs, kind of image)
EDGE = {
    "gt_edge": ("gt_edge", 2, 1, 14, 17, 16, {}, "labels255"),
    "superpixel_edge": ("superpixel_edge", 1, 3, 11, 13, 8, {}, "labels"),
    "canny": ("canny", 2, 1, 12, 15, 8, {}, "binary"),
    "sobel": ("sobel", 2, 3, 10, 12, 4, {}, "unit"),
    "edge_net_sigmoid": ("edge_net_sigmoid", 1, 1, 10, 12, 16, {}, "unit"),
    "edge_net": ("edge_net", 2, 1, 9, 14, 8, {}, "unit"),
    "kernel_cue_real": ("kernel_cue_real", 1, 3, 13, 16, 16, {"sigma": 10.0}, "rgb"),
    "kernel_cue_binary": ("kernel_cue_binary", 1, 3, 13, 16, 8, {"sigma": 40.0}, "rgb"),
    "threshold": ("threshold", 1, 3, 12, 12, 8, {"threshold": 3000.0, "penalty": 2.0}, "rgb"),
    "shifted": ("anything_else", 2, 2, 7, 9, 16, {}, "unit"),
    "tiny_image": ("sobel", 1, 1, 2, 2, 16, {}, "unit"),          # steps of 2 leave no patch
}


def stereo_pair(name):
    H, W, C, L = STEREO[name][:4]
    rng = np.random.default_rng(sum(map(ord, name)))
    wide = W + 2 * L + 8
    scene = rng.integers(0, 256, (H, wide // 4 + 2, C)).astype(np.float64)
    scene = np.repeat(scene, 4, axis=1)[:, :wide]                 # 4-pixel-wide constant runs
    scene = scene + rng.normal(0, 6, scene.shape)
    left = scene[:, L + 4:L + 4 + W]
    disp = rng.integers(0, max(L // 2, 1), H)
    right = np.stack([scene[y, L + 4 + disp[y]:L + 4 + disp[y] + W] for y in range(H)])
    right = right + rng.normal(0, 3, right.shape)
    to_u8 = lambda a: np.clip(np.rint(a), 0, 255).astype(np.uint8)  # noqa: E731
    return to_u8(left), to_u8(right)


def edge_image(name):
    mode, B, C, H, W, D, kw, kind = EDGE[name]
    rng = np.random.default_rng(1000 + sum(map(ord, name)))
    if kind == "labels255":
        img = rng.integers(0, 3, (B, C, H, W)).astype(np.float32)
        img[rng.random((B, C, H, W)) < 0.15] = 255
    elif kind == "labels":
        img = np.repeat(rng.integers(0, 3, (B, 1, H, W)), C, axis=1).astype(np.float32)
        img[:, 0][rng.random((B, H, W)) < 0.2] += 1
    elif kind == "binary":
        img = (rng.random((B, C, H, W)) < 0.3).astype(np.float32)
    elif kind == "rgb":
        img = np.floor(rng.random((B, C, H, W)) * 256).astype(np.float32)
    else:
        img = rng.random((B, C, H, W)).astype(np.float32)
    return img
