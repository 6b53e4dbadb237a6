"""Seeded synthetic inputs with the shapes and value distributions of the five benchmark
configurations (they stand in for the stereo pairs, denoising images and PASCAL VOC crops the
reference was run on; no item of those datasets is used).

Every generator returns a dict of CPU tensors in the operator API's layouts:
  unary [B,1,L,H,W] (cost volume), label_context [L] or [L,L], edge_weights [B,D,H,W] or None,
plus mode / n_dir / n_iter / training.
"""
import math

import torch
import torch.nn.functional as F

STEPS = [(0, 1), (0, -1), (1, 0), (-1, 0), (1, 1), (-1, -1), (1, -1), (-1, 1), (1, 2), (-1, -2),
         (2, 1), (-2, -1), (2, -1), (-2, 1), (1, -2), (-1, 2)]


def _gen(seed):
    g = torch.Generator()
    g.manual_seed(int(seed))
    return g


def _smooth_noise(g, b, c, h, w, sigma):
    x = torch.rand(b, c, h, w, generator=g)
    r = int(3 * sigma)
    k = torch.exp(-torch.arange(-r, r + 1, dtype=torch.float32) ** 2 / (2 * sigma * sigma))
    k = (k / k.sum()).view(1, 1, 1, -1)
    x = x.reshape(b * c, 1, h, w)
    x = F.conv2d(F.pad(x, (r, r, 0, 0), mode="reflect"), k)
    x = F.conv2d(F.pad(x, (0, 0, r, r), mode="reflect"), k.transpose(2, 3))
    x = x.reshape(b, c, h, w)
    lo, hi = x.amin(dim=(2, 3), keepdim=True), x.amax(dim=(2, 3), keepdim=True)
    return (x - lo) / (hi - lo + 1e-12)


def edge_weights_from_image(img, n_dir, sigma=0.1):
    """exp(-|I(cur) - I(front)|^2 / (2 sigma^2)) stored at the receiving pixel `cur`, 0 where the
    pixel has no predecessor in that direction (convention of the reference's
    utils/edge_weights.py:58-104)."""
    b, c, h, w = img.shape
    out = torch.zeros(b, n_dir, h, w)
    for d in range(n_dir):
        hs, ws = STEPS[d]
        h0, h1 = max(hs, 0), h + min(hs, 0)
        w0, w1 = max(ws, 0), w + min(ws, 0)
        if h1 <= h0 or w1 <= w0:
            continue
        cur = img[:, :, h0:h1, w0:w1]
        front = img[:, :, h0 - hs:h1 - hs, w0 - ws:w1 - ws]
        diff2 = ((cur - front) ** 2).sum(dim=1)
        out[:, d, h0:h1, w0:w1] = torch.exp(-diff2 / (2 * sigma * sigma))
    return out


def config1(mode="TRWP", seed=0):
    """B1 D4 64x64 L21 I5, unary N(0,1), Potts, edge weights U[0.5,1] (the reference's CPU-runnable case)."""
    g = _gen(seed)
    L, H, W, D = 21, 64, 64, 4
    return dict(mode=mode, n_dir=D, n_iter=5, training=True,
                unary=torch.randn(1, 1, L, H, W, generator=g),
                label_context=1.0 - torch.eye(L),
                edge_weights=0.5 + 0.5 * torch.rand(1, D, H, W, generator=g))


def config2_stereo(seed=0, H=375, W=1242, L=192, n_iter=3, training=False):
    """Stereo TRWP forward: piecewise-planar disparity from 20 planes over a Voronoi partition,
    unary min(|d-d_gt|/8, 1) + U[0,0.3], 10% outlier pixels U[0,1]; truncated linear pairwise."""
    g = _gen(seed)
    ys, xs = torch.meshgrid(torch.arange(H, dtype=torch.float32), torch.arange(W, dtype=torch.float32),
                            indexing="ij")
    sites = torch.rand(20, 2, generator=g) * torch.tensor([H, W], dtype=torch.float32)
    d2 = (ys[None] - sites[:, 0, None, None]) ** 2 + (xs[None] - sites[:, 1, None, None]) ** 2
    region = d2.argmin(0)
    a = (torch.rand(20, generator=g) - 0.5) * 0.1
    b = (torch.rand(20, generator=g) - 0.5) * 0.1
    c = torch.rand(20, generator=g) * (L - 1)
    dgt = (a[region] * (xs - W / 2) + b[region] * (ys - H / 2) + c[region]).clamp(0, L - 1)
    lab = torch.arange(L, dtype=torch.float32).view(L, 1, 1)
    unary = ((lab - dgt[None]).abs() / 8).clamp(max=1.0) + 0.3 * torch.rand(L, H, W, generator=g)
    outl = torch.rand(H, W, generator=g) < 0.1
    noise = torch.rand(L, H, W, generator=g)
    unary = torch.where(outl[None], noise, unary)
    ctx = torch.arange(L, dtype=torch.float32).clamp(max=2.0)
    return dict(mode="TRWP", n_dir=4, n_iter=n_iter, training=training,
                unary=unary.view(1, 1, L, H, W).contiguous(), label_context=ctx, edge_weights=None)


def config3_denoise(seed=0, H=256, W=256, L=256, n_iter=50, training=False):
    """Denoise ISGMR forward: 12 constant rectangles/discs + N(0,20^2), unary (l-obs)^2/256,
    truncated quadratic pairwise 25*min(k^2, 200)."""
    g = _gen(seed)
    img = torch.full((H, W), float(torch.randint(0, 256, (1,), generator=g)))
    ys, xs = torch.meshgrid(torch.arange(H), torch.arange(W), indexing="ij")
    for i in range(12):
        val = float(torch.randint(0, 256, (1,), generator=g))
        cy, cx = int(torch.randint(0, H, (1,), generator=g)), int(torch.randint(0, W, (1,), generator=g))
        r = int(torch.randint(H // 16, H // 4, (1,), generator=g))
        if i % 2 == 0:
            m = ((ys - cy).abs() < r) & ((xs - cx).abs() < r)
        else:
            m = (ys - cy) ** 2 + (xs - cx) ** 2 < r * r
        img[m] = val
    obs = (img + 20.0 * torch.randn(H, W, generator=g)).clamp(0, 255)
    lab = torch.arange(L, dtype=torch.float32).view(L, 1, 1)
    unary = (lab - obs[None]) ** 2 / 256.0
    k = torch.arange(L, dtype=torch.float32)
    ctx = 25.0 * (k * k).clamp(max=200.0)
    return dict(mode="ISGMR", n_dir=4, n_iter=n_iter, training=training,
                unary=unary.view(1, 1, L, H, W).contiguous(), label_context=ctx, edge_weights=None)


def config4_segmentation(batch=2, seed=0, H=512, W=512, L=21, n_dir=4, n_iter=5, mode="TRWP"):
    """Segmentation training step (TRWP fwd+bwd): DeepLab-like logits N(0,1) + 3 on a blob class
    map, turned into non-negative costs as mpnet.py:162-163 does; learned dense 21x21 context
    U[0,2] with zero diagonal; edge weights exp(-|grad I|^2 / 2 sigma^2), sigma = 0.1."""
    g = _gen(seed)
    coarse = torch.randint(0, L, (batch, 1, max(H // 32, 1), max(W // 32, 1)), generator=g).float()
    cls = F.interpolate(coarse, size=(H, W), mode="nearest").long()[:, 0]
    score = torch.randn(batch, L, H, W, generator=g)
    score += 3.0 * F.one_hot(cls, L).permute(0, 3, 1, 2).float()
    cost = -score
    cost = cost - cost.amin(dim=1, keepdim=True)
    a = torch.triu(2.0 * torch.rand(L, L, generator=g), 1)
    ctx = a + a.t()
    img = _smooth_noise(g, batch, 3, H, W, sigma=4.0)
    ew = edge_weights_from_image(img, n_dir, sigma=0.1)
    return dict(mode=mode, n_dir=n_dir, n_iter=n_iter, training=True,
                unary=cost.unsqueeze(1).contiguous(), label_context=ctx, edge_weights=ew)


def config5_large(batch=1, seed=0, H=1024, W=1024, L=64, n_dir=8, n_iter=10):
    """Large ISGMR fwd+bwd: unary U[0,1], dense symmetric 64x64 context U[0,1] with zero diagonal,
    edge weights U[0.2,1], 8 directions."""
    g = _gen(seed)
    a = torch.triu(torch.rand(L, L, generator=g), 1)
    return dict(mode="ISGMR", n_dir=n_dir, n_iter=n_iter, training=True,
                unary=torch.rand(batch, 1, L, H, W, generator=g), label_context=a + a.t(),
                edge_weights=0.2 + 0.8 * torch.rand(batch, n_dir, H, W, generator=g))


def make_args(cfg):
    """`args` namespace of the operator API for a generated configuration."""
    import types
    L = cfg["unary"].shape[2]
    return types.SimpleNamespace(mpnet_mrf_mode=cfg["mode"], mpnet_max_iter=cfg["n_iter"],
                                 mpnet_n_dirs=cfg["n_dir"], n_classes=L, mpnet_smoothness_train=None,
                                 mpnet_term_weight=1.0, mpnet_diag_value=0.0, enable_symmetric=True,
                                 mpnet_smoothness_mode="Potts", mpnet_smoothness_trunct_value=-1,
                                 mpnet_smoothness_trunct_loc=-1, enable_cuda=True)
