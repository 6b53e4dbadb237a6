"""Labelling energy on the GPU against a numpy restatement, and the property it exists for: the
energy of the per-iteration labellings of a forward call goes down (here: ends below the energy
of the unary-only labelling)."""
import numpy as np
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu

STEPS = [(0, 1), (0, -1), (1, 0), (-1, 0), (1, 1), (-1, -1), (1, -1), (-1, 1), (1, 2), (-1, -2), (2, 1), (-2, -1),
         (2, -1), (-2, 1), (1, -2), (-1, 2)]


def _energy_numpy(unary, ctx, ew, lab, D):
    B, CV, H, W, L = unary.shape
    cm = ctx if ctx.ndim == 2 else ctx[np.abs(np.arange(L)[:, None] - np.arange(L)[None, :])]
    cm = np.triu(cm) + np.triu(cm, 1).T if ctx.ndim == 2 else cm   # the kernels read the upper triangle
    eu = np.take_along_axis(unary.astype(np.float64), lab[..., None].astype(np.int64), -1).sum()
    ep = 0.0
    for d in range(0, D, 2):
        hs, ws = STEPS[d]
        for h in range(H):
            for w in range(W):
                fh, fw = h - hs, w - ws
                if 0 <= fh < H and 0 <= fw < W:
                    e = 1.0 if ew is None else ew[d, :, :, h, w].astype(np.float64)
                    ep += (e * cm[lab[:, :, h, w], lab[:, :, fh, fw]].astype(np.float32)).sum()
    return eu, ep


@pytest.mark.parametrize("D,L,kind,with_ew", [(4, 7, "sym2d", True), (8, 12, "tl1d", True), (16, 5, "sym2d", False)])
def test_energy_matches_numpy(D, L, kind, with_ew):
    from mplayers_b200.energy import labeling_energy
    rng = np.random.default_rng(31)
    B, CV, H, W, I = 2, 1, 9, 11, 3
    unary = rng.standard_normal((B, CV, H, W, L)).astype(np.float32)
    ctx = cases.make_context(kind, L, rng)
    ew = rng.uniform(0.2, 1.5, size=(D, B, CV, H, W)).astype(np.float32) if with_ew else None
    lab = rng.integers(0, L, size=(I, B, CV, H, W)).astype(np.uint8)
    got = labeling_energy(torch.from_numpy(unary).cuda(), torch.from_numpy(ctx).cuda(),
                          torch.from_numpy(ew).cuda() if with_ew else None, torch.from_numpy(lab).cuda(), D).cpu().numpy()
    for i in range(I):
        eu, ep = _energy_numpy(unary, ctx, ew, lab[i], D)
        assert abs(got[i, 0] - eu) < 1e-4 * max(abs(eu), 1.0)
        assert abs(got[i, 1] - ep) < 1e-4 * max(abs(ep), 1.0)


def test_message_passing_lowers_the_energy():
    import types
    from mplayers_b200 import MPModule
    from mplayers_b200.energy import labeling_energy
    g = torch.Generator().manual_seed(8)
    B, L, H, W, D, I = 1, 16, 48, 64, 4, 8
    truth = torch.randint(0, L, (B, 1, H // 8, W // 8), generator=g).float()
    truth = torch.nn.functional.interpolate(truth, size=(H, W), mode="nearest")[:, 0].long()
    unary = (torch.arange(L).view(1, L, 1, 1) - truth.unsqueeze(1)).abs().float().clamp(max=3)
    unary = (unary + torch.rand(B, L, H, W, generator=g) * 3).unsqueeze(1).cuda()        # [B,cv,L,H,W]
    ctx = torch.minimum(torch.arange(L, dtype=torch.float32), torch.tensor(2.0)).cuda()  # truncated linear
    for mode in ("TRWP", "ISGMR"):
        args = types.SimpleNamespace(mpnet_mrf_mode=mode, mpnet_max_iter=I, mpnet_n_dirs=D, n_classes=L,
                                     mpnet_smoothness_train=None, mpnet_term_weight=1.0, mpnet_diag_value=0.0,
                                     enable_symmetric=True)
        layer = MPModule(args, enable_saving_label=True).cuda().eval()
        layer.set_label_context(ctx, None, None)
        with torch.no_grad():
            cost, _, label_all, _, _ = layer(unary)
        u_hwl = unary.permute(0, 1, 3, 4, 2).contiguous()
        e_iter = labeling_energy(u_hwl, ctx, None, label_all, D).sum(1).cpu().numpy()
        unary_only = u_hwl.argmin(-1).to(torch.uint8)
        e0 = float(labeling_energy(u_hwl, ctx, None, unary_only, D).sum())
        assert e_iter[-1] < e0, (mode, e0, e_iter)
        assert e_iter[-1] <= e_iter[0] + 1e-6 * abs(e0), (mode, e_iter)
