"""Generates the golden vectors in this directory from the REFERENCE's own implementation.

Run in a container that has the reference checkout (its path in $MPL_REFERENCE_DIR; the default is
the directory mounted next to this repository):   python tests/golden/make_golden.py

The generator imports the reference's pure-PyTorch autograd implementation
(pytorch/message_passing.py, MessagePassingModule) in float64, feeds it the seeded inputs of
cases.py and stores, per case: final cost, gradients w.r.t. unary / label context / edge
weights for the loss sum(cost * dcost), and (small cases) the saved argmin indices derived from
the reference's full edge vectors.  Mapping of the reference's per-direction dense context
gradient G_d[a,b] onto the extension's convention (MPLayers/TRWP/TRWP_backward.cu:102-112):
  2-D: dctx[a,b] = sum_d (G_d[a,b] + G_d[b,a]) for a<b, 0 elsewhere (diagonal kept separately);
  1-D: dctx[k]   = sum_d sum_{|a-b|=k} G_d[a,b] for k>0, k=0 kept separately.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402

# the reference checkout: $MPL_REFERENCE_DIR, else a directory `reference` next to this repository
REF = os.environ.get("MPL_REFERENCE_DIR",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))


def import_reference_oracle():
    # pytorch/message_passing.py:5 imports two helpers from tools/python/utils.py, which needs
    # matplotlib; they are only used for debugging output.
    pkg = types.ModuleType("python")
    mod = types.ModuleType("python.utils")
    mod.check_valid = lambda x, enable_zero=False: True
    mod.check_data_input = lambda *a, **k: None
    pkg.utils = mod
    sys.modules["python"] = pkg
    sys.modules["python.utils"] = mod
    sys.path.insert(0, os.path.join(REF, "pytorch"))
    from message_passing import MessagePassingModule
    return MessagePassingModule


def run_case(MessagePassingModule, name, store_indices):
    inp = cases.make_inputs(name)
    mode, D, I = inp["mode"], inp["n_dir"], inp["n_iter"]
    unary = torch.from_numpy(inp["unary"]).double()          # [B,1,H,W,L]
    B, _, H, W, L = unary.shape
    ctx = inp["ctx"]
    if ctx.ndim == 1:
        idx = np.abs(np.arange(L)[:, None] - np.arange(L)[None, :])
        dense = ctx[idx]
    else:
        dense = ctx
    lc = torch.from_numpy(dense).double().view(1, L, L).repeat(D, 1, 1).clone()
    ew = torch.from_numpy(inp["ew"]).double()[:, :, 0].permute(1, 0, 2, 3).contiguous()  # [B,D,H,W]
    ew.requires_grad_(True)
    score = (-unary[:, 0].permute(0, 3, 1, 2)).contiguous().requires_grad_(True)        # [B,L,H,W]
    m = MessagePassingModule(max_iter=I, n_labels=L, n_dirs=D, mode=mode,
                             ISGMR_parallel=(mode == "ISGMR"), enable_debug=False,
                             target="Stereo", graph_model="min_sum", label_context=lc,
                             n_edge_feats=1, llambda=1., enable_Gaussian=False,
                             enable_message_vector=store_indices,
                             enable_soft_weight=cases.is_soft(name))
    out = m.forward(score, torch.zeros(B, 3, H, W, dtype=torch.float64), ew)
    cost = -out[0]                                            # [B,L,H,W]
    dcost = torch.from_numpy(inp["dcost"]).double()[:, 0].permute(0, 3, 1, 2)
    (cost * dcost).sum().backward()
    res = {}
    res["cost"] = cost.detach().permute(0, 2, 3, 1).unsqueeze(1).numpy()            # [B,1,H,W,L]
    res["dunary"] = (-score.grad).permute(0, 2, 3, 1).unsqueeze(1).numpy()
    res["dew"] = ew.grad.permute(1, 0, 2, 3).unsqueeze(2).numpy()                    # [D,B,1,H,W]
    G = m.label_context.grad.numpy()                                                 # [D,L,L]
    Gs = G.sum(0)
    if ctx.ndim == 2:
        dctx = np.triu(Gs + Gs.T, 1)
        res["dctx_diag"] = np.diag(Gs).copy()
    else:
        k = np.abs(np.arange(L)[:, None] - np.arange(L)[None, :])
        dctx = np.array([Gs[k == kk].sum() for kk in range(L)])
        res["dctx_diag"] = np.array([dctx[0]])
        dctx[0] = 0.0
    res["dctx"] = dctx
    if cases.is_soft(name):
        # soft TRWP accumulates the label-context gradient on the diagonal as well
        # (MPLayers/TRWP_hard_soft/TRWP_backward_soft.cu:114-126) and saves the edge values
        # themselves ([f][c] for even directions, [c][f] for odd ones) instead of argmin indices
        if ctx.ndim == 2:
            res["dctx"] = dctx + np.diag(np.diag(Gs))
        else:
            res["dctx"] = dctx.copy()
            res["dctx"][0] = res["dctx_diag"][0]
        res["edge_label"] = out[5].detach().numpy()
        res["norm_idx"] = out[6].detach().numpy().astype(np.uint8)
        return res
    if store_indices:
        mv = out[5].detach().numpy()      # [I,D,B,1,H,W,L,L]
        ni = out[6].detach().numpy()      # [I,D,B,1,H,W]
        mi = np.zeros(mv.shape[:-1], np.uint8)
        for d in range(D):
            # even directions: front label on axis -2, odd: on axis -1 (message_passing.py:367-396)
            vec = mv[:, d] if d % 2 == 0 else np.swapaxes(mv[:, d], -1, -2)   # [..., f, c]
            # highest index among equal minima, as the extension does
            mi[:, d] = (L - 1 - np.argmin(vec[..., ::-1, :], axis=-2)).astype(np.uint8)
        # pixels without a predecessor in direction d are never visited: the extension leaves
        # their (zero-initialised) index entries untouched
        steps = [(0, 1), (0, -1), (1, 0), (-1, 0), (1, 1), (-1, -1), (1, -1), (-1, 1), (1, 2),
                 (-1, -2), (2, 1), (-2, -1), (2, -1), (-2, 1), (1, -2), (-1, 2)]
        hh, ww = np.meshgrid(np.arange(H), np.arange(W), indexing="ij")
        for d in range(D):
            fh, fw = hh - steps[d][0], ww - steps[d][1]
            start = (fh < 0) | (fh >= H) | (fw < 0) | (fw >= W)
            mi[:, d][..., start, :] = 0
            assert (ni[:, d][..., start] == 0).all()
        res["min_idx"] = mi
        res["norm_idx"] = ni.astype(np.uint8)
    return res


def main():
    MPM = import_reference_oracle()
    only = [a for a in sys.argv[1:] if not a.startswith("-")]
    for name in cases.CASES:
        if only and name not in only:
            continue
        small = not name.endswith("config1")
        with torch.enable_grad():
            res = run_case(MPM, name, store_indices=small)
        out = {}
        for k, v in res.items():
            out[k] = v if v.dtype == np.uint8 else v.astype(np.float32)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(name, {k: v.shape for k, v in out.items()}, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
