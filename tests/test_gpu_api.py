"""The operator API (MPModule / autograd Functions) on the GPU against the CPU oracle."""
import types

import numpy as np
import pytest
import torch

from helpers import COST_RTOL, GRAD_RTOL, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu


def _args(mode, n_iter, n_dir, L):
    return types.SimpleNamespace(mpnet_mrf_mode=mode, mpnet_max_iter=n_iter, mpnet_n_dirs=n_dir,
                                 n_classes=L, mpnet_smoothness_train=None, mpnet_term_weight=1.0,
                                 mpnet_diag_value=0.0, enable_symmetric=True, mpnet_enable_soft=False)


def _inputs(seed, B, L, H, W, D, rank):
    rng = np.random.default_rng(seed)
    unary = rng.standard_normal((B, 1, L, H, W)).astype(np.float32)
    if rank == 2:
        a = np.triu(rng.uniform(0, 2, (L, L)), 1)
        ctx = (a + a.T).astype(np.float32)
    else:
        ctx = np.minimum(np.arange(L), 3).astype(np.float32)
    ew = rng.uniform(0.2, 1.0, (B, D, H, W)).astype(np.float32)
    g = rng.uniform(0, 1, (B, 1, L, H, W)).astype(np.float32)
    return unary, ctx, ew, g


def _to_ext(unary, ew, g):
    un = np.ascontiguousarray(unary.transpose(0, 1, 3, 4, 2))
    en = None if ew is None else np.ascontiguousarray(ew[:, None].transpose(2, 0, 1, 3, 4))
    gn = np.ascontiguousarray(g.transpose(0, 1, 3, 4, 2))
    return un, en, gn


@pytest.mark.parametrize("mode,module,rank,L,D,use_ew", [
    ("TRWP", "plain", 2, 21, 4, True), ("ISGMR", "plain", 2, 21, 8, True),
    ("TRWP", "hard_soft", 2, 21, 4, True), ("TRWP", "plain", 1, 48, 4, False),
    ("ISGMR", "plain", 1, 40, 4, True),
])
def test_module_forward_backward(mode, module, rank, L, D, use_ew):
    from mplayers_b200 import MP_module, MP_module_hard_soft
    unary, ctx, ew, g = _inputs(5, 2, L, 11, 13, D, rank)
    if not use_ew:
        ew = None
    args = _args(mode, 3, D, L)
    mod = (MP_module_hard_soft if module == "hard_soft" else MP_module).MPModule(args)
    param = torch.nn.Parameter(torch.from_numpy(ctx).cuda())
    mod.set_label_context(param, None, None)
    mod.train()
    u = torch.from_numpy(unary).cuda().requires_grad_(True)
    e = torch.from_numpy(ew).cuda().requires_grad_(True) if use_ew else None
    out = mod(u, e)
    assert len(out) == 5 and out[0].shape == u.shape and out[1].shape == (1,) + ctx.shape
    (out[0] * torch.from_numpy(g).cuda()).sum().backward()
    torch.cuda.synchronize()

    un, en, gn = _to_ext(unary, ew, g)
    fw = oracle.forward(mode, un, ctx, en, D, 3)
    bw = oracle.backward(mode, ctx, en, gn, fw["min_idx"], fw["norm_idx"], keep_diag=(module == "hard_soft"))
    got = out[0].detach().permute(0, 1, 3, 4, 2).cpu().numpy()
    assert rel_err(got, fw["cost"]) < COST_RTOL
    assert rel_err(u.grad.permute(0, 1, 3, 4, 2).cpu().numpy(), bw["dunary"]) < GRAD_RTOL
    assert rel_err(param.grad.cpu().numpy(), bw["dctx"]) < GRAD_RTOL
    if use_ew:
        assert rel_err(e.grad[:, None].permute(2, 0, 1, 3, 4).cpu().numpy(), bw["dew"]) < GRAD_RTOL

    # inference mode: same costs, per-iteration labels on request, nothing saved for backward
    args2 = _args(mode, 3, D, L)
    mod2 = MP_module.MPModule(args2, enable_saving_label=True)
    mod2.set_label_context(param, None, None)
    mod2.eval()
    with torch.no_grad():
        cost2, _, labels, _, _ = mod2(u.detach(), e.detach() if use_ew else None)
    assert torch.equal(cost2, out[0].detach())
    want = oracle.forward(mode, un, ctx, en, D, 3, training=False, save_labels=True)
    assert np.array_equal(labels.cpu().numpy(), want["label_all"])


def test_sgm_and_errors():
    from mplayers_b200 import MP_module, TRWP
    unary, ctx, ew, g = _inputs(9, 1, 21, 9, 10, 4, 2)
    args = _args("SGM", 1, 4, 21)
    mod = MP_module.MPModule(args)
    mod.set_label_context(torch.from_numpy(ctx).cuda(), None, None)
    mod.eval()
    with torch.no_grad():
        cost = mod(torch.from_numpy(unary).cuda(), torch.from_numpy(ew).cuda())[0]
    un, en, _ = _to_ext(unary, ew, g)
    want = oracle.forward("ISGMR", un, ctx, en, 4, 1, enable_sgm=True, training=False)
    assert rel_err(cost.permute(0, 1, 3, 4, 2).cpu().numpy(), want["cost"]) < COST_RTOL

    u = torch.zeros(1, 1, 4, 5, 300, device="cuda")
    with pytest.raises(RuntimeError, match="n_disp"):
        TRWP.forward(0.5, 1, 0, u, torch.zeros(300, device="cuda"), torch.zeros(0, device="cuda"),
                     torch.zeros(4, 1, 1, 4, 5, 300, device="cuda"), torch.zeros_like(u),
                     torch.zeros(0, dtype=torch.uint8, device="cuda"),
                     torch.zeros(0, dtype=torch.uint8, device="cuda"), torch.zeros(0, device="cuda"),
                     torch.zeros(0, dtype=torch.uint8, device="cuda"))
    # the context stays usable after a rejected call
    assert torch.zeros(2, device="cuda").sum().item() == 0


def test_identical_samples_give_identical_results():
    """Twelve copies of one sample in a batch must come out bit-identical (the check the
    reference's pytorch/test_multi_batch.py does by eye)."""
    from mplayers_b200 import MP_module
    unary, ctx, ew, g = _inputs(2, 1, 21, 17, 19, 4, 2)
    args = _args("TRWP", 4, 4, 21)
    mod = MP_module.MPModule(args)
    mod.set_label_context(torch.from_numpy(ctx).cuda(), None, None)
    mod.eval()
    u = torch.from_numpy(unary).cuda().repeat(12, 1, 1, 1, 1)
    e = torch.from_numpy(ew).cuda().repeat(12, 1, 1, 1)
    with torch.no_grad():
        cost = mod(u, e)[0]
    for b in range(1, 12):
        assert torch.equal(cost[b], cost[0])


@pytest.mark.parametrize("soft", [False, True])
def test_supplied_norm_index_replaces_the_saved_one_in_backward(soft):
    """pytorch/MP_module_hard_soft.py:76,169-171: `msg_norm_index` given to forward() is used by
    the backward pass instead of the indices the forward pass saved; the forward result does not
    change."""
    from mplayers_b200 import MP_module_hard_soft
    L, D, I = 21, 4, 2
    unary, ctx, ew, g = _inputs(9, 1, L, 9, 10, D, 2)
    args = _args("TRWP", I, D, L)
    args.mpnet_enable_soft = soft
    mod = MP_module_hard_soft.MPModule(args)
    mod.set_label_context(torch.from_numpy(ctx).cuda(), None, None)
    mod.train()
    rng = np.random.default_rng(1)
    given = rng.integers(0, L, (I, D, 1, 1, 9, 10)).astype(np.uint8)
    u = torch.from_numpy(unary).cuda().requires_grad_(True)
    e = torch.from_numpy(ew).cuda()
    out_plain = mod(u, e)
    out = mod(u, e, msg_norm_index=torch.from_numpy(given))
    assert torch.equal(out[0], out_plain[0])
    (out[0] * torch.from_numpy(g).cuda()).sum().backward()
    un, en, gn = _to_ext(unary, ew, g)
    if soft:
        fw = oracle.forward_soft(un, ctx, en, D, I)
        bw = oracle.backward_soft(ctx, en, gn, fw["edge_label"], given)
    else:
        fw = oracle.forward("TRWP", un, ctx, en, D, I)
        bw = oracle.backward("TRWP", ctx, en, gn, fw["min_idx"], given, keep_diag=True)
    assert rel_err(u.grad.permute(0, 1, 3, 4, 2).cpu().numpy(), bw["dunary"]) < GRAD_RTOL
    with pytest.raises(RuntimeError, match="msg_norm_index"):
        mod(u, e, msg_norm_index=torch.zeros(1, D, 1, 1, 9, 10, dtype=torch.uint8))
    with pytest.raises(RuntimeError, match="n_disp"):
        mod(u, e, msg_norm_index=torch.full((I, D, 1, 1, 9, 10), 200, dtype=torch.uint8))


def test_energy_mat_file(tmp_path):
    scio = pytest.importorskip("scipy.io")
    from mplayers_b200 import energy
    H, W, L, I, D = 6, 7, 5, 3, 4
    unary = torch.rand(1, 1, H, W, L, device="cuda")
    ctx = torch.rand(L, L, device="cuda")
    labels = torch.randint(0, L, (I, 1, 1, H, W), dtype=torch.uint8, device="cuda")
    path = str(tmp_path / "run.mat")
    energy.save_energy_mat(path, unary, ctx, labels, I, D, 0.5, "TL", 10, 2)
    m = scio.loadmat(path)
    assert m["unary"].shape == (H, W, L) and m["label_context"].shape == (L, L, D) and m["seg_all"].shape == (H, W, I)
    assert np.array_equal(m["seg_all"][:, :, 1], labels[1, 0, 0].cpu().numpy()) and int(m["n_disp"].item()) == L
