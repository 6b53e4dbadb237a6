"""Stand-alone soft-weighted message ops (`soft_weighted_message`, `soft_weighted_message_back` of
the reference's TRWP_hard_soft extension) against the float64 restatement, and next to the
reference's own CUDA kernels where those are built.  Floating point: 1e-5 of the largest value
for the forward, 1e-4 for the gradient; the index of the minimum must agree wherever the two
smallest column sums are further apart than that tolerance."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oracle import ref_cuda, terms as oracle_terms  # noqa: E402
from tests.helpers import COST_RTOL, GRAD_RTOL, rel_err  # noqa: E402

pytestmark = pytest.mark.gpu


def _run(mod, message, dnorm):
    import torch
    T, L, _ = message.shape
    norm = message.new_zeros(T, L)
    ind = torch.zeros(T, 1, dtype=torch.uint8, device=message.device)
    mod.soft_weighted_message(message, norm, ind)
    dmsg = torch.zeros_like(message)
    mod.soft_weighted_message_back(dnorm, message, ind, dmsg)
    return norm, ind, dmsg


@pytest.mark.parametrize("T,L,scale", [(1024, 21, 1.0), (300, 5, 4.0), (64, 32, 2.0), (40, 64, 1.0), (9, 200, 3.0),
                                       (3, 256, 1.0), (5, 1, 1.0)])
def test_against_restatement(T, L, scale):
    import torch
    import mplayers_b200
    g = torch.Generator().manual_seed(T + L)
    message = (torch.rand(T, L, L, generator=g) * scale).cuda()
    dnorm = (torch.rand(T, L, generator=g) - 0.3).cuda()
    norm, ind, dmsg = _run(mplayers_b200.TRWP, message, dnorm)
    enorm, eind, esoft = oracle_terms.soft_weighted_message(message.cpu().numpy())
    ind = ind.cpu().numpy().reshape(-1)
    srt = np.sort(esoft, axis=1)
    clear = (srt[:, 1] - srt[:, 0] > 1e-5 * max(np.abs(esoft).max(), 1e-30)) if L > 1 else np.ones(T, bool)
    assert np.array_equal(ind[clear], eind[clear])
    # compare the normalised sums against the restatement normalised at OUR index
    mine = esoft - np.take_along_axis(esoft, ind[:, None].astype(np.int64), 1)
    assert np.abs(norm.cpu().numpy() - mine).max() <= COST_RTOL * max(np.abs(esoft).max(), 1e-30)
    assert rel_err(dmsg.cpu().numpy(), oracle_terms.soft_weighted_message_back(dnorm.cpu().numpy(),
                                                                               message.cpu().numpy(), ind)) < GRAD_RTOL


def test_highest_index_wins_ties_and_empty_stack():
    import torch
    import mplayers_b200
    message = torch.zeros(2, 6, 6, device="cuda")          # every column sum is 0
    norm, ind, _ = _run(mplayers_b200.TRWP, message, torch.ones(2, 6, device="cuda"))
    assert ind.cpu().reshape(-1).tolist() == [5, 5] and float(norm.abs().max()) == 0.0
    empty = torch.zeros(0, 6, 6, device="cuda")
    _run(mplayers_b200.TRWP, empty, torch.zeros(0, 6, device="cuda"))
    with pytest.raises(RuntimeError, match="T,L,L"):
        mplayers_b200.TRWP.soft_weighted_message(torch.zeros(2, 5, 6, device="cuda"), torch.zeros(2, 6, device="cuda"),
                                                 torch.zeros(2, 1, dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("T,L", [(512, 32), (128, 64)])
def test_next_to_reference_cuda(T, L):
    """Label counts that fill whole warps: for others the reference's warp sums read lanes that do
    not take part in the shuffle (TRWP_swbp.cu:47-70), so its result is not defined."""
    if not ref_cuda.available("TRWP_hard_soft"):
        pytest.skip("reference CUDA extension TRWP_hard_soft not built (python oracle/build.py --ref-cuda)")
    import torch
    import mplayers_b200
    ref_mod = ref_cuda._load("TRWP_hard_soft")
    g = torch.Generator().manual_seed(L)
    message = torch.rand(T, L, L, generator=g).cuda()
    dnorm = torch.rand(T, L, generator=g).cuda()
    a = _run(mplayers_b200.TRWP, message, dnorm)
    b = _run(ref_mod, message, dnorm)
    assert torch.equal(a[1], b[1])
    assert rel_err(a[0].cpu().numpy(), b[0].cpu().numpy()) < COST_RTOL
    assert rel_err(a[2].cpu().numpy(), b[2].cpu().numpy()) < GRAD_RTOL
