"""CPU-only checks of the C-ABI library and the host-side layer: the library loads, exports
every symbol the header declares, validates its arguments before touching CUDA, and enumerates
chains correctly.  No compute call is made here."""
import ctypes
import os
import re
import types

import numpy as np
import pytest
import torch

from mplayers_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_exports_every_declared_symbol():
    with open(os.path.join(ROOT, "include", "mplayers_b200.h")) as f:
        header = f.read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    names = set(re.findall(r"\b(mpl_[a-z0-9_]+)\s*\(", header))
    assert {"mpl_trwp_forward", "mpl_trwp_backward", "mpl_isgmr_forward", "mpl_isgmr_backward",
            "mpl_last_error", "mpl_forward_workspace_bytes", "mpl_backward_workspace_bytes"} <= names
    lib = _lib.lib()
    for n in names:
        assert hasattr(lib, n), n
    assert lib.mpl_version() >= 100


def _prob(**kw):
    d = dict(n_iter=2, n_dir=4, batch=1, n_cv=1, height=8, width=9, n_disp=21, context_rank=2,
             enable_min_a_dir=0, enable_sgm=0, keep_diag=0, rho=0.5, context_window=0, chain_part=0, chain_parts=0,
             cost_labels_first=0)
    d.update(kw)
    return _lib.Problem(*[d[n] for n, _ in _lib.Problem._fields_])


@pytest.mark.parametrize("kw,code,word", [
    (dict(n_disp=300), 2, "n_disp"), (dict(n_disp=0), 2, "n_disp"), (dict(n_dir=3), 2, "n_dir"),
    (dict(n_dir=18), 2, "n_dir"), (dict(context_rank=3), 1, "context_rank"),
    (dict(height=0), 1, "shape"), (dict(height=70000, width=70000, n_disp=2), 2, "2^31"),
])
def test_rejects_bad_problems_before_any_cuda_call(kw, code, word):
    lib = _lib.lib()
    p = _prob(**kw)
    one = ctypes.c_void_p(16)   # never dereferenced: validation fails first
    rc = lib.mpl_trwp_forward(ctypes.byref(p), one, one, None, one, one, None, None, None, one, 1 << 20, None)
    assert rc == code
    assert word in lib.mpl_last_error().decode()
    rc = lib.mpl_isgmr_backward(ctypes.byref(p), one, None, one, one, one, one, one, None, one, one, one,
                                1 << 20, None)
    assert rc == code


def test_rejects_null_pointers_and_small_workspace():
    lib = _lib.lib()
    p = _prob()
    one = ctypes.c_void_p(16)
    rc = lib.mpl_trwp_forward(ctypes.byref(p), None, one, None, one, one, None, None, None, one, 1 << 20, None)
    assert rc == 1 and "NULL" in lib.mpl_last_error().decode()
    rc = lib.mpl_trwp_forward(ctypes.byref(p), one, one, None, one, one, one, None, None, one, 1 << 20, None)
    assert rc == 1 and "both" in lib.mpl_last_error().decode()
    rc = lib.mpl_trwp_backward(ctypes.byref(p), one, None, one, one, one, one, one, None, one, one, 8, None)
    assert rc == 1 and "workspace" in lib.mpl_last_error().decode()


def test_workspace_sizes():
    lib = _lib.lib()
    p = _prob(batch=2, height=512, width=512)
    assert lib.mpl_forward_workspace_bytes(ctypes.byref(p)) >= 16
    # a 256-byte header (context analysis, status word at byte 64) + one partial 21x21 table per chain
    # of all four directions (4 x 2 images x 512 rows; an ISGMR launch covers every direction at once)
    assert lib.mpl_backward_workspace_bytes(ctypes.byref(p)) == 256 + 4096 * 441 * 4
    assert lib.mpl_workspace_status_offset() == 64


@pytest.mark.parametrize("hw", [(1, 1), (1, 7), (5, 1), (2, 3), (6, 7), (13, 4)])
def test_chains_partition_the_image(hw):
    H, W = hw
    lib = _lib.lib()
    out = (ctypes.c_int32 * 5)()
    for d in range(16):
        cov = np.zeros((H, W), int)
        for t in range(lib.mpl_chain_count(d, H, W)):
            assert lib.mpl_chain_geometry(d, H, W, t, out) == 0
            h, w, n, hs, ws = list(out)
            assert not (0 <= h - hs < H and 0 <= w - ws < W)          # starts where there is no predecessor
            assert not (0 <= h + n * hs < H and 0 <= w + n * ws < W)  # ends where there is no successor
            for i in range(n):
                cov[h + i * hs, w + i * ws] += 1
        assert (cov == 1).all()
    assert lib.mpl_chain_count(16, H, W) == -1


def test_host_layer_rejects_cpu_and_strided_tensors():
    from mplayers_b200 import TRWP
    u = torch.zeros(1, 1, 4, 5, 3)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        TRWP.forward(0.5, 1, 0, u, torch.zeros(3, 3), torch.zeros(0), torch.zeros(4, 1, 1, 4, 5, 3),
                     torch.zeros_like(u), torch.zeros(0, dtype=torch.uint8), torch.zeros(0, dtype=torch.uint8),
                     torch.zeros(0), torch.zeros(0, dtype=torch.uint8))
    with pytest.raises(RuntimeError, match="contiguous"):
        _lib.require(torch.zeros(4, 6)[:, ::2], "x", torch.float32)
    with pytest.raises(RuntimeError, match="float32"):
        _lib.require(torch.zeros(4, dtype=torch.float64), "x", torch.float32)


def test_context_rank_rules():
    assert _lib.context_rank(torch.zeros(7), 7) == 1
    assert _lib.context_rank(torch.zeros(7, 7), 7) == 2
    assert _lib.context_rank(torch.zeros(4, 21, 21), 21) == 2     # the reference reads the first matrix
    assert _lib.context_rank(torch.zeros(4, 48, 48), 48) == 1     # ... or its first row as a function
    with pytest.raises(RuntimeError):
        _lib.context_rank(torch.zeros(5), 7)


def _args(n_classes, mode, train=None, trunc=-1, loc=-1, weight=2.0):
    return types.SimpleNamespace(n_classes=n_classes, mpnet_smoothness_mode=mode,
                                 mpnet_smoothness_train=train, mpnet_smoothness_trunct_value=trunc,
                                 mpnet_smoothness_trunct_loc=loc, mpnet_term_weight=weight,
                                 enable_cuda=False)


@pytest.mark.parametrize("n,mode,trunc,loc,sym", [
    (21, "Potts", -1, -1, True), (21, "TL", 3, -1, True), (21, "TQ", 5, 2, False),
    (21, "NPotts", -1, -1, True), (48, "TL", 2, -1, True), (48, "TQ", 30, 4, True), (16, "Potts", -1, -1, True),
])
def test_label_context_builder_matches_reference_when_present(n, mode, trunc, loc, sym):
    from mplayers_b200.label_context import create_label_context
    lc, where, diag = create_label_context(_args(n, mode, None, trunc, loc), enable_symmetric=sym)
    assert lc.shape == ((n, n) if n == 21 else (n,))
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref_dir = os.environ.get("MPL_REFERENCE_DIR", os.path.join(os.path.dirname(repo), "reference"))
    path = os.path.join(ref_dir, "utils", "label_context.py")
    if not os.path.exists(path):
        pytest.skip("reference checkout not present")
    import importlib.util
    spec = importlib.util.spec_from_file_location("_ref_label_context", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    want, wwhere, wdiag = mod.create_label_context(_args(n, mode, None, trunc, loc), enable_symmetric=sym)
    assert torch.equal(lc.detach(), want.detach())
    assert lc.requires_grad == want.requires_grad
    assert [np.asarray(x).tolist() for x in where] == [np.asarray(x).tolist() for x in wwhere] \
        if n == 21 else list(where) == list(wwhere)
