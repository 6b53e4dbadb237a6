"""The extension-level forward and backward are plain asynchronous launches on the current stream
(no allocation, no synchronisation inside the library for training-mode calls), so a whole
forward + backward step can be captured into a CUDA graph and replayed: same results as the eager
calls, and no host work per step beyond one graph launch."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tensors(mode, B, H, W, L, D, I, seed):
    g = torch.Generator().manual_seed(seed)
    dev = "cuda"
    unary = torch.randn(B, 1, H, W, L, generator=g).to(dev)
    a = torch.triu(torch.rand(L, L, generator=g) * 2, 1)
    ctx = (a + a.t()).to(dev)
    ew = (torch.rand(D, B, 1, H, W, generator=g) * 0.8 + 0.2).to(dev)
    dcost = torch.rand(B, 1, H, W, L, generator=g).to(dev)
    z = lambda *s, **k: torch.zeros(*s, device=dev, **k)  # noqa: E731
    t = dict(unary=unary, ctx=ctx, ew=ew, dcost=dcost, msg=z(D, B, 1, H, W, L), msg2=z(D, B, 1, H, W, L),
             cost=z(B, 1, H, W, L), mi=z(I, D, B, 1, H, W, L, dtype=torch.uint8),
             ni=z(I, D, B, 1, H, W, dtype=torch.uint8), lab=torch.empty(0, dtype=torch.uint8, device=dev),
             none=torch.empty(0, device=dev), dun=z(B, 1, H, W, L), dctx=z(L, L), dew=z(D, B, 1, H, W),
             dmsg=z(D, B, 1, H, W, L), dmsg2=z(D, B, 1, H, W, L))
    return t


def _step(mode, t, I):
    from mplayers_b200 import ISGMR, TRWP
    # the library expects zeroed message / accumulation buffers on entry
    t["msg"].zero_(), t["msg2"].zero_(), t["dctx"].zero_(), t["dew"].zero_()
    if mode == "TRWP":
        TRWP.forward(0.5, I, 0, t["unary"], t["ctx"], t["ew"], t["msg"], t["cost"], t["mi"], t["ni"], t["none"], t["lab"])
        TRWP.backward(0.5, t["ctx"], t["ew"], t["dcost"], t["mi"], t["ni"], t["dun"], t["dctx"], t["dew"], t["dmsg"],
                      t["none"])
    else:
        ISGMR.forward(0, 1.0, I, 0, t["unary"], t["ctx"], t["ew"], t["msg"], t["cost"], t["mi"], t["ni"], t["none"],
                      t["msg2"], t["lab"])
        ISGMR.backward(0, 1.0, t["ctx"], t["ew"], t["dcost"], t["mi"], t["ni"], t["dun"], t["dctx"], t["dew"],
                       t["dmsg"], t["none"], t["dmsg2"])


@pytest.mark.parametrize("mode,shape", [("TRWP", (2, 32, 48, 21, 4, 3)), ("ISGMR", (1, 24, 40, 21, 8, 2)),
                                        ("ISGMR", (1, 20, 24, 64, 8, 2))])
def test_forward_backward_step_replays_from_a_cuda_graph(mode, shape, monkeypatch):
    B, H, W, L, D, I = shape
    monkeypatch.setenv("MPL_CHECK_STATUS", "0")   # the status read-back synchronises: not capturable
    t = _tensors(mode, B, H, W, L, D, I, seed=3)
    _step(mode, t, I)                              # eager: warms caches (tensor maps, attributes)
    torch.cuda.synchronize()
    want = {k: t[k].clone() for k in ("cost", "msg", "mi", "ni", "dun", "dctx", "dew")}

    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        _step(mode, t, I)                          # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        _step(mode, t, I)
    # new inputs in the captured buffers, replay, compare with an eager run on the same inputs
    g = torch.Generator().manual_seed(11)
    new_unary = torch.randn(B, 1, H, W, L, generator=g).cuda()
    t["unary"].copy_(new_unary)
    graph.replay()
    torch.cuda.synchronize()
    got = {k: t[k].clone() for k in want}
    _step(mode, t, I)
    torch.cuda.synchronize()
    for k in want:
        assert torch.equal(got[k], t[k]), k
    assert not torch.equal(got["cost"], want["cost"])   # the replay really used the new inputs


@pytest.mark.parametrize("window", [0, 2])
def test_rank1_inference_is_capturable(window, monkeypatch):
    """Inference with a rank-1 context and more than 32 labels.  Outside a capture the library may read
    its context analysis back (it waits for the stream); inside one it must not: with
    context_window = 0 it evaluates all candidates instead, with the caller's statement
    (context_window = R) it runs the windowed kernels.  Either way the captured call replays to the
    eager result."""
    from mplayers_b200 import TRWP
    monkeypatch.setenv("MPL_CHECK_STATUS", "0")
    L, D, I, H, W = 96, 4, 2, 12, 16
    g = torch.Generator().manual_seed(5)
    unary = torch.randn(1, 1, H, W, L, generator=g).cuda()
    ctx = torch.clamp(torch.arange(L, dtype=torch.float32), max=2.0).cuda()
    none, lab = torch.empty(0, device="cuda"), torch.empty(0, dtype=torch.uint8, device="cuda")
    msg, cost = torch.zeros(D, 1, 1, H, W, L, device="cuda"), torch.zeros(1, 1, H, W, L, device="cuda")

    def run():
        msg.zero_()
        TRWP.forward(0.5, I, 0, unary, ctx, none, msg, cost, lab, lab, none, lab, context_window=window)

    run()
    torch.cuda.synchronize()
    want = cost.clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run()
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        run()
    cost.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(cost, want)
