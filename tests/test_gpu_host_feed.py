"""HostFeeder: the prefetched device copies are the host tensors of the step they were issued for,
also when the host buffers are rewritten between steps and the consumer lags behind."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_prefetched_copies_arrive_in_order_and_survive_reuse():
    from mplayers_b200.host_feed import HostFeeder
    dev = torch.device("cuda", 0)
    steps = [[torch.full((257, 33), float(i)).pin_memory(), torch.arange(100, dtype=torch.float32).add_(i).pin_memory()]
             for i in range(7)]
    feeder = HostFeeder(steps[0], dev)
    sums = []
    feeder.prefetch(steps[0])
    for i in range(len(steps)):
        a, b = feeder.get()
        if i + 1 < len(steps):
            feeder.prefetch(steps[i + 1])
        # a long-running consumer of the set: the next copy into this set must wait for it
        x = a
        for _ in range(50):
            x = x * 1.0 + 0.0
        sums.append((x.sum() + b.sum()).clone())
        feeder.release()
    torch.cuda.synchronize()
    for i, s in enumerate(sums):
        want = 257 * 33 * float(i) + (sum(range(100)) + 100 * i)
        assert float(s) == want


def test_get_without_prefetch_and_none_entries():
    from mplayers_b200.host_feed import HostFeeder
    dev = torch.device("cuda", 0)
    h = torch.randn(64, 64).pin_memory()
    feeder = HostFeeder([h, None], dev)
    a, b = feeder.get([h, None])
    feeder.release()
    torch.cuda.synchronize()
    assert b is None and torch.equal(a.cpu(), h)
    with pytest.raises(RuntimeError):
        feeder.prefetch([h, None]), feeder.prefetch([h, None]), feeder.prefetch([h, None])
