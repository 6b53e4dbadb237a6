"""Double-buffered host-to-device feeding for callers whose inputs live in (pinned) host memory.

The layers run on the current stream; a training or inference loop that reads its inputs from the
host every step spends a PCIe copy in front of every call (52 MB per step for the segmentation
configuration, about a millisecond).  `HostFeeder` issues the copy of step i + 1 on a side stream
while step i computes, into one of two device buffer sets, with events in both directions (the
compute stream waits for the copy; the next copy into the same set waits for the compute that
used it), so the copy disappears behind the kernels.  Plumbing only: torch streams and events.
"""
import torch


class HostFeeder:
    """feeder = HostFeeder([unary_host, weights_host], device); then per step
    `tensors = feeder.get(host_tensors)` returns device copies, already prefetched when
    `feeder.prefetch(next_host_tensors)` was called during the previous step; call
    `feeder.release()` after the step's kernels have been enqueued."""

    def __init__(self, like, device, depth=2):
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device)
        self.depth = depth
        self.bufs = [[None if t is None else torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in like]
                     for _ in range(depth)]
        self.ready = [torch.cuda.Event() for _ in range(depth)]   # copy into the set has finished
        self.free = [torch.cuda.Event() for _ in range(depth)]    # compute that used the set has finished
        self.used = [False] * depth
        self.next_in = 0     # set the next prefetch writes
        self.next_out = 0    # set the next get() hands out
        self.pending = 0

    def prefetch(self, host_tensors):
        if self.pending >= self.depth:
            raise RuntimeError("more prefetches in flight than buffer sets")
        k = self.next_in
        with torch.cuda.stream(self.stream):
            if self.used[k]:
                self.stream.wait_event(self.free[k])
            for dst, src in zip(self.bufs[k], host_tensors):
                if dst is not None:
                    dst.copy_(src, non_blocking=True)
            self.ready[k].record(self.stream)
        self.next_in = (k + 1) % self.depth
        self.pending += 1

    def get(self, host_tensors=None):
        """Device tensors of the oldest prefetched step (prefetching `host_tensors` now if nothing
        is in flight); the current stream is made to wait for their copy."""
        if self.pending == 0:
            self.prefetch(host_tensors)
        k = self.next_out
        torch.cuda.current_stream(self.device).wait_event(self.ready[k])
        self.current = k
        self.next_out = (k + 1) % self.depth
        self.pending -= 1
        return self.bufs[k]

    def release(self):
        """Marks the end of the work that reads the set handed out by the last get()."""
        k = self.current
        self.free[k].record(torch.cuda.current_stream(self.device))
        self.used[k] = True
