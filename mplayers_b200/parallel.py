"""Multi-GPU use of the layers: one process per GPU, the batch sharded across ranks.

Samples are independent in the forward and in the backward pass (no term of the reference's
kernels couples two batch entries, MPLayers/TRWP/TRWP_forward.cu:107), so every rank runs the layer
on its own slice with no data-path collective.  The only quantity that is a sum over samples is
the gradient of the shared `label_context` parameter: one all-reduce (sum) of L or L*L floats
after backward -- what the reference's nn.DataParallel wrapper does implicitly (main.py:113-115).
"""
import torch
import torch.distributed as dist


def shard_bounds(global_batch, rank, world_size):
    """Contiguous slice [lo, hi) of a batch of `global_batch` samples owned by `rank`; the first
    `global_batch % world_size` ranks own one sample more."""
    if not (0 <= rank < world_size):
        raise ValueError("rank %d outside world of %d" % (rank, world_size))
    base, rem = divmod(global_batch, world_size)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch(tensor, rank, world_size, dim=0):
    """This rank's slice of a batch-major tensor (a view)."""
    lo, hi = shard_bounds(tensor.size(dim), rank, world_size)
    return tensor.narrow(dim, lo, hi - lo)


def allreduce_label_context_grad(grad, group=None):
    """Sum the label-context gradient over all ranks, in place.  Accepts the gradient tensor or a
    parameter (whose .grad is reduced).  No-op without an initialised process group.

    A collective: EVERY rank of the group must call it once per step, also a rank whose parameter
    received no gradient in that step (its slice did not reach the layer).  Pass the parameter in
    that case: a missing .grad takes part as zeros and is set to the reduced sum, so the ranks stay
    in step instead of the others waiting forever.  A bare None cannot take part (its shape is
    unknown) and raises while a group is active."""
    param = None
    if isinstance(grad, torch.nn.Parameter):
        param, grad = grad, grad.grad
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return grad
    if grad is None:
        if param is None:
            raise RuntimeError("allreduce_label_context_grad(None): every rank must take part in the "
                               "all-reduce; pass the parameter so that zeros of its shape can be reduced")
        grad = torch.zeros_like(param)
        param.grad = grad
    dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=group)
    return grad


def attach_grad_allreduce(param, group=None):
    """Registers a hook that all-reduces `param.grad` as soon as backward has accumulated it.  The
    hook fires only on ranks whose backward reached the parameter; a rank that may skip the layer in
    some step must call allreduce_label_context_grad(param) itself in that step (see there)."""
    if not param.requires_grad:
        return None

    def hook(p):
        allreduce_label_context_grad(p, group)

    return param.register_post_accumulate_grad_hook(hook)
