"""ISGMR on ONE image spread over several GPUs by direction.

Within an ISGMR iteration every direction reads only the previous iteration's messages
(MPLayers/ISGMR/ISGMR_forward.cu:514-619), so the D sweeps are independent; what couples them is
the per-pixel sum of all directions' messages that the next iteration's update
UU_d = (U + sum_k M_k - M_d) * rho - M_inv(d) needs (ISGMR_forward.cu:101-121), and in the
backward pass the sum of all directions' scatter fields.  Rank r owns whole direction pairs
(d, d^1) -- so the partner message of every owned direction is local -- or, when there are more
ranks than pairs, one part of the chains of one pair (chains of a direction are independent of one
another, and both directions of a pair walk the same lines).  It runs its sweeps through the
iteration-level C ABI (mpl_isgmr_forward_directions & co. of include/mplayers_b200.h) on buffers
that hold only the slices it owns, and the ranks exchange exactly one all-reduce (sum) of a
[B,cv,H,W,L] field per iteration and pass, plus one small all-reduce of the label-context gradient
and one of the edge-weight gradients at the end.  Up to four ranks the field is summed and reduced in chunks: while
the collective works on one chunk the next one is being summed.  Every rank holds the whole image
and ends with the whole result.

The next iteration's sweeps need the reduced field at every pixel from their first step, so the
collective itself cannot hide behind sweeps: per iteration a rank spends (its share of the sweeps)
+ (one all-reduce of the field), and the second term does not shrink with the number of ranks.

The sum over directions is formed as (local partial sums) + all-reduce, not in the single-GPU
order, so results agree with the single-GPU layer to rounding (costs ~1e-6 relative; a saved
index can differ where two candidates are within rounding of each other), not bit for bit.

The batch-sharded mode of `parallel.py` is the scaling mode for training; this one shortens the
latency of one large image (batch 1), which batch sharding cannot split.
"""
import ctypes

import torch
import torch.distributed as dist

from . import _lib


def direction_shards(n_dir, world_size):
    """[(first_direction, direction_count)] per rank: contiguous runs of whole pairs (d, d^1); the
    first `pairs % world_size` ranks own one pair more; ranks beyond the pair count own nothing
    (they still take part in the collectives)."""
    if n_dir < 2 or n_dir % 2:
        raise ValueError("n_dir must be even and >= 2, got %d" % n_dir)
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    pairs = n_dir // 2
    base, rem = divmod(pairs, world_size)
    out, lo = [], 0
    for r in range(world_size):
        n = base + (1 if r < rem else 0)
        out.append((2 * lo, 2 * n))
        lo += n
    return out


def shard_plan(n_dir, world_size):
    """[(first_direction, direction_count, chain_part, chain_parts)] per rank.  Up to n_dir/2 ranks:
    whole pairs as in direction_shards, every chain of them.  More ranks: world_size // (n_dir/2)
    ranks share each pair, each taking one part of its chains; ranks left over own nothing."""
    pairs = n_dir // 2
    if world_size <= pairs:
        return [(f, c, 0, 1) for f, c in direction_shards(n_dir, world_size)]
    if n_dir < 2 or n_dir % 2:
        raise ValueError("n_dir must be even and >= 2, got %d" % n_dir)
    per_pair = world_size // pairs
    plan = []
    for r in range(world_size):
        if r < pairs * per_pair:
            plan.append((2 * (r // per_pair), 2, r % per_pair, per_pair))
        else:
            plan.append((n_dir, 0, 0, 1))
    return plan


class TorchDistComm:
    """The collectives of this module over torch.distributed (NCCL on GPUs)."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)

    def all_reduce(self, t):
        if self.world_size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def all_reduce_async(self, t):
        """Starts the all-reduce of `t` behind the work already queued on the current stream and
        returns a handle; later work on the current stream does not wait for it until wait()."""
        if self.world_size > 1:
            return dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        return None

    @staticmethod
    def wait(handle):
        if handle is not None:
            handle.wait()   # the current stream waits; the host does not


def _owned_ptr(t, d0):
    """Pointer the C ABI can index by ABSOLUTE direction for a tensor that holds only the slices
    d0 .. d0+dc-1 ([dc, ...]): the address slice d0 would have if slices 0 .. d0-1 preceded it.
    Only owned slices are ever dereferenced.  None for an empty tensor."""
    if t is None or t.numel() == 0:
        return None
    return ctypes.c_void_p(t.data_ptr() - d0 * t[0].numel() * t.element_size())


class CudaBackend:
    """The iteration-level entry points of the C ABI on torch CUDA tensors (current stream).
    Per-direction tensors hold the owned slices only ([dc, ...])."""

    @staticmethod
    def problem(unary, n_iter, n_dir, context, rho, enable_sgm, keep_diag=0, part=0, parts=1):
        b, cv, h, w, l = unary.shape
        return _lib.Problem(int(n_iter), int(n_dir), b, cv, h, w, l, _lib.context_rank(context, l), 0,
                            int(enable_sgm), int(keep_diag), float(rho), 0, int(part), int(parts))

    @staticmethod
    def _ws(prob, dev, backward):
        f = _lib.lib().mpl_backward_workspace_bytes if backward else _lib.lib().mpl_forward_workspace_bytes
        n = f(ctypes.byref(prob))
        return _lib.workspace(n, dev), n

    def forward_directions(self, prob, d0, dc, aggregate, context, ew, msg_read, msg_write, min_idx, norm_idx):
        if dc == 0:
            return
        dev = aggregate.device
        with torch.cuda.device(dev):
            ws, n = self._ws(prob, dev, False)
            _lib.check(_lib.lib().mpl_isgmr_forward_directions(
                ctypes.byref(prob), d0, dc, _lib.ptr(aggregate), _lib.ptr(context), _lib.ptr(ew),
                _owned_ptr(msg_read, d0), _owned_ptr(msg_write, d0), _owned_ptr(min_idx, d0),
                _owned_ptr(norm_idx, d0), _lib.ptr(ws), n, _lib.stream_ptr(dev)))
            _lib.check_status(ws, "ISGMR forward (direction-sharded)")

    def sum_directions(self, prob, d0, dc, fields, out, first=0, count=None, base=None):
        """out[first : first + count] (flat) = base + sum over the owned slices of `fields`
        (base None: plain sum; zeros when nothing is owned)."""
        dev = out.device
        count = out.numel() - first if count is None else count
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().mpl_sum_directions_range(
                ctypes.byref(prob), d0 if dc else 0, dc, _lib.ptr(base) if base is not None else None, 1.0,
                _owned_ptr(fields, d0) if dc else None, _lib.ptr(out), int(first), int(count),
                _lib.stream_ptr(dev)))
        return out

    def backward_workspace(self, prob, dev):
        return self._ws(prob, dev, True)[0]

    def backward_directions(self, prob, d0, dc, context, ew, dmsg_update, min_idx, norm_idx, scatter, dew, ws,
                            clear):
        dev = ws.device
        with torch.cuda.device(dev):
            # with no owned direction the call only clears the workspace (the pointers are not used)
            one = _lib.ptr(ws)
            _lib.check(_lib.lib().mpl_isgmr_backward_directions(
                ctypes.byref(prob), d0 if dc else 0, dc, _lib.ptr(context), _lib.ptr(ew),
                _owned_ptr(dmsg_update, d0) if dc else one, _owned_ptr(min_idx, d0) if dc else one,
                _owned_ptr(norm_idx, d0) if dc else one, _owned_ptr(scatter, d0) if dc else one,
                (_owned_ptr(dew, d0) if dc else one) if ew is not None else None, _lib.ptr(ws),
                ws.numel(), int(clear), _lib.stream_ptr(dev)))
            _lib.check_status(ws, "ISGMR backward (direction-sharded)")

    def combine(self, prob, d0, dc, scatter_total, scatter, dmsg_update, dunary):
        dev = scatter_total.device
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().mpl_isgmr_backward_combine(
                ctypes.byref(prob), d0 if dc else 0, dc, _lib.ptr(scatter_total), _owned_ptr(scatter, d0),
                _owned_ptr(dmsg_update, d0), _lib.ptr(dunary), _lib.stream_ptr(dev)))

    def context_finish(self, prob, ws, dcontext):
        dev = dcontext.device
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().mpl_backward_context_finish(
                ctypes.byref(prob), _lib.ptr(ws), ws.numel(), _lib.ptr(dcontext), _lib.stream_ptr(dev)))


def _sum_and_reduce(backend, comm, prob, d0, dc, fields, out, chunks, base=None):
    """out = all-reduce over the ranks of (sum over this rank's slices of `fields`), formed chunk by
    chunk: the collective of chunk k runs while chunk k + 1 is being summed.  `base` (given on ONE
    rank only) is added to that rank's partial sum, so that it ends up in the total once."""
    n = out.numel()
    flat = out.view(-1)
    start = getattr(comm, "all_reduce_async", None)
    if start is None or chunks <= 1 or comm.world_size == 1:
        backend.sum_directions(prob, d0, dc, fields, out, base=base)
        comm.all_reduce(out)
        return out
    handles = []
    for k in range(chunks):
        lo, hi = n * k // chunks, n * (k + 1) // chunks
        backend.sum_directions(prob, d0, dc, fields, out, lo, hi - lo, base=base)
        handles.append(start(flat[lo:hi]))
    for h in handles:
        comm.wait(h)
    return out


class DirectionShardedISGMRFunction(torch.autograd.Function):
    """ISGMRFunction (pytorch/MP_module.py:89-161) with the directions of each iteration spread over
    the ranks of `comm`.  Same tensors in and out on EVERY rank (unary [B,cv,H,W,L], label_context
    [L] or [L,L], edge_weights [D,B,cv,H,W] or None); every rank returns the complete cost_final
    and receives the complete gradients.  Saving per-iteration labels and `enable_min_a_dir` are
    not offered in this mode."""
    # Pieces the per-iteration field is summed and all-reduced in, None = by world size.  Measured on
    # a 268 MB field over NVLink: the all-reduce takes 0.54 / 0.69 / 0.72 ms whole and 0.61 / 0.75 /
    # 1.14 ms in four pieces on 2 / 4 / 8 ranks, against 0.1 - 0.2 ms of summing that the pieces hide:
    # four pieces up to four ranks, one beyond.
    chunks = None

    @staticmethod
    def _chunks(world_size):
        c = DirectionShardedISGMRFunction.chunks
        return c if c is not None else (4 if world_size <= 4 else 1)

    @staticmethod
    def forward(ctx, unary, label_context, edge_weights, args, comm, backend):
        if getattr(args, "enable_min_a_dir", False) or getattr(args, "enable_saving_label", False):
            raise RuntimeError("direction sharding offers neither enable_min_a_dir nor per-iteration labels")
        b, cv, h, w, l = unary.shape
        rho, n_iter, n_dir, training = args.rho, int(args.mpnet_max_iter), int(args.mpnet_n_dirs), args.training
        sgm = int(bool(getattr(args, "enable_sgm", False)))
        factor = float(n_dir) if sgm else 1.0
        unary = unary.contiguous()
        label_context = label_context.contiguous()
        ew = edge_weights.contiguous() if edge_weights is not None else None
        d0, dc, part, parts = shard_plan(n_dir, comm.world_size)[comm.rank]
        prob = backend.problem(unary, n_iter, n_dir, label_context, rho, sgm, part=part, parts=parts)
        chunks = DirectionShardedISGMRFunction._chunks(comm.world_size)
        # only the owned slices exist here; pixels of chains another rank walks stay zero in them
        rd = unary.new_zeros(dc, b, cv, h, w, l)
        wr = unary.new_zeros(dc, b, cv, h, w, l)
        if training:
            min_idx = torch.zeros(n_iter, dc, b, cv, h, w, l, dtype=torch.uint8, device=unary.device)
            norm_idx = torch.zeros(n_iter, dc, b, cv, h, w, dtype=torch.uint8, device=unary.device)
        else:
            min_idx = norm_idx = None
        # The aggregate A = U + (sum over ALL directions of the newest messages) comes straight out of the
        # all-reduce: rank 0 adds the unaries to its partial sum.  The sweeps of the next iteration read
        # it, and the sum after them overwrites it (same stream, after the sweeps).
        aggregate = unary
        total = torch.empty_like(unary)
        for it in range(n_iter):
            backend.forward_directions(prob, d0, dc, aggregate, label_context, ew, rd, wr,
                                       min_idx[it] if training else None, norm_idx[it] if training else None)
            _sum_and_reduce(backend, comm, prob, d0, dc, wr, total, chunks,
                            base=unary if comm.rank == 0 else None)
            aggregate = total
            rd, wr = wr, rd
        if n_iter == 0:
            cost_final = unary * factor
        else:
            cost_final = total if factor == 1.0 else total.add_(unary, alpha=factor - 1.0)
        ctx.intermediate_results = (sgm, rho, min_idx, norm_idx, label_context, ew, comm, backend, d0, dc, n_dir,
                                    part, parts)
        return cost_final

    @staticmethod
    def backward(ctx, dcost_final):
        (sgm, rho, min_idx, norm_idx, label_context, ew, comm, backend, d0, dc, n_dir, part,
         parts) = ctx.intermediate_results
        del ctx.intermediate_results
        if min_idx is None:
            raise RuntimeError("backward needs the indices saved by a training-mode forward "
                               "(args.training was False)")
        g = dcost_final.contiguous()
        n_iter = min_idx.size(0)
        b, cv, h, w, l = g.shape
        factor = float(n_dir) if sgm else 1.0
        prob = backend.problem(g, n_iter, n_dir, label_context, rho, sgm, part=part, parts=parts)
        chunks = DirectionShardedISGMRFunction._chunks(comm.world_size)
        dunary = g * factor
        x = g.new_zeros(dc, b, cv, h, w, l)        # gradient w.r.t. the messages an iteration produced
        if dc:
            x[:] = g
        scatter = g.new_zeros(dc, b, cv, h, w, l)
        q_total = torch.empty_like(g)
        dew_own = g.new_zeros(dc, b, cv, h, w) if ew is not None else None
        ws = backend.backward_workspace(prob, g.device)
        for k, it in enumerate(range(n_iter - 1, -1, -1)):
            backend.backward_directions(prob, d0, dc, label_context, ew, x, min_idx[it], norm_idx[it], scatter,
                                        dew_own, ws, clear=(k == 0))
            _sum_and_reduce(backend, comm, prob, d0, dc, scatter, q_total, chunks)
            backend.combine(prob, d0, dc, q_total, scatter, x, dunary)
        dcontext = torch.zeros_like(label_context)
        if n_iter == 0:
            backend.backward_directions(prob, d0, 0, label_context, ew, x, min_idx, norm_idx, scatter, dew_own, ws,
                                        clear=True)
        backend.context_finish(prob, ws, dcontext)
        comm.all_reduce(dcontext)
        dew = None
        if ew is not None:
            dew = torch.zeros_like(ew)
            if dc:
                dew[d0:d0 + dc] = dew_own
            comm.all_reduce(dew)   # every (slice, pixel) is non-zero on at most one rank
        return dunary, dcontext, dew, None, None, None


def isgmr_direction_sharded(unary, label_context, edge_weights, args, group=None, comm=None, backend=None):
    """Runs ISGMR (or single-iteration SGM) on `unary` with each iteration's directions spread over
    the ranks of `group` (default: the world).  Call it on every rank with the same tensors."""
    comm = comm if comm is not None else TorchDistComm(group)
    backend = backend if backend is not None else CudaBackend()
    return DirectionShardedISGMRFunction.apply(unary, label_context, edge_weights, args, comm, backend)
