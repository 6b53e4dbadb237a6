"""Operator API of the TRWP / ISGMR message-passing layers: `MPModule`, `TRWPFunction`,
`ISGMRFunction`, with the interface of the reference's pytorch/MP_module.py:17-234 (same
constructor arguments, same `args` attributes read and written, same tensor layouts in and out),
so that the reference's callers (mpnet.py:168, MPLayers/main.py:257-290) work unchanged.

Under the API everything runs in hand-written sm_100a kernels behind a C ABI
(include/mplayers_b200.h).  Differences from the reference that a caller can observe:
  * the context convention follows the rank of `label_context` ([L] or [L,L]) rather than
    `n_disp == 21`, so `dlabel_context` always has the shape of `label_context`;
  * no `unary_update`-style scratch tensors are allocated (the kernels are fused);
  * when `edge_weights` is None no tensor of ones is materialised;
  * CUDA tensors only: there is no CPU path, CPU inputs raise.
"""
import torch
import torch.nn as nn

from . import glue as _glue

from . import ISGMR as _ISGMR
from . import TRWP as _TRWP
from .label_context import create_label_context


def _empty_u8(device):
    return torch.empty(0, dtype=torch.uint8, device=device)


def _alloc_indices(unary, n_iter, n_dir, is_training, enable_saving_label):
    batch, cv, h, w, n_disp = unary.size()
    dev = unary.device
    if is_training:
        # Every entry that a sweep visits is overwritten and the backward pass reads exactly those
        # (pixels without a predecessor have no index: the reference leaves its zero fill there,
        # pytorch/MP_module.py:34-35).  The two tensors never leave the autograd context, so they
        # are not cleared: 231 MB of memset per segmentation training step.
        message_index = torch.empty(n_iter, n_dir, batch, cv, h, w, n_disp, dtype=torch.uint8, device=dev)
        cost_index = torch.empty(n_iter, n_dir, batch, cv, h, w, dtype=torch.uint8, device=dev)
    else:
        message_index, cost_index = _empty_u8(dev), _empty_u8(dev)
    if enable_saving_label:
        label_all = torch.zeros(n_iter, batch, cv, h, w, dtype=torch.uint8, device=dev)
    else:
        label_all = _empty_u8(dev)
    return message_index, cost_index, label_all


def _norm_index_override(args, cost_index, n_disp):
    """The `msg_norm_index` hook of pytorch/MP_module_hard_soft.py:76,169-171: normalisation
    indices supplied by the caller replace the saved ones in the backward pass (the forward pass
    is unaffected).  Returns the tensor to use, or None."""
    given = getattr(args, "msg_norm_index", None)
    if given is None:
        return None
    if cost_index.numel() == 0:
        return None   # inference: there is no backward
    given = given.to(device=cost_index.device, dtype=torch.uint8).contiguous()
    if given.shape != cost_index.shape:
        raise RuntimeError("msg_norm_index must be [I,D,B,cv,H,W] = %s, got %s" %
                           (tuple(cost_index.shape), tuple(given.shape)))
    if int(given.max()) >= n_disp:
        raise RuntimeError("msg_norm_index holds a label >= n_disp (%d)" % n_disp)
    return given


class TRWPFunction(torch.autograd.Function):
    """pytorch/MP_module.py:17-86.  unary [B,cv,H,W,L]; label_context [L] or [L,L];
    edge_weights [D,B,cv,H,W] or None.  Returns (cost_final [B,cv,H,W,L], label_all)."""
    keep_diag = False

    @staticmethod
    def forward(ctx, unary, label_context, edge_weights, args):
        batch, cv, h, w, n_disp = unary.size()
        rho, n_iter, n_dir, is_training = args.rho, args.mpnet_max_iter, args.mpnet_n_dirs, args.training
        unary = unary.contiguous()
        label_context = label_context.contiguous()
        message = unary.new_zeros(n_dir, batch, cv, h, w, n_disp)
        lf = bool(getattr(args, "cost_labels_first", False))  # cost_final as [B,cv,L,H,W]
        cost_final = unary.new_empty(batch, cv, n_disp, h, w) if lf else torch.empty_like(unary)
        message_index, cost_index, label_all = _alloc_indices(unary, n_iter, n_dir, is_training,
                                                              args.enable_saving_label)
        enable_edge_weights = edge_weights is not None
        ew = edge_weights.contiguous() if enable_edge_weights else _empty_f32(unary.device)
        _TRWP.forward(rho, int(n_iter), int(args.enable_min_a_dir), unary, label_context, ew, message,
                      cost_final, message_index, cost_index, _empty_f32(unary.device), label_all,
                      context_window=int(getattr(args, "context_window", 0) or 0), cost_labels_first=lf)
        ctx.cost_labels_first = lf
        ctx.intermediate_results = rho, message_index, cost_index, label_context, ew, enable_edge_weights
        ctx.context_window = int(getattr(args, "context_window", 0) or 0)
        ctx.norm_index_override = _norm_index_override(args, cost_index, n_disp)
        ctx.mark_non_differentiable(label_all)
        return cost_final, label_all

    @staticmethod
    def backward(ctx, dcost_final, dmessage_all):
        rho, message_index, cost_index, label_context, ew, enable_edge_weights = ctx.intermediate_results
        del ctx.intermediate_results
        if message_index.numel() == 0:
            raise RuntimeError("backward needs the indices saved by a training-mode forward "
                               "(args.training was False)")
        if ctx.norm_index_override is not None:
            cost_index = ctx.norm_index_override
        dcost_final = dcost_final.contiguous()
        n_iter, n_dir, batch, cv, h, w, n_disp = message_index.size()
        dunary = dcost_final.new_empty(batch, cv, h, w, n_disp)
        dmessage = dcost_final.new_empty(n_dir, batch, cv, h, w, n_disp)
        dlabel_context = torch.zeros_like(label_context)
        dedge_weights = torch.zeros_like(ew) if enable_edge_weights else _empty_f32(dcost_final.device)
        _TRWP.backward(rho, label_context, ew, dcost_final, message_index, cost_index, dunary,
                       dlabel_context, dedge_weights, dmessage, _empty_f32(dcost_final.device),
                       keep_diag=ctx._forward_cls.keep_diag, context_window=ctx.context_window,
                       cost_labels_first=ctx.cost_labels_first)
        return dunary, dlabel_context, (dedge_weights if enable_edge_weights else None), None


class ISGMRFunction(torch.autograd.Function):
    """pytorch/MP_module.py:89-161 (ISGMR and single-iteration SGM)."""

    @staticmethod
    def forward(ctx, unary, label_context, edge_weights, args):
        batch, cv, h, w, n_disp = unary.size()
        rho, n_iter, n_dir, is_training = args.rho, args.mpnet_max_iter, args.mpnet_n_dirs, args.training
        unary = unary.contiguous()
        label_context = label_context.contiguous()
        message = unary.new_zeros(n_dir, batch, cv, h, w, n_disp)
        message_tmp = unary.new_zeros(n_dir, batch, cv, h, w, n_disp)
        lf = bool(getattr(args, "cost_labels_first", False))  # cost_final as [B,cv,L,H,W]
        cost_final = unary.new_empty(batch, cv, n_disp, h, w) if lf else torch.empty_like(unary)
        message_index, cost_index, label_all = _alloc_indices(unary, n_iter, n_dir, is_training,
                                                              args.enable_saving_label)
        enable_edge_weights = edge_weights is not None
        ew = edge_weights.contiguous() if enable_edge_weights else _empty_f32(unary.device)
        _ISGMR.forward(int(args.enable_sgm), rho, int(n_iter), int(args.enable_min_a_dir), unary,
                       label_context, ew, message, cost_final, message_index, cost_index,
                       _empty_f32(unary.device), message_tmp, label_all,
                       context_window=int(getattr(args, "context_window", 0) or 0), cost_labels_first=lf)
        ctx.cost_labels_first = lf
        ctx.intermediate_results = args.enable_sgm, rho, message_index, cost_index, label_context, ew, \
            enable_edge_weights
        ctx.context_window = int(getattr(args, "context_window", 0) or 0)
        ctx.mark_non_differentiable(label_all)
        return cost_final, label_all

    @staticmethod
    def backward(ctx, dcost_final, dmessage_all):
        enable_sgm, rho, message_index, cost_index, label_context, ew, enable_edge_weights = \
            ctx.intermediate_results
        del ctx.intermediate_results
        if message_index.numel() == 0:
            raise RuntimeError("backward needs the indices saved by a training-mode forward "
                               "(args.training was False)")
        dcost_final = dcost_final.contiguous()
        n_iter, n_dir, batch, cv, h, w, n_disp = message_index.size()
        dunary = dcost_final.new_empty(batch, cv, h, w, n_disp)
        dmessage = dcost_final.new_empty(n_dir, batch, cv, h, w, n_disp)
        dmessage_tmp = dcost_final.new_empty(n_dir, batch, cv, h, w, n_disp)
        dlabel_context = torch.zeros_like(label_context)
        dedge_weights = torch.zeros_like(ew) if enable_edge_weights else _empty_f32(dcost_final.device)
        _ISGMR.backward(int(enable_sgm), rho, label_context, ew, dcost_final, message_index, cost_index,
                        dunary, dlabel_context, dedge_weights, dmessage,
                        _empty_f32(dcost_final.device), dmessage_tmp, context_window=ctx.context_window,
                        cost_labels_first=ctx.cost_labels_first)
        return dunary, dlabel_context, (dedge_weights if enable_edge_weights else None), None


def _empty_f32(device):
    return torch.empty(0, dtype=torch.float32, device=device)


class MPModule(torch.nn.Module):
    """pytorch/MP_module.py:164-234.  `args` is the reference's namespace; attributes read:
    mpnet_mrf_mode ('TRWP' | 'ISGMR' | 'SGM'), mpnet_max_iter, mpnet_n_dirs, n_classes,
    mpnet_smoothness_train, mpnet_term_weight, mpnet_diag_value, enable_symmetric (and the
    label-context builder's); attributes written: rho, enable_saving_label, enable_min_a_dir,
    enable_sgm, enable_seg, training."""

    def __init__(self, args, enable_create_label_context=False, enable_saving_label=False,
                 enable_min_a_dir=False):
        super(MPModule, self).__init__()
        self.args = args
        self.args.rho = 0.5 if (args.mpnet_mrf_mode == 'TRWP') else 1
        self.args.enable_saving_label = enable_saving_label
        self.args.enable_min_a_dir = enable_min_a_dir
        self.args.enable_sgm = args.mpnet_mrf_mode == 'SGM'
        self.args.enable_seg = True if (args.n_classes == 21) else False
        self.direction_comm = None
        if enable_create_label_context:
            self.create_label_context()

    def shard_directions(self, group=None, comm=None):
        """ISGMR / SGM only, no counterpart in the reference: from now on every rank of `group`
        (torch.distributed; default the world) calls this module with the SAME tensors, each
        iteration's directions are spread over the ranks, and every rank gets the complete result
        (direction_sharding.py).  `shard_directions(comm=False)` switches it off."""
        if comm is False:
            self.direction_comm = None
            return self
        if self.args.mpnet_mrf_mode not in {'ISGMR', 'SGM'}:
            raise RuntimeError("direction sharding needs independent directions: ISGMR / SGM only "
                               "(TRWP updates them one after the other)")
        if comm is None:
            from .direction_sharding import TorchDistComm
            comm = TorchDistComm(group)
        self.direction_comm = comm
        return self

    def get_label_context(self):
        return self.label_context, self.label_context_loc, self.label_context_diag_loc

    def set_label_context(self, label_context, label_context_loc, label_context_diag_loc):
        self.label_context = label_context
        self.label_context_loc = label_context_loc
        self.label_context_diag_loc = label_context_diag_loc

    def create_label_context(self):
        self.label_context, self.label_context_loc, self.label_context_diag_loc = \
            create_label_context(self.args, enable_seg=self.args.enable_seg,
                                 enable_symmetric=self.args.enable_symmetric)

    def _transformed_label_context(self):
        # pytorch/MP_module.py:208-220
        label_context = self.label_context * 1
        train = getattr(self.args, 'mpnet_smoothness_train', None)
        if train == 'sigmoid':
            valid = label_context[self.label_context_loc].flatten()
            label_context[self.label_context_loc] = 2 * self.args.mpnet_term_weight * torch.sigmoid(valid)
        elif train == 'softmax':
            valid = label_context[self.label_context_loc].flatten()
            norm = nn.Softmax(dim=0)(valid)
            label_context[self.label_context_loc] = norm * valid.max() / norm.max()
        if train in {'sigmoid', 'softmax'}:
            label_context[self.label_context_diag_loc] = self.args.mpnet_diag_value
        return label_context

    def _context_window(self, label_context, edge_weights):
        """A rank-1 context with more than 32 labels: the kernels' windowed evaluation needs to know
        where the context saturates.  The library can find out per call, but then the
        call waits for the stream; here the answer is computed once per state of the context
        parameter (its version counter tells when an optimiser step or an assignment changed it) and
        handed down as a statement (mpl_problem::context_window).  Only without edge weights: those
        are new tensors every call, and the statement covers them too."""
        if label_context.dim() != 1 or edge_weights is not None:
            return 0
        if label_context.numel() <= 32:
            return 0
        src = self.label_context
        key = (id(src), src._version, src.data_ptr(), getattr(self.args, 'mpnet_smoothness_train', None),
               getattr(self.args, 'mpnet_term_weight', None), getattr(self.args, 'mpnet_diag_value', None))
        if getattr(self, "_window_key", None) != key:
            from . import _lib
            self._window_value = _lib.analyze_context(label_context)
            self._window_key = key
        return self._window_value

    def forward_native(self, unary, edge_weights=None):
        """The layer in the extension's own layouts, without the two permutes of forward():
        unary [B,cv,H,W,L], edge_weights [D,B,cv,H,W] or None -> (cost_final [B,cv,H,W,L],
        label_context).  Used by glue.mp_on_scores."""
        label_context = self._transformed_label_context()
        self.args.training = self.training
        self.args.cost_labels_first = False
        self.args.context_window = self._context_window(label_context, edge_weights)
        if self.args.mpnet_mrf_mode in {'ISGMR', 'SGM'}:
            cost_final, _ = ISGMRFunction.apply(unary, label_context, edge_weights, self.args)
        else:
            cost_final, _ = TRWPFunction.apply(unary, label_context, edge_weights, self.args)
        return cost_final, label_context.unsqueeze(0)

    def forward(self, unary, edge_weights=None):
        # unary [B,cv,L,H,W]; edge_weights [B,D,H,W]
        unary = _glue.labels_last(unary)
        edge_weights = edge_weights.unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous() \
            if (edge_weights is not None) else edge_weights
        if self.args.mpnet_mrf_mode == 'SGM':
            assert self.args.mpnet_max_iter == 1
        label_context = self._transformed_label_context()
        if edge_weights is not None:
            assert unary.size()[-3:-1] == edge_weights.size()[-2:]
        self.args.training = self.training
        self.args.context_window = self._context_window(label_context, edge_weights)
        # The layer writes cost_final (and reads its gradient) with the labels first, the layout the
        # reference reaches with a permute here (pytorch/MP_module.py:232): no layout pass on the way
        # out.  (The direction-sharded mode keeps its own path.)
        self.args.cost_labels_first = self.direction_comm is None
        if self.args.mpnet_mrf_mode in {'ISGMR', 'SGM'} and self.direction_comm is not None:
            from .direction_sharding import isgmr_direction_sharded
            cost_final = isgmr_direction_sharded(unary, label_context, edge_weights, self.args,
                                                 comm=self.direction_comm)
            cost_final = _glue.labels_first(cost_final)
            cost_all = _empty_u8(unary.device)
        elif self.args.mpnet_mrf_mode in {'ISGMR', 'SGM'}:
            cost_final, cost_all = ISGMRFunction.apply(unary, label_context, edge_weights, self.args)
        elif self.args.mpnet_mrf_mode == 'TRWP':
            cost_final, cost_all = TRWPFunction.apply(unary, label_context, edge_weights, self.args)
        else:
            assert False
        self.args.cost_labels_first = False
        label_context = label_context.unsqueeze(0)
        return cost_final, label_context, cost_all, None, None
