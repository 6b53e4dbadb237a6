"""Hard (min-sum) branch of the reference's pytorch/MP_module_hard_soft.py:13-182, the module
mpnet.py imports for TRWP (mpnet.py:8,35).  Same interface and return tuple; relative to
MP_module.MPModule it (i) multiplies `label_context` by `mpnet_term_weight` inside forward
(:151), (ii) keeps the label-context gradient on the diagonal (the TRWP_hard_soft backward does
not skip c == f), (iii) returns two extra values.  With `args.mpnet_enable_soft` the soft
(expected-value) branch runs: the message is the expectation of the edge values under softmin
weights; in training it saves the edge values [I,D,B,cv,H,W,L,L] (returned as `message_vector`)
and the normalisation indices (returned as `message_index`), as the reference does
(pytorch/MP_module_hard_soft.py:37-48,92-97); it is built for n_classes <= 64.
"""
import torch
import torch.nn as nn

from . import glue as _glue

from . import TRWP as _TRWP
from .MP_module import TRWPFunction as _TRWPFunctionBase
from .MP_module import _norm_index_override
from .label_context import create_label_context


class TRWPFunction(_TRWPFunctionBase):
    keep_diag = True


class TRWPSoftFunction(torch.autograd.Function):
    """Soft branch of pytorch/MP_module_hard_soft.py:13-110.  Returns (cost_final, label_all,
    message_edge_label, cost_index)."""

    @staticmethod
    def forward(ctx, unary, label_context, edge_weights, args):
        batch, cv, h, w, n_disp = unary.size()
        rho, n_iter, n_dir, is_training = args.rho, args.mpnet_max_iter, args.mpnet_n_dirs, args.training
        dev = unary.device
        unary = unary.contiguous()
        label_context = label_context.contiguous()
        message = unary.new_zeros(n_dir, batch, cv, h, w, n_disp)
        cost_final = torch.empty_like(unary)
        e0 = torch.empty(0, dtype=torch.float32, device=dev)
        e8 = torch.empty(0, dtype=torch.uint8, device=dev)
        enable_edge_weights = edge_weights is not None
        ew = edge_weights.contiguous() if enable_edge_weights else e0
        label_all = torch.zeros(n_iter, batch, cv, h, w, dtype=torch.uint8, device=dev) \
            if args.enable_saving_label else e8
        if is_training:
            # entries of pixels without a predecessor are never written and stay 0, as in the reference
            message_edge_label = unary.new_zeros(n_iter, n_dir, batch, cv, h, w, n_disp, n_disp)
            cost_index = torch.zeros(n_iter, n_dir, batch, cv, h, w, dtype=torch.uint8, device=dev)
        else:
            message_edge_label, cost_index = e0, e8
        _TRWP.forward_soft(rho, int(n_iter), unary, label_context, ew, message, message_edge_label,
                           cost_index, cost_final, e0, label_all)
        ctx.intermediate_results = rho, message_edge_label, cost_index, label_context, ew, enable_edge_weights
        ctx.norm_index_override = _norm_index_override(args, cost_index, n_disp)
        ctx.mark_non_differentiable(label_all, message_edge_label, cost_index)
        return cost_final, label_all, message_edge_label, cost_index

    @staticmethod
    def backward(ctx, dcost_final, dlabel_all, dmessage_edge_label, dcost_index):
        rho, message_edge_label, cost_index, label_context, ew, enable_edge_weights = ctx.intermediate_results
        del ctx.intermediate_results
        if cost_index.numel() == 0:
            raise RuntimeError("backward needs the edge values saved by a training-mode forward "
                               "(args.training was False)")
        if ctx.norm_index_override is not None:
            cost_index = ctx.norm_index_override
        dcost_final = dcost_final.contiguous()
        n_iter, n_dir, batch, cv, h, w = cost_index.size()
        n_disp = dcost_final.size(-1)
        dunary = torch.empty_like(dcost_final)
        dmessage = dcost_final.new_empty(n_dir, batch, cv, h, w, n_disp)
        dlabel_context = torch.zeros_like(label_context)
        e0 = torch.empty(0, dtype=torch.float32, device=dcost_final.device)
        dedge_weights = torch.zeros_like(ew) if enable_edge_weights else e0
        _TRWP.backward_soft(rho, dcost_final, label_context, ew, message_edge_label, cost_index, dunary,
                            dlabel_context, dedge_weights, dmessage, e0)
        return dunary, dlabel_context, (dedge_weights if enable_edge_weights else None), None


class MPModule(torch.nn.Module):
    def __init__(self, args, enable_create_label_context=False, enable_saving_label=False):
        super(MPModule, self).__init__()
        self.args = args
        self.args.enable_saving_label = enable_saving_label
        self.args.rho = 0.5 if (args.mpnet_mrf_mode == 'TRWP') else 1
        self.args.enable_seg = True if (args.n_classes == 21) else False
        self.args.enable_min_a_dir = False
        if enable_create_label_context:
            self.create_label_context()

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

    def forward(self, unary, edge_weights=None, msg_norm_index=None, pairwise_terms=None):
        # pytorch/MP_module_hard_soft.py:169-171: indices given here replace the saved
        # normalisation indices in the backward pass
        self.args.msg_norm_index = msg_norm_index
        assert self.args.mpnet_mrf_mode == 'TRWP'
        unary = _glue.labels_last(unary)
        edge_weights = edge_weights.unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous() \
            if (edge_weights is not None) else edge_weights
        label_context = self.label_context * self.args.mpnet_term_weight
        train = getattr(self.args, 'mpnet_smoothness_train', None)
        if train == 'sigmoid':
            valid = label_context[self.label_context_loc].flatten()
            label_context[self.label_context_loc] = 2 * torch.sigmoid(valid)
        elif train == 'softmax':
            valid = label_context[self.label_context_loc].flatten()
            norm = nn.Softmax(dim=0)(valid)
            label_context[self.label_context_loc] = norm * valid.max() / norm.max()
        if train in {'sigmoid', 'softmax'}:
            label_context[self.label_context_diag_loc] = self.args.mpnet_diag_value
        if edge_weights is not None:
            assert unary.size()[-3:-1] == edge_weights.size()[-2:]
        self.args.training = self.training
        self.args.cost_labels_first = False
        if getattr(self.args, 'mpnet_enable_soft', False):
            cost_final, cost_all, message_vector, message_index = \
                TRWPSoftFunction.apply(unary, label_context, edge_weights, self.args)
            cost_final = _glue.labels_first(cost_final)
            return cost_final, label_context.unsqueeze(0), cost_all, message_vector, message_index
        # the layer writes cost_final (and reads its gradient) with the labels first: no layout pass
        # on the way out (pytorch/MP_module_hard_soft.py permutes here)
        self.args.cost_labels_first = True
        cost_final, cost_all = TRWPFunction.apply(unary, label_context, edge_weights, self.args)
        self.args.cost_labels_first = False
        label_context = label_context.unsqueeze(0)
        empty = torch.empty(0, dtype=torch.float32, device=unary.device)
        return cost_final, label_context, cost_all, empty, empty
