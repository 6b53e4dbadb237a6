"""Hard (min-sum) branch of the reference's pytorch/MP_module_hard_soft.py:13-182, the module
mpnet.py imports for TRWP (mpnet.py:8,35).  Same interface and return tuple; relative to
MP_module.MPModule it (i) multiplies `label_context` by `mpnet_term_weight` inside forward
(:151), (ii) keeps the label-context gradient on the diagonal (the TRWP_hard_soft backward does
not skip c == f), (iii) returns two extra values.  The soft (marginal) branch
(`args.mpnet_enable_soft`) is not implemented and raises.
"""
import torch
import torch.nn as nn

from .MP_module import TRWPFunction as _TRWPFunctionBase
from .label_context import create_label_context


class TRWPFunction(_TRWPFunctionBase):
    keep_diag = True


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
        if getattr(self.args, 'mpnet_enable_soft', False):
            raise NotImplementedError("the soft (marginal) TRWP branch is not part of this library")
        if msg_norm_index is not None:
            raise NotImplementedError("externally supplied msg_norm_index (a debugging hook of the "
                                      "reference) is not supported")
        assert self.args.mpnet_mrf_mode == 'TRWP'
        unary = unary.permute(0, 1, 3, 4, 2).contiguous()
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
        cost_final, cost_all = TRWPFunction.apply(unary, label_context, edge_weights, self.args)
        cost_final = cost_final.permute(0, 1, 4, 2, 3).contiguous()
        label_context = label_context.unsqueeze(0)
        empty = torch.empty(0, dtype=torch.float32, device=unary.device)
        return cost_final, label_context, cost_all, empty, empty
