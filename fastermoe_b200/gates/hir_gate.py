"""Topology-aware top-2 gate (fmoe/gates/hir_gate.py:18-123).

Workers are grouped into nodes of ``nw_per_node``.  A token's first choice may
leave its node only for a limited share of the tokens (``ogn_ratio``); experts
whose parameters are shadowed on every worker count as local.
"""
import torch
import torch.nn.functional as F

from .naive_gate import NaiveGate
from .gshard_gate import balance_loss_top1
from ..functions import count_by_gate, gate_topk

nw_per_node = 4


class HirGate(NaiveGate):
    def __init__(self, d_model, n_expert, world_size, node_rank, workers_per_node=None):
        super().__init__(d_model, n_expert, world_size, top_k=2)
        wpn = nw_per_node if workers_per_node is None else workers_per_node
        self.ne_per_node = wpn * n_expert
        self.ogn_ratio = 0.14
        self.node_rank = node_rank
        on_node = torch.arange(n_expert * world_size) // self.ne_per_node == node_rank
        self.register_buffer("mask", on_node, persistent=False)
        self.stored_models = None
        self.policy_fn = None
        self.last_stored = None     # the policy's answer of the latest forward (bool [W, E], CPU)

    def forward(self, inp):
        gate_score = self.gate(inp)
        off_node = ~self.mask.to(inp.device)

        top2_val, top2_idx = gate_topk(gate_score, 2)
        n_tok = gate_score.shape[0]
        with torch.no_grad():
            top1_idx = top2_idx.view(-1, 2)[:, 0]
            top1_val = top2_val.view(-1, 2)[:, 0].clone()
        self.set_loss(balance_loss_top1(top1_idx, gate_score, self.tot_expert, self.num_expert))

        with torch.no_grad():
            _, _, aec, _, _ = count_by_gate(top2_idx, self.num_expert, self.world_size, require_pos=False)
            w, e = self.world_size, self.num_expert
            # one copy to the host: the table seen from the receivers is its transpose
            aec_host = aec.view(-1).cpu().view(w, w, e) if w > 1 else aec.cpu().view(1, 1, e)
            agec_host = aec_host.transpose(0, 1).contiguous()
            stored = self.policy_fn(aec_host, agec_host, e, w, inp.shape[-1], True)
            self.last_stored = stored.reshape(w, e).cpu()
            # Experts shadowed on every worker are as good as local ones.
            limited = off_node & ~stored.reshape(-1).to(off_node.device)
            leaving = limited[top1_idx]
            ogn_thres = int(n_tok * self.ogn_ratio)

        if int(leaving.sum().item()) < ogn_thres:
            return top2_idx, F.softmax(top2_val, dim=-1)

        with torch.no_grad():
            # The ogn_thres tokens with the strongest off-node first choice keep it
            # (in slot 1); everything else is chosen among the allowed experts.
            top1_val[~leaving] = float("-inf")
            _, keep = torch.topk(top1_val.view(-1), k=ogn_thres)
            cand = gate_score.detach().clone()
            cand[:, limited] = float("-inf")
            _, topk_idx = gate_topk(cand, self.top_k)
            topk_idx[keep, 1] = top1_idx.view(-1)[keep]

        rows = torch.arange(n_tok, device=inp.device).repeat_interleave(2)
        topk_val = gate_score[rows, topk_idx.view(-1)].view(-1, self.top_k)
        return topk_idx, F.softmax(topk_val, dim=-1)


class HirCapacityGate(HirGate):
    """HirGate followed by the capacity limit of the GShard-style gates (fmoe/gates/gshard_gate.py:36-39
    applied to fmoe/gates/hir_gate.py's selection): each expert accepts at most ceil(cap_rate * tokens)
    rows, entries beyond that become -1; scores are those of the selection before pruning.

    ``spare_shadowed``: experts that the shadowing policy (consulted by HirGate on the unpruned counts)
    replicates on every worker are exempt from the limit -- their rows are computed where they
    originate, so no single GPU is overloaded by them.  ``last_selection`` keeps the unpruned indices."""

    def __init__(self, d_model, n_expert, world_size, node_rank, workers_per_node=None, cap_rate=1.2,
                 spare_shadowed=False, rank=0):
        super().__init__(d_model, n_expert, world_size, node_rank, workers_per_node)
        self.cap_rate, self.spare_shadowed, self.rank = cap_rate, spare_shadowed, rank
        self.last_selection = None

    def forward(self, inp):
        import math
        from .utils import limit_by_capacity
        idx, score = super().forward(inp)
        self.last_selection = idx
        cap = math.ceil(self.cap_rate * inp.shape[0])
        if self.spare_shadowed and self.last_stored is not None:
            per_expert = torch.full((self.num_expert,), cap, dtype=torch.int32)
            per_expert[self.last_stored[self.rank]] = torch.iinfo(torch.int32).max
            cap = per_expert
        _, _, idx = limit_by_capacity(idx.contiguous(), self.num_expert, self.world_size, cap)
        return idx, score


def gen_hir_capacity_gate(rank, workers_per_node=None, cap_rate=1.2, spare_shadowed=False):
    """Gate factory like gen_hir_gate for HirCapacityGate."""
    wpn = nw_per_node if workers_per_node is None else workers_per_node

    def _gen(d_model, n_expert, world_size, top_k=2):
        assert top_k == 2
        return HirCapacityGate(d_model, n_expert, world_size, rank // wpn, workers_per_node=wpn, cap_rate=cap_rate,
                               spare_shadowed=spare_shadowed, rank=rank)
    return _gen


def gen_hir_gate(rank, workers_per_node=None):
    """Gate factory for the worker with global rank ``rank`` (fmoe/gates/hir_gate.py:119-123)."""
    wpn = nw_per_node if workers_per_node is None else workers_per_node

    def _gen(d_model, n_expert, world_size, top_k=2):
        assert top_k == 2
        return HirGate(d_model, n_expert, world_size, rank // wpn, workers_per_node=wpn)
    return _gen
