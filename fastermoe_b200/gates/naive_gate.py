"""Linear gate with top-k selection (fmoe/gates/naive_gate.py:21-42)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .base_gate import BaseGate
from ..functions import gate_topk


class NaiveGate(BaseGate):
    r"""Scores tokens with one linear layer and keeps the k largest logits.

    The reference returns the *raw* top-k logits as scores: it computes their
    softmax and then discards it (fmoe/gates/naive_gate.py:38-42).  That is the
    default here too; ``softmax_scores=True`` (or the module attribute of the
    same name) returns the softmax over the k selected logits instead.
    """

    def __init__(self, d_model, num_expert, world_size, top_k=2, softmax_scores=False):
        super().__init__(num_expert, world_size)
        self.gate = nn.Linear(d_model, self.tot_expert)
        self.top_k = top_k
        self.softmax_scores = softmax_scores

    def forward(self, inp, return_all_scores=False):
        gate = self.gate(inp)
        top_val, top_idx = gate_topk(gate, self.top_k)
        top_val = top_val.view(-1, self.top_k)
        if self.softmax_scores:
            top_val = F.softmax(top_val, dim=-1)
        if return_all_scores:
            return top_idx, top_val, gate
        return top_idx, top_val
