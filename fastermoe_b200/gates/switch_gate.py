"""Switch-Transformer top-1 gate with capacity (fmoe/gates/switch_gate.py:24-59)."""
import math

import torch
import torch.nn.functional as F

from .naive_gate import NaiveGate
from ..functions import gate_topk
from .utils import limit_by_capacity


class SwitchGate(NaiveGate):
    def __init__(self, d_model, num_expert, world_size, topk=1, switch_eps=0.1, capacity=(1.2, 2.4)):
        assert topk == 1, "topk should be 1 in switch"
        super().__init__(d_model, num_expert, world_size, top_k=1)
        self.switch_eps = switch_eps
        self.capacity = capacity

    def forward(self, inp):
        score = self.gate(inp)
        if self.training:
            noise = torch.rand_like(score)
            score = score + (noise * 2 * self.switch_eps + 1.0 - self.switch_eps)
        score = F.softmax(score.float(), dim=-1)
        top1_score, top1_idx = gate_topk(score, 1)
        top1_score = top1_score.to(dtype=inp.dtype)

        cap_rate = self.capacity[0 if self.training else 1]
        capacity = math.ceil(cap_rate * inp.shape[0])
        _, _, top1_idx = limit_by_capacity(top1_idx, self.num_expert, self.world_size, capacity)

        valid_idx = top1_idx[top1_idx > -1]
        denom = max(valid_idx.numel(), 1)
        fraction_expert = torch.scatter_add(torch.zeros(self.tot_expert, device=valid_idx.device), 0,
                                            valid_idx, torch.ones_like(valid_idx, dtype=torch.float)) / denom
        prob_expert = score.sum(dim=0) / denom
        self.set_loss((fraction_expert * prob_expert).sum() * self.tot_expert)
        return top1_idx, top1_score
