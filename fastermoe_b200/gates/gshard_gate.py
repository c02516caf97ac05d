"""GShard-style top-2 gate with capacity (fmoe/gates/gshard_gate.py:19-46)."""
import math

import torch
import torch.nn.functional as F

from .naive_gate import NaiveGate
from .utils import limit_by_capacity


def balance_loss_top1(top1_idx, gate_score, tot_expert, num_expert):
    """mean(fraction routed * mean softmax prob) * num_expert^2 (gshard_gate.py:27-35)."""
    S = gate_score.shape[0]
    c_e = torch.scatter_add(torch.zeros(tot_expert, device=top1_idx.device), 0, top1_idx,
                            torch.ones_like(top1_idx, dtype=torch.float)) / S
    m_e = torch.mean(F.softmax(gate_score, dim=1), dim=0)
    return torch.mean(c_e * m_e) * (num_expert ** 2)


class GShardGate(NaiveGate):
    def __init__(self, d_model, num_expert, world_size, topk=2, capacity=(1.2, 2.4), random_routing=True):
        assert topk == 2, "topk should be 2 in gshard"
        super().__init__(d_model, num_expert, world_size, top_k=2)
        self.capacity = capacity
        self.random_routing = random_routing

    def forward(self, x):
        topk_idx, topk_val, gate_score = super().forward(x, return_all_scores=True)
        top1_idx = topk_idx.view(-1, self.top_k)[:, 0]
        self.set_loss(balance_loss_top1(top1_idx, gate_score, self.tot_expert, self.num_expert))

        cap_rate = self.capacity[0 if self.training else 1]
        capacity = math.ceil(cap_rate * x.shape[0])
        _, _, topk_idx = limit_by_capacity(topk_idx, self.num_expert, self.world_size, capacity)

        if self.random_routing:
            prob = torch.rand(gate_score.size(0), device=x.device)
            mask = 2 * topk_val[:, 1] < prob
            topk_idx[:, 1].masked_fill_(mask, -1)
        return topk_idx, topk_val
