"""Noisy top-k gate (fmoe/gates/noisy_gate.py:13-144): logits = x W_g + noise * softplus(x W_n),
top-k over the noisy logits, softmax over the selected ones, and a load-balancing loss made of the
squared coefficients of variation of the experts' importance and (smoothed) load."""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .base_gate import BaseGate
from ..functions import gate_topk


def _cv_squared(x):
    """var / mean^2 of a sample (0 for a single element)."""
    if x.shape[0] == 1:
        return x.new_zeros(())
    x = x.float()
    return x.var() / (x.mean() ** 2 + 1e-10)


class NoisyGate(BaseGate):
    def __init__(self, d_model, num_expert, world_size, top_k=2):
        super().__init__(num_expert, world_size)
        self.w_gate = nn.Parameter(torch.zeros(d_model, self.tot_expert))
        self.w_noise = nn.Parameter(torch.zeros(d_model, self.tot_expert))
        self.top_k = top_k
        self.noise_epsilon = 1e-2
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.w_gate, a=math.sqrt(5))
        nn.init.kaiming_uniform_(self.w_noise, a=math.sqrt(5))

    def _prob_in_top_k(self, clean, noisy, stddev, top_values):
        """P(expert stays / gets into the top k under fresh noise), per token and expert: the threshold
        is the (k+1)-th noisy logit for experts that are in, the k-th for those that are out."""
        thr_in = top_values[:, self.top_k].unsqueeze(1)
        thr_out = top_values[:, self.top_k - 1].unsqueeze(1)
        is_in = noisy > thr_in
        normal = torch.distributions.normal.Normal(clean.new_zeros(1), clean.new_ones(1))
        return torch.where(is_in, normal.cdf((clean - thr_in) / stddev), normal.cdf((clean - thr_out) / stddev))

    def forward(self, inp, noise=None):
        """``noise``: the standard-normal sample to use (default: drawn here), for reproducible tests."""
        clean = inp @ self.w_gate
        stddev = (F.softplus(inp @ self.w_noise) + self.noise_epsilon) * float(self.training)
        if noise is None:
            noise = torch.randn_like(clean)
        noisy = clean + noise * stddev
        m = min(self.top_k + 1, self.tot_expert)
        top_values, top_idx = gate_topk(noisy, m)
        top_k_idx = top_idx[:, : self.top_k]
        top_k_gates = F.softmax(top_values[:, : self.top_k], dim=1)
        gates = torch.zeros_like(noisy).scatter(1, top_k_idx, top_k_gates)
        # Without noise (eval mode) the smoothed load is undefined: the reference divides by a zero
        # standard deviation there and fails; the load is then the count of tokens per expert.
        if self.top_k < self.tot_expert and self.training:
            load = self._prob_in_top_k(clean, noisy, stddev, top_values).sum(0)
        else:
            load = (gates > 0).sum(0)
        self.set_loss(_cv_squared(gates.sum(0)) + _cv_squared(load))
        return top_k_idx.contiguous().view(-1), top_k_gates.contiguous().unsqueeze(1)
