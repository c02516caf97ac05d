"""Gate contract (fmoe/gates/base_gate.py:7-25)."""
import torch.nn as nn


class BaseGate(nn.Module):
    """forward(x) -> (idx [T,k] int64, score [T,k]); an auxiliary loss may be left in ``loss``."""

    def __init__(self, num_expert, world_size):
        super().__init__()
        self.world_size = world_size
        self.num_expert = num_expert
        self.tot_expert = world_size * num_expert
        self.loss = None

    def forward(self, x):
        raise NotImplementedError("BaseGate is abstract")

    def set_loss(self, loss):
        self.loss = loss

    def get_loss(self, clear=True):
        loss = self.loss
        if clear:
            self.loss = None
        return loss
