r"""Gradient synchronisation by parameter tag (mirrors fmoe/distributed.py)."""
import torch
import torch.nn as nn
from torch._utils import _flatten_dense_tensors, _unflatten_dense_tensors

from .utils import get_torch_default_comm


class DistributedGroupedDataParallel(nn.Module):
    r"""Wraps a module whose parameters carry a ``dp_comm`` tag ('dp', 'moe', 'world',
    'mp' or 'none') and all-reduces each tag's gradients over the matching process
    group when ``allreduce_params`` is called (fmoe/distributed.py:10-121).
    Parameters tagged 'none' (experts) are left alone."""

    def __init__(self, module, mp_group=None, dp_group=None, moe_group=None, world_group=None,
                 auto_allreduce=False):
        assert not auto_allreduce, "Automatic all-reduce is not implemented yet"
        super().__init__()
        self.module = module
        self.comms = {}
        if mp_group is not None:
            self.comms["mp"] = mp_group
        self.comms["dp"] = dp_group if dp_group is not None else get_torch_default_comm()
        self.comms["moe"] = moe_group if moe_group is not None else get_torch_default_comm()
        self.comms["world"] = world_group if world_group is not None else get_torch_default_comm()
        self._sync_params()

    def _buckets(self, with_grad):
        groups = {}
        for p in self.module.parameters():
            if with_grad and (not p.requires_grad or p.grad is None):
                continue
            tag = getattr(p, "dp_comm", "dp")
            groups.setdefault((tag, p.dtype), []).append(p)
        return groups

    def allreduce_params(self, no_scale=False, reduce_after=False, fp32_allreduce=False):
        """All-reduces gradients per (tag, dtype) bucket; averages unless ``no_scale``."""
        for (tag, _), params in self._buckets(True).items():
            if tag not in self.comms:
                continue
            comm = self.comms[tag]
            grads = [p.grad.data for p in params]
            flat = _flatten_dense_tensors(grads)
            if fp32_allreduce:
                flat = flat.float()
            if not no_scale and not reduce_after:
                flat /= comm.size()
            torch.distributed.all_reduce(flat, group=comm)
            if not no_scale and reduce_after:
                flat /= comm.size()
            for g, s in zip(grads, _unflatten_dense_tensors(flat, grads)):
                g.copy_(s)

    def _sync_params(self):
        """Broadcasts every tagged parameter from the first rank of its group."""
        for (tag, _), params in self._buckets(False).items():
            if tag not in self.comms:
                continue
            comm = self.comms[tag]
            datas = [p.data for p in params]
            flat = _flatten_dense_tensors(datas)
            torch.distributed.broadcast(flat, torch.distributed.get_global_rank(comm, 0), group=comm)
            for d, s in zip(datas, _unflatten_dense_tensors(flat, datas)):
                d.copy_(s)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)
