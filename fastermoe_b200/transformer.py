r"""MoE MLP block of a Transformer (mirrors fmoe/transformer.py)."""
import os

import torch
import torch.nn as nn

from .gates import NaiveGate
from .layers import FMoE, FMoELinear
from .functions import FusedExpertMLP, ExpertCounts, activation_code

# Hardware constants of the shadowing cost model.  "reference" are the values
# hard-coded in fmoe/transformer.py:35-38 (V100-era cluster); "b200" are this
# machine's measured figures (bf16 tensor throughput, NVLink per direction).
POLICY_CONSTANTS = {
    "reference": dict(bw_net=50 * 1e9 / 8, bw_mm=11.5e12, data_size=4),
    "b200": dict(bw_net=770e9, bw_mm=1.36e15, data_size=2),
}


class _Expert(nn.Module):
    r"""All experts of one worker as two grouped linear layers with an activation
    in between (fmoe/transformer.py:10-30).  When the activation is ReLU or
    exact GELU it is applied inside the GEMM epilogues."""

    def __init__(self, num_expert, d_model, d_hidden, activation, rank=0, bias=True):
        super().__init__()
        self.htoh4 = FMoELinear(num_expert, d_model, d_hidden, bias=bias, rank=rank)
        self.h4toh = FMoELinear(num_expert, d_hidden, d_model, bias=bias, rank=rank)
        self.activation = activation

    def consumes_arrival(self, inp):
        """True when forward() reads its input with the fused kernels, which can start on rows of an
        exchange that are still arriving (and later on the arriving output gradient)."""
        return inp.is_cuda and activation_code(self.activation) is not None

    def forward(self, inp, fwd_expert_count):
        code = activation_code(self.activation)
        exch = getattr(fwd_expert_count, "exchange", None)
        if code is None or not inp.is_cuda:
            if exch is not None:
                exch.flush()
            x = self.htoh4(inp, fwd_expert_count)
            x = self.activation(x)
            return self.h4toh(x, fwd_expert_count)
        counts = ExpertCounts.wrap(fwd_expert_count, inp.device)
        return FusedExpertMLP.apply(inp, counts.offsets, self.htoh4.weight, self.htoh4.bias,
                                    self.h4toh.weight, self.h4toh.bias, code, exch)


def _gen_policy(alpha, constants=None):
    r"""Returns the shadowing policy selected by FMOE_ENABLE_DYNREP (fmoe/transformer.py:33-86).

    The policy maps the all-gathered count tables to a bool [W, E] of expert
    sets to replicate on every worker.  ``constants`` is a key of
    POLICY_CONSTANTS or a dict; default: env FMOE_POLICY_CONSTANTS or "reference".
    """
    if constants is None:
        constants = os.environ.get("FMOE_POLICY_CONSTANTS", "reference")
    c = POLICY_CONSTANTS[constants] if isinstance(constants, str) else constants
    bw_net, bw_mm, data_size = c["bw_net"], c["bw_mm"], c["data_size"]

    def _global_policy(all_experts_count, all_global_expert_count, num_expert, world_size, d_model, fused):
        # The reference evaluates this with a few dozen torch operators on tiny CPU tensors per call
        # (several hundred microseconds at 8 workers, twice per layer call when the gate consults it
        # too).  Same arithmetic here on numpy scalars, in float32 where torch computes in float32
        # (int64 tensor x Python float); torch.sort gives the order so that ties break as there.
        import numpy as np
        f32 = np.float32
        agec = all_global_expert_count.detach().cpu().numpy().astype(np.int64)
        if fused:
            agec = agec.sum(-1).reshape(world_size, world_size, 1)
        if agec.shape[2] != 1:
            raise RuntimeError("the shadowing policy works at whole-worker granularity (fused experts) only")
        recv = agec[:, :, 0]                                   # [worker, source]: rows worker's experts get from source
        load = recv.sum(1)                                     # rows each worker's experts process
        order = torch.from_numpy(load.reshape(world_size, 1).copy()).sort(0, descending=True)[1][:, 0].numpy()

        unit = alpha * d_model ** 2 * data_size
        busiest = int(load.max())
        lat_plain = f32(f32(f32(12 * busiest) * f32(unit)) / f32(bw_mm)) + f32(f32(4 * busiest * d_model * data_size) / f32(bw_net))
        model_cost = 2 * unit * num_expert / bw_net * 2
        comp_time = 12 * unit / bw_mm

        best = f32(np.inf)
        load = load.copy()
        i = 0
        for i, index in enumerate(order):
            # Shadowing worker `index`: its rows are computed where they originate.
            load[index] = 0
            load += recv[index]
            lat = f32(f32(f32(int(load.max())) * f32(comp_time)) + f32((i + 1) * model_cost))
            if lat < best:
                best = lat
            elif lat > best:
                break
        res = torch.zeros(world_size, num_expert, dtype=torch.bool)
        if lat_plain > best:
            res[torch.from_numpy(order[:i].astype(np.int64))] = True
        return res

    def _no_policy(all_experts_count, all_global_expert_count, num_expert, world_size, d_model, fused):
        return all_experts_count.new_zeros(world_size, num_expert, dtype=torch.bool)

    if os.environ.get("FMOE_ENABLE_DYNREP", "0") == "1":
        return _global_policy
    _no_policy.never_shadows = True      # lets the layer skip the shadowing plan altogether
    return _no_policy


class FMoETransformerMLP(FMoE):
    r"""Drop-in MoE replacement of a Transformer MLP (fmoe/transformer.py:89-139).
    ``activation`` is applied between the two expert linears; ``d_hidden`` is
    their inner width."""

    def __init__(self, num_expert=32, d_model=1024, d_hidden=4096, world_size=1, mp_group=None,
                 moe_group=None, activation=torch.nn.GELU(), gate=NaiveGate, top_k=2,
                 expert_dp_comm="none", gate_hook=None, bias=True, mask=None, mask_dict=None):
        super().__init__(num_expert=num_expert, d_model=d_model, gate=gate, top_k=top_k,
                         world_size=world_size, mp_group=mp_group, moe_group=moe_group,
                         gate_hook=gate_hook, mask=mask, policy_fn=_gen_policy(d_hidden / d_model),
                         mask_dict=mask_dict)
        self.experts = _Expert(num_expert, d_model, d_hidden, activation, rank=self.mp_rank, bias=bias)
        self.mark_parallel_comm(expert_dp_comm)

    def forward(self, inp):
        original_shape = inp.shape
        out = super().forward(inp.reshape(-1, self.d_model))
        return out.reshape(original_shape)
