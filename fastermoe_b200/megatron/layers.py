r"""Modules that take the place of Megatron-LM's MLP blocks (fmoe/megatron/layers.py:106-258)."""
import math

import numpy as np
import torch

from ..transformer import FMoETransformerMLP
from ..utils import get_torch_default_comm
from . import host
from .balance import generate_megatron_gate_hook, reset_gate_hook
from .distributed import set_moe_group


def _gate_class(strategy, moe_group):
    """The gate a ``--balance-strategy`` names (fmoe/megatron/layers.py:121-145)."""
    from .. import gates
    if not strategy or strategy == "naive":
        return gates.NaiveGate
    if strategy == "noisy":
        return gates.NoisyGate
    if strategy == "gshard":
        return gates.GShardGate
    if strategy == "switch":
        return gates.SwitchGate
    if strategy == "hir":
        return gates.gen_hir_gate(moe_group.rank() if moe_group is not None else 0)
    raise ValueError(f"balance strategy {strategy!r} is not available in this package "
                     "(naive, noisy, gshard, switch, hir)")


def _normal_init(linear, rng, sigma):
    """weight ~ N(0, sigma) drawn from a numpy generator (the host framework pins torch's seeds for its own
    purposes), bias zero."""
    w = rng.normal(loc=0.0, scale=sigma, size=tuple(linear.weight.shape))
    with torch.no_grad():
        linear.weight.copy_(torch.from_numpy(w).to(linear.weight.dtype))
        if linear.bias is not None:
            linear.bias.zero_()


class MegatronMLP(FMoETransformerMLP):
    """The MoE block with the call convention of Megatron's ParallelMLP: ``forward`` returns
    ``(output, bias)`` with a zero bias, experts are spread over ``tensor x data`` parallel ranks when
    ``args.distributed_experts`` is set, and the weights are initialised the way Megatron initialises an MLP
    (N(0, sigma) going in, N(0, sigma / sqrt(2 * num_layers)) going out)."""

    def __init__(self, args, mp_group, moe_group, layer_idx):
        if (args.seq_length * args.micro_batch_size) % args.tensor_model_parallel_size:
            raise ValueError("batch size x sequence length must be a multiple of the tensor-parallel size")
        distributed = bool(getattr(args, "distributed_experts", True))
        world_size = args.tensor_model_parallel_size * args.data_parallel_size if distributed else 1
        super().__init__(args.num_experts, top_k=args.top_k, d_model=args.hidden_size,
                         d_hidden=args.hidden_hidden_size, world_size=world_size, mp_group=mp_group,
                         moe_group=moe_group, expert_dp_comm="none" if distributed else "dp",
                         gate_hook=generate_megatron_gate_hook(layer_idx, args.num_experts * world_size),
                         gate=_gate_class(getattr(args, "balance_strategy", None), moe_group))
        self.hidden_size = args.hidden_size
        self.rank = args.rank if distributed else 0
        self.sigma, self.num_layers = args.init_method_std, args.num_layers
        self.reset_parameters()

    def reset_parameters(self):
        rng = np.random.default_rng(np.random.randint(2048) + self.rank)
        _normal_init(self.experts.htoh4, rng, self.sigma)
        _normal_init(self.experts.h4toh, rng, self.sigma / math.sqrt(2.0 * self.num_layers))

    def forward(self, inp):
        return super().forward(inp), torch.zeros(self.hidden_size, dtype=inp.dtype, device=inp.device)


def _layers_of(model):
    lm = model.language_model
    stack = getattr(lm, "transformer", None) or lm.encoder
    return stack.layers


def fmoefy(model, num_experts=None, distributed_experts=True, hidden_hidden_size=None, top_k=None):
    """Replaces the ``mlp`` of every transformer layer of a Megatron-style model
    (``model.language_model.transformer.layers[i].mlp``) by a MegatronMLP and returns the model.

    ``distributed_experts``: experts differ from rank to rank (expert parallelism over the tensor x data
    ranks of a pipeline stage); False: every rank holds the same experts and trains them data-parallel.
    With pipeline parallelism the MoE group is the set of ranks of this rank's stage."""
    args, mpu = host.get_args(), host.get_mpu()
    if num_experts is not None:
        args.num_experts = num_experts
    if getattr(args, "num_experts", None) is None:
        raise ValueError("num_experts must be given, in the arguments or to fmoefy")
    if hidden_hidden_size is not None:
        args.hidden_hidden_size = hidden_hidden_size
    elif getattr(args, "hidden_hidden_size", None) is None:
        args.hidden_hidden_size = args.hidden_size * 4
    if top_k is not None:
        args.top_k = top_k
    elif getattr(args, "top_k", None) is None:
        args.top_k = 2
    if distributed_experts is not None:
        args.distributed_experts = distributed_experts

    mp = getattr(mpu, "get_tensor_model_parallel_group", None) or mpu.get_model_parallel_group
    mp_group = mp()
    if args.pipeline_model_parallel_size == 1:
        # (a single process without a process group: one worker, no group needed)
        moe_group = get_torch_default_comm() if torch.distributed.is_initialized() else None
    else:
        stage = args.world_size // args.pipeline_model_parallel_size
        moe_group = None
        for first in range(0, args.world_size, stage):           # every rank creates every group
            ranks = list(range(first, first + stage))
            group = torch.distributed.new_group(ranks)
            if args.rank in ranks:
                moe_group = group
        set_moe_group(moe_group)
    layers = _layers_of(model)
    for idx, layer in enumerate(layers):
        layer.mlp = MegatronMLP(args, mp_group, moe_group, idx)
    reset_gate_hook(len(layers))
    return model
