r"""Load-balance monitoring and the balance loss for a Megatron-style training loop
(fmoe/megatron/balance.py:11-144, fmoe/balance.py:4-28).

Per layer the gate hook records three imbalance figures of the step's routing (from the histogram of the
chosen experts) and, for gates that define one, the balance loss; ``add_balance_log`` averages them over the
ranks and writes them to a summary writer; ``patch_forward_step`` adds the weighted mean of the layers'
balance losses to the training loss.
"""
import torch

from ..utils import get_torch_default_comm
from . import host
from .distributed import get_moe_group

METRICS = {
    "coefficient-variation": lambda c: torch.std(c) / torch.mean(c),
    "Lmax-over-Lmin": lambda c: (torch.max(c) + 1) / (torch.min(c) + 1),
    "Lmax-over-Lmean": lambda c: torch.max(c) / torch.mean(c),
}
NO_LOSS = {"naive", "neighbor", "baselayer", "baseorig"}

balance_dict = {}
_num_layers = 0


def reset_gate_hook(num_layers=None):
    """Empties the per-layer records (one slot per layer and figure)."""
    global _num_layers
    if num_layers is not None:
        _num_layers = num_layers
    strategy = getattr(host.get_args(), "balance_strategy", None)
    balance_dict.clear()
    for key in METRICS:
        balance_dict[key] = [None] * _num_layers
    if strategy:
        balance_dict[f"{strategy}_loss"] = [None] * _num_layers


def get_balance_profile():
    return balance_dict


def generate_megatron_gate_hook(layer_idx, num_expert_global):
    """The ``gate_hook`` of layer ``layer_idx``: called by the layer with (top-k indices, top-k scores, context).
    The reference leaves the body of its update function empty (fmoe/balance.py:20-28); here the hook fills
    the three figures from the indices it is given, on the device, without a host read."""
    def hook(gate_top_k_idx, _gate_score_top_k, _gate_context):
        if layer_idx >= _num_layers:
            return
        with torch.no_grad():
            flat = gate_top_k_idx.reshape(-1)
            counts = torch.bincount(flat[flat >= 0], minlength=num_expert_global).float()
            for key, fn in METRICS.items():
                balance_dict[key][layer_idx] = fn(counts)
    return hook


def _layers_of(model):
    while hasattr(model, "module"):
        model = model.module
    lm = model.language_model
    stack = getattr(lm, "transformer", None) or lm.encoder          # newer Megatron-LM names it encoder
    return stack.layers


def add_balance_log(model, writer, iteration, is_last_rank=None):
    """Writes the balance figures of the step to a summary writer as ``balance-<name>/layer-<i>`` and
    ``balance-<name>/all`` (the mean over the layers), averaged over the ranks
    (fmoe/megatron/balance.py:48-72).  Names: the three imbalance figures the gate hooks recorded, and
    ``<strategy>_loss`` with the balance loss each layer's gate stored (the gates' losses are cleared)."""
    layers = _layers_of(model)
    strategy = getattr(host.get_args(), "balance_strategy", None)
    if strategy:
        key = f"{strategy}_loss"
        balance_dict.setdefault(key, [None] * len(layers))
        for i, layer in enumerate(layers):
            loss = layer.mlp.gate.get_loss(clear=True)
            if loss is not None and i < len(balance_dict[key]):
                balance_dict[key][i] = loss.detach().reshape(())
    names = list(balance_dict)
    device = next((v.device for vals in balance_dict.values() for v in vals if v is not None), torch.device("cpu"))
    table = torch.full((len(names), max(_num_layers, len(layers))), float("nan"), device=device)
    for r, name in enumerate(names):
        for i, v in enumerate(balance_dict[name]):
            if v is not None:
                table[r, i] = v.float()
    if torch.distributed.is_initialized():
        group = get_torch_default_comm()
        torch.distributed.all_reduce(table, group=group)
        table /= torch.distributed.get_world_size(group=group)
    if is_last_rank is None:
        try:
            from megatron import is_last_rank as native
            is_last_rank = native()
        except ImportError:
            is_last_rank = not torch.distributed.is_initialized() or \
                torch.distributed.get_rank() == torch.distributed.get_world_size() - 1
    if writer and is_last_rank:
        for r, name in enumerate(names):
            row = table[r]
            seen = ~torch.isnan(row)
            for i in torch.nonzero(seen).reshape(-1).tolist():
                writer.add_scalar(f"balance-{name}/layer-{i}", row[i].item(), iteration)
            if bool(seen.any()):
                writer.add_scalar(f"balance-{name}/all", row[seen].mean().item(), iteration)


def patch_forward_step(forward_step_func, is_pipeline_last_stage=None):
    """Wraps Megatron's ``forward_step`` so that the loss it returns includes
    ``balance_loss_weight x mean over layers of the gates' balance loss``, and the loss dictionary the
    MoE-group average of that term under ``<strategy>_loss`` (fmoe/megatron/balance.py:80-128)."""
    args = host.get_args()
    strategy = getattr(args, "balance_strategy", None)
    if not strategy:
        return forward_step_func
    if is_pipeline_last_stage is None:
        try:
            from megatron.mpu import is_pipeline_last_stage
        except ImportError:
            is_pipeline_last_stage = lambda: True       # noqa: E731  (no pipeline without Megatron)

    def forward_step_with_balance_loss(data_iterator, model, *rest):
        output = forward_step_func(data_iterator, model, *rest)
        if not is_pipeline_last_stage() or strategy in NO_LOSS:
            return output
        loss, stats = output
        terms = [l.mlp.gate.get_loss(clear=False).view(1) for l in _layers_of(model)]
        balance = torch.cat(terms).mean() * args.balance_loss_weight
        averaged = balance.clone().detach()
        group = get_moe_group()
        if torch.distributed.is_initialized():
            torch.distributed.all_reduce(averaged, group=group)
            averaged /= torch.distributed.get_world_size(group=group)
        stats[strategy + "_loss"] = averaged
        return loss + balance, stats

    return forward_step_with_balance_loss


def patch_model_provider(model_provider):
    """A model provider whose model has its MLPs replaced (fmoe/megatron/balance.py:131-144): the hidden
    width is divided by top_k so that a token costs what it cost in the dense model."""
    def fmoefied_model_provider(*a, **kw):
        from .layers import fmoefy
        args = host.get_args()
        return fmoefy(model_provider(*a, **kw), num_experts=args.num_experts,
                      hidden_hidden_size=4 * args.hidden_size // args.top_k, top_k=args.top_k)
    return fmoefied_model_provider
