r"""Plug-in for Megatron-style trainers (fmoe/megatron/__init__.py:4-19): ``fmoefy`` swaps a model's MLP
blocks for MoE blocks, ``DistributedDataParallel`` reduces gradients per parameter tag,
``save_checkpoint`` / ``load_checkpoint`` write and read expert-sharded checkpoints, and the balance helpers
monitor the routing.  Megatron-LM itself is optional: ``bind(args=..., mpu=...)`` supplies what the adapter
would otherwise import from it."""
from .host import bind, unbind, add_fmoe_args
from .layers import MegatronMLP, fmoefy
from .checkpoint import (GridPosition, checkpoint_name, expert_entries, expert_optimizer_state, overlay, save_shard,
                         load_shard, write_tracker, read_tracker, save_checkpoint, load_checkpoint)
from .distributed import DistributedDataParallel, set_moe_group, get_moe_group
from .balance import (reset_gate_hook, get_balance_profile, generate_megatron_gate_hook, add_balance_log,
                      patch_forward_step, patch_model_provider)
