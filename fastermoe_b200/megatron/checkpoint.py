r"""Expert-sharded checkpoints in the reference's on-disk layout (fmoe/megatron/checkpoint.py:12-386).

What the format is.  Data-parallel rank 0 of every model-parallel position writes a complete Megatron
checkpoint.  Every other data-parallel rank holds different experts but the same everything else, so it
writes only what is its own: the model tensors tagged ``dp_comm == "none"`` and the optimizer state of
those parameters, into a sibling directory whose name carries the data-parallel rank::

    <root>/iter_0000100/mp_rank_00/model_optim_rng.pt                 dp rank 0 (Megatron's own name)
    <root>/iter_0000100/mp_rank_00_dp_rank_0003/model_optim_rng.pt    dp rank 3, experts only
    <root>/iter_0000100/mp_rank_00_001_dp_rank_0003/...               the same with pipeline stages
    <root>/latest_checkpointed_iteration.txt                          "100" or "release"

A rank other than 0 loads rank 0's file and its own and overlays the second on the first.

The core below needs nothing from Megatron-LM: positions in the parallel grid are passed in as
``GridPosition``, optimizers are plain ``torch.optim`` objects (or Megatron's fp16 wrapper, recognised by its
``optimizer`` / ``fp32_from_fp16_params`` entries).  ``save_checkpoint`` / ``load_checkpoint`` at the end keep
the reference's signatures and fetch the grid position and the arguments from an installed Megatron-LM.
"""
import os
from collections import OrderedDict, namedtuple

import torch

TRACKER = "latest_checkpointed_iteration.txt"
FILE = "model_optim_rng.pt"
EXPERT_TAG = "none"

GridPosition = namedtuple("GridPosition", "dp_rank tp_rank pp_rank pp_world", defaults=(0, 0, 0, 1))


def checkpoint_dir(root, iteration, release=False):
    return os.path.join(root, "release" if release else "iter_{:07d}".format(iteration))


def checkpoint_name(root, iteration, pos, release=False):
    """Path of the file that the rank at ``pos`` writes (fmoe/megatron/checkpoint.py:12-48)."""
    stem = "mp_rank_{:02d}".format(pos.tp_rank)
    if pos.pp_world > 1:
        stem += "_{:03d}".format(pos.pp_rank)
    if pos.dp_rank > 0:
        stem += "_dp_rank_{:04d}".format(pos.dp_rank)
    return os.path.join(checkpoint_dir(root, iteration, release), stem, FILE)


def _is_expert(t, tag):
    return getattr(t, "dp_comm", None) == tag


def expert_entries(state, tag=EXPERT_TAG):
    """The sub-tree of a (nested) state dict whose leaves are tagged ``dp_comm == tag``; the state dict must
    have been taken with ``keep_vars=True`` so that the leaves still are the parameters.  Empty branches
    are dropped; the kept tensors are detached (fmoe/megatron/checkpoint.py:83-95)."""
    out = state.__class__()
    for key, value in state.items():
        if isinstance(value, (dict, OrderedDict)):
            sub = expert_entries(value, tag)
            if len(sub):
                out[key] = sub
        elif _is_expert(value, tag):
            out[key] = value.detach()
    return out


def _is_fp16_wrapper(optim_state):
    return "optimizer" in optim_state and "fp32_from_fp16_params" in optim_state


def expert_optimizer_state(optim_state, params_in_order, tag=EXPERT_TAG, master_params=None):
    """Reduces an optimizer state dict to the entries of expert parameters.

    ``params_in_order``: the optimizer's parameters in ``param_groups`` order (state keys are their indices).
    ``master_params`` (Megatron's fp16 wrapper only): its ``fp32_from_fp16_params`` groups; the copy keeps the
    expert entries and ``None`` elsewhere.  ``param_groups`` is dropped: rank 0 saves it
    (fmoe/megatron/checkpoint.py:98-142)."""
    state = dict(optim_state)
    inner = dict(state["optimizer"]) if _is_fp16_wrapper(state) else state
    kept = {}
    for index, p in enumerate(params_in_order):
        if _is_expert(p, tag) and index in inner["state"]:
            kept[index] = inner["state"][index]
    inner["state"] = kept
    inner.pop("param_groups", None)
    if _is_fp16_wrapper(state):
        state["optimizer"] = inner
        groups = master_params if master_params is not None else state["fp32_from_fp16_params"]
        state["fp32_from_fp16_params"] = [[p if _is_expert(p, tag) else None for p in g] for g in groups]
    return state


def overlay(full, local):
    """Writes the expert-only checkpoint ``local`` over the complete one ``full`` in place and returns it
    (fmoe/megatron/checkpoint.py:169-211): model leaves, optimizer state entries, fp32 master copies."""
    def over(dst, src):
        for key, value in src.items():
            if isinstance(value, (dict, OrderedDict)):
                over(dst[key], value)
            else:
                dst[key] = value
    over(full["model"], local.get("model", {}))
    if "optimizer" in local and "optimizer" in full:
        wrapped = _is_fp16_wrapper(local["optimizer"])
        dst = full["optimizer"]["optimizer"] if wrapped else full["optimizer"]
        src = local["optimizer"]["optimizer"] if wrapped else local["optimizer"]
        for index, entry in src["state"].items():
            dst["state"][index] = entry
        if wrapped:
            for g, group in enumerate(local["optimizer"]["fp32_from_fp16_params"]):
                for i, p in enumerate(group):
                    if p is not None:
                        full["optimizer"]["fp32_from_fp16_params"][g][i] = p
    return full


def _optimizer_params(optimizer):
    inner = getattr(optimizer, "optimizer", optimizer)        # Megatron's wrappers hold the torch optimizer
    return [p for group in inner.param_groups for p in group["params"]]


def save_shard(root, iteration, model, optimizer, pos, extra=None, save_optim=True, tag=EXPERT_TAG):
    """Writes this rank's file.  ``model`` needs ``state_dict(keep_vars=...)`` (or Megatron's
    ``state_dict_for_save_checkpoint``).  Rank 0 writes everything plus ``extra`` (iteration, args, rng states,
    scheduler ...); the others their experts.  Returns the path.  The caller synchronises the ranks and then
    calls ``write_tracker`` on one of them."""
    getter = getattr(model, "state_dict_for_save_checkpoint", model.state_dict)
    blob = {}
    if pos.dp_rank == 0:
        blob.update(extra or {})
        blob["iteration"] = iteration
        blob["model"] = getter()
        if save_optim and optimizer is not None:
            blob["optimizer"] = optimizer.state_dict()
    else:
        blob["model"] = expert_entries(getter(keep_vars=True), tag)
        if save_optim and optimizer is not None:
            blob["optimizer"] = expert_optimizer_state(optimizer.state_dict(), _optimizer_params(optimizer), tag,
                                                       getattr(optimizer, "fp32_from_fp16_params", None))
    path = checkpoint_name(root, iteration, pos)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    torch.save(blob, path)
    return path


def write_tracker(root, iteration):
    with open(os.path.join(root, TRACKER), "w") as f:
        f.write(str(iteration))


def read_tracker(root):
    """(iteration, release) of the newest checkpoint under ``root``; (0, False) when there is none."""
    path = os.path.join(root, TRACKER)
    if not os.path.isfile(path):
        return 0, False
    text = open(path).read().strip()
    if text == "release":
        return 0, True
    try:
        return int(text), False
    except ValueError:
        raise RuntimeError(f"{path}: expected an iteration number or 'release', found {text!r}") from None


def load_shard(root, model, optimizer, pos, load_optim=True, strict=True):
    """Loads the newest checkpoint for the rank at ``pos``: rank 0's file, overlaid with this rank's own
    expert file when ``pos.dp_rank > 0``.  Returns the merged dict (``["iteration"]`` etc. for the caller),
    or None when ``root`` holds no checkpoint."""
    iteration, release = read_tracker(root)
    if iteration == 0 and not release:
        return None
    first = checkpoint_name(root, iteration, pos._replace(dp_rank=0), release)
    blob = torch.load(first, map_location="cpu", weights_only=False)
    if pos.dp_rank > 0:
        own = torch.load(checkpoint_name(root, iteration, pos, release), map_location="cpu", weights_only=False)
        blob = overlay(blob, own)
    model.load_state_dict(blob["model"], strict=strict)
    if load_optim and optimizer is not None and "optimizer" in blob:
        optimizer.load_state_dict(blob["optimizer"])
    return blob


# ---- the reference's entry points, for a process in which Megatron-LM is importable ----------------------

def _megatron():
    try:
        import megatron
        from megatron import mpu
    except ImportError as e:
        raise ImportError("fastermoe_b200.megatron.save_checkpoint / load_checkpoint read the parallel grid and the "
                          "arguments from Megatron-LM, which is not importable here; use save_shard / load_shard "
                          "with an explicit GridPosition instead") from e
    return megatron, mpu


def _position(mpu):
    return GridPosition(mpu.get_data_parallel_rank(), mpu.get_tensor_model_parallel_rank(),
                        mpu.get_pipeline_model_parallel_rank(), mpu.get_pipeline_model_parallel_world_size())


def save_checkpoint(iteration, model, optimizer, lr_scheduler):
    """fmoe/megatron/checkpoint.py:51-166: data-parallel rank 0 saves through Megatron, the others save their
    experts beside it."""
    megatron, mpu = _megatron()
    if mpu.get_data_parallel_rank() == 0:
        from megatron.checkpointing import save_checkpoint as native
        return native(iteration, model, optimizer, lr_scheduler)
    args = megatron.get_args()
    while hasattr(model, "module"):
        model = model.module
    save_shard(args.save, iteration, model, optimizer, _position(mpu), save_optim=not args.no_save_optim)
    torch.distributed.barrier()
    if torch.distributed.get_rank() == 0:
        write_tracker(args.save, iteration)
    torch.distributed.barrier()


def load_checkpoint(model, optimizer, lr_scheduler, load_arg="load"):
    """fmoe/megatron/checkpoint.py:214-386: returns the iteration to resume from."""
    megatron, mpu = _megatron()
    if mpu.get_data_parallel_rank() == 0:
        from megatron.checkpointing import load_checkpoint as native
        return native(model, optimizer, lr_scheduler, load_arg)
    args = megatron.get_args()
    while hasattr(model, "module"):
        model = model.module
    release = read_tracker(getattr(args, load_arg))[1]
    fresh = release or args.finetune
    blob = load_shard(getattr(args, load_arg), model, optimizer, _position(mpu),
                      load_optim=not (fresh or args.no_load_optim))
    if blob is None:
        return 0
    if lr_scheduler is not None and not fresh and not args.no_load_optim and "lr_scheduler" in blob:
        lr_scheduler.load_state_dict(blob["lr_scheduler"])
    torch.distributed.barrier()
    return 0 if fresh else blob.get("iteration", blob.get("total_iters", 0))
