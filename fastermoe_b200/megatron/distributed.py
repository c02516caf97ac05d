r"""Data-parallel wrapper with the interface Megatron-LM expects of its DDP module
(fmoe/megatron/distributed.py:10-52)."""
from ..distributed import DistributedGroupedDataParallel
from . import host

_groups = {"moe": None}


def set_moe_group(moe_group):
    """Remembers the process group over which the experts are spread (fmoefy sets it when pipeline stages
    split the world)."""
    _groups["moe"] = moe_group


def get_moe_group():
    return _groups["moe"]


class DistributedDataParallel(DistributedGroupedDataParallel):
    """Replaces Megatron's DDP: gradients are reduced per ``dp_comm`` tag over the model-parallel, the
    data-parallel and the MoE group, so expert parameters (tag "none") are left alone.  State-dict calls go
    to the wrapped module, so checkpoints look as they do without the wrapper."""

    def __init__(self, module):
        mpu = host.get_mpu()
        model_parallel = getattr(mpu, "get_model_parallel_group", None) or mpu.get_tensor_model_parallel_group
        super().__init__(module, mp_group=model_parallel(), dp_group=mpu.get_data_parallel_group(),
                         moe_group=get_moe_group())


def _forward_to_module(name):
    def call(self, *args, **kwargs):
        return getattr(self.module, name)(*args, **kwargs)
    call.__name__ = name
    call.__doc__ = f"``module.{name}`` (Megatron calls it on the wrapper)."
    return call


for _name in ("state_dict", "state_dict_for_save_checkpoint", "load_state_dict"):
    setattr(DistributedDataParallel, _name, _forward_to_module(_name))
