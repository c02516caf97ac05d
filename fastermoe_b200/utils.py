"""Small helpers shared by the layer code."""
import torch.distributed as dist


def get_torch_default_comm():
    """The default ``torch.distributed`` process group (fmoe/utils.py:9-30).

    The reference digs an NCCL communicator out of this object; here it is only
    used as a channel to broadcast the id of the library's own communicator.
    """
    if not dist.is_available() or not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    return dist.distributed_c10d._get_default_group()
