"""Expert-parallel path on 2 (or more) GPUs over NCCL; skipped on a single-GPU box."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

import dist_worker

pytestmark = pytest.mark.gpu


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def world_sizes():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [w for w in (2, 4) if w <= n]


def needs_gpus():
    if not world_sizes():
        pytest.skip("needs at least 2 GPUs")


@pytest.mark.parametrize("fn", ["gpu_exchange", "gpu_layer", "gpu_layer_bf16"])
def test_expert_parallel(fn):
    needs_gpus()
    for world in world_sizes():
        mp.spawn(getattr(dist_worker, fn), args=(world, free_port()), nprocs=world, join=True)
