"""world_size-2 and -4 gloo runs of the host-side logic of the multi-GPU path (no GPU needed)."""
import socket

import pytest
import torch.multiprocessing as mp

import dist_worker


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
def test_exchange_plan_over_gloo(world):
    mp.spawn(dist_worker.cpu_plan_exchange, args=(world, free_port()), nprocs=world, join=True)


def test_grouped_data_parallel_over_gloo():
    mp.spawn(dist_worker.cpu_grouped_ddp, args=(2, free_port()), nprocs=2, join=True)


@pytest.mark.parametrize("world", [2, 3])
def test_slice_and_allgather_over_gloo(world):
    mp.spawn(dist_worker.cpu_slice_allgather, args=(world, free_port()), nprocs=world, join=True)


def test_megatron_wrapper_and_sharded_checkpoint_over_gloo(tmp_path):
    mp.spawn(dist_worker.cpu_megatron_ddp_checkpoint, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)


def test_reference_named_checkpoint_functions_over_gloo(tmp_path):
    mp.spawn(dist_worker.cpu_megatron_named_checkpoint, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
