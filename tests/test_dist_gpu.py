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
    return [w for w in (2, 4, 8) if w <= n]


def needs_gpus():
    if not world_sizes():
        pytest.skip("needs at least 2 GPUs")


def run_ranks(fn, world, limit_s=240):
    """Spawns the ranks and ends them if they do not finish in time (a mismatched exchange
    would otherwise wait for ever)."""
    import time
    ctx = mp.spawn(fn, args=(world, free_port()), nprocs=world, join=False)
    deadline = time.time() + limit_s
    try:
        while not ctx.join(timeout=5):
            if time.time() > deadline:
                raise TimeoutError(f"{fn.__name__} on {world} ranks did not finish within {limit_s} s")
    finally:
        for p in ctx.processes:
            if p.is_alive():
                p.terminate()


@pytest.mark.parametrize("fn", ["gpu_exchange", "gpu_layer", "gpu_layer_bf16", "gpu_config5", "gpu_graph_step"])
def test_expert_parallel(fn):
    needs_gpus()
    for world in world_sizes():
        run_ranks(getattr(dist_worker, fn), world)


def test_full_size_configs():
    """Per-GPU sizes of the Zipf-routed and the one-expert-per-GPU workloads, on 2 GPUs (property checks)."""
    needs_gpus()
    run_ranks(dist_worker.gpu_full_size, 2, limit_s=400)


def test_receive_pool_exhaustion(monkeypatch):
    """With a 1 MB receive pool some exchange outputs fit in it and most do not: rows are then received
    through the landing slots and copied; both ways in one run give the same layer results."""
    needs_gpus()
    monkeypatch.setenv("FMOE_B200_PEER_POOL_MB", "1")
    run_ranks(dist_worker.gpu_layer_bf16, 2)
    monkeypatch.setenv("FMOE_B200_PEER_POOL_MB", "0")
    run_ranks(dist_worker.gpu_layer_bf16, 2)
