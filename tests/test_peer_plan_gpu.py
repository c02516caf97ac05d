"""The exchange plan as the DEVICE builds it (fmoe_peer_plan_from_table: one GPU, no communicator)
against the library's host mirror (fmoe_peer_plan, itself checked against the oracle's layouts on
the CPU) and against the oracle directly, for every rank of 2..8-rank worlds, with shadowed experts."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from test_peer_plan import plan as host_plan, stored_cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fc():
    from fastermoe_b200 import fmoe_cuda
    return fmoe_cuda


@pytest.mark.parametrize("W,E", [(2, 1), (2, 3), (3, 2), (4, 4), (8, 16), (5, 1), (8, 4), (8, 64)])
def test_device_plan_matches_host_mirror_and_oracle(fc, W, E):
    rng = np.random.default_rng(W * 1000 + E)
    for trial in range(3):
        hi = 9 if trial < 2 else 3000
        lecs = [rng.integers(0, hi, size=W * E).astype(np.int64) for _ in range(W)]
        if trial == 1:
            lecs[0][:] = 0
            for l in lecs:
                l[(W - 1) * E:] = 0
        table, _, gecs = O.expert_exchange(lecs, E, W)
        tab_dev = torch.from_numpy(np.ascontiguousarray(table)).cuda()
        for stored in stored_cases(W, E, rng):
            st_dev = torch.from_numpy(stored.astype(np.uint8)).cuda()
            for r in range(W):
                p = fc.peer_plan_from_table(tab_dev, st_dev, r, E, W)
                assert torch.equal(p.table.cpu(), torch.from_numpy(table))
                for reverse in (0, 1):
                    push, pull, _ = host_plan(table, stored, r, E, W, reverse)
                    got_push, ex_rows, tok_rows, overflow = p.read(2 * reverse)
                    got_pull = p.read(2 * reverse + 1)[0]
                    assert overflow == 0
                    assert got_push == push, f"rank {r} reverse {reverse}: push segments differ"
                    assert got_pull == pull, f"rank {r} reverse {reverse}: pull segments differ"
                    assert tok_rows == int(lecs[r].sum())
                    assert ex_rows == int(O.generate_cached_count(lecs[r], gecs[r], stored, r, E, W).sum())
                # offsets of this rank's experts in its expert-side buffer, from the oracle's row map
                moves, total = O.scatter_moves(lecs, stored, r, E, W)
                own = p.own_offsets.cpu().numpy()
                shadow_before = sum(int(lecs[r][j * E + i]) for j in range(r) for i in range(E) if stored[j * E + i])
                recv = np.array([sum(int(lecs[j][r * E + i]) for j in range(W) if (not stored[r * E + i] or j == r))
                                 for i in range(E)])
                want = shadow_before + np.concatenate([[0], np.cumsum(recv)])
                assert np.array_equal(own, want)
    assert fc.device_status() == 0


def test_device_plan_capacity_overflow(fc):
    """A rank that would receive more rows than its announced capacity empties every rank's plan
    (each rank computes the same verdict from the same table) and raises status bit 64."""
    W, E = 4, 2
    rng = np.random.default_rng(1)
    lecs = [rng.integers(1, 50, size=W * E).astype(np.int64) for _ in range(W)]
    table, _, gecs = O.expert_exchange(lecs, E, W)
    tab_dev = torch.from_numpy(np.ascontiguousarray(table)).cuda()
    recv = [int(g.sum()) for g in gecs]
    caps = torch.tensor([recv[0], recv[1] - 1, recv[2], 10 ** 9], dtype=torch.int64, device="cuda")
    for r in range(W):
        p = fc.peer_plan_from_table(tab_dev, None, r, E, W, caps=caps)
        segs, ex_rows, tok_rows, overflow = p.read(0)
        assert overflow == 1 and segs == [] and ex_rows == 0 and tok_rows == 0
        assert not p.own_offsets.any()
    assert fc.device_status() & 64
    assert fc.lib.fmoe_device_status_clear() == 0
    caps[1] += 1                      # exactly enough room
    p = fc.peer_plan_from_table(tab_dev, None, 1, E, W, caps=caps)
    assert p.read(0)[3] == 0 and int(p.own_offsets[-1]) == recv[1]
    assert fc.device_status() == 0


def test_device_plan_rejects_insane_counts(fc):
    W, E = 2, 2
    table = torch.zeros(W, W, E, dtype=torch.int64, device="cuda")
    table[0, 1, 0] = -5
    p = fc.peer_plan_from_table(table, None, 0, E, W)
    assert p.read(0)[3] == 1 and not p.own_offsets.any()
    table[0, 1, 0] = 2 ** 33
    p = fc.peer_plan_from_table(table, None, 1, E, W)
    assert p.read(2)[3] == 1
