"""Routing kernels against the oracle: counts, positions, capacity (bit-exact)."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

CASES = [(0, 4), (1, 1), (5, 3), (64, 16), (257, 7), (4096, 64), (32768, 16), (32768, 32), (100003, 257),
         (70000, 4096), (1 << 22, 16)]


def make_gate(n, E, seed, frac_skip=0.1):
    rng = np.random.default_rng(seed)
    g = rng.integers(0, E, size=n)
    g[rng.random(n) < frac_skip] = -1
    return g


@pytest.fixture(scope="module")
def fc():
    from fastermoe_b200 import fmoe_cuda
    return fmoe_cuda


@pytest.mark.parametrize("n,E", CASES)
def test_expert_count(fc, n, E):
    g = make_gate(n, E, n + E)
    gate = torch.from_numpy(g).cuda()
    cnt = torch.zeros(E, dtype=torch.int32, device="cuda")
    fc.expert_count(gate, cnt)
    want = O.expert_count(g, E)
    assert np.array_equal(cnt.cpu().numpy(), want)
    fc.expert_count(gate, cnt)  # accumulates, like the reference
    assert np.array_equal(cnt.cpu().numpy(), 2 * want)


@pytest.mark.parametrize("n,E", CASES)
def test_assign_pos(fc, n, E):
    g = make_gate(n, E, 3 * n + E)
    gate = torch.from_numpy(g).cuda()
    cnt = O.expert_count(g, E)
    cum = torch.from_numpy(np.cumsum(cnt).astype(np.int32)).cuda()
    pos = torch.full((int(cnt.sum()),), -7, dtype=torch.int64, device="cuda")
    fc.assign_pos(cum, gate, pos)
    assert np.array_equal(pos.cpu().numpy(), O.assign_pos(g, E))
    # the reference's atomicSub leaves the exclusive prefix sum behind
    assert np.array_equal(cum.cpu().numpy(), (np.cumsum(cnt) - cnt).astype(np.int32))


@pytest.mark.parametrize("n,E", CASES)
def test_count_and_pos(fc, n, E):
    g = make_gate(n, E, 5 * n + E)
    gate = torch.from_numpy(g).cuda()
    lec, off, pos, inv = fc.count_and_pos(gate, E)
    cnt = O.expert_count(g, E).astype(np.int64)
    want_pos = O.assign_pos(g, E)
    assert np.array_equal(lec.cpu().numpy(), cnt)
    assert np.array_equal(off.cpu().numpy(), np.concatenate([[0], np.cumsum(cnt)]))
    p = pos.cpu().numpy()
    assert np.array_equal(p[:len(want_pos)], want_pos)
    assert np.all(p[len(want_pos):] == -1)
    assert np.array_equal(inv.cpu().numpy(), O.inverse_pos(want_pos, n))


def test_unaligned_gate_pointer(fc):
    g = make_gate(5001, 9, 77)
    base = torch.from_numpy(np.concatenate([[0], g])).cuda()
    gate = base[1:]  # 8-byte aligned only: the 16-byte load path must not be taken
    assert gate.data_ptr() % 16 == 8
    lec, off, pos, inv = fc.count_and_pos(gate, 9)
    want_pos = O.assign_pos(g, 9)
    assert np.array_equal(pos.cpu().numpy()[:len(want_pos)], want_pos)
    cnt = torch.zeros(9, dtype=torch.int32, device="cuda")
    fc.expert_count(gate, cnt)
    assert np.array_equal(cnt.cpu().numpy(), O.expert_count(g, 9))


def test_run_to_run_determinism(fc):
    g = make_gate(200000, 32, 5)
    gate = torch.from_numpy(g).cuda()
    a = fc.count_and_pos(gate, 32)[2].clone()
    for _ in range(3):
        assert torch.equal(fc.count_and_pos(gate, 32)[2], a)


@pytest.mark.parametrize("W,E", [(1, 4), (2, 1), (8, 2), (8, 4), (64, 33)])
def test_limit_by_capacity(fc, W, E):
    rng = np.random.default_rng(W * 100 + E)
    ec = rng.integers(0, 50, size=W * E)
    cap = rng.integers(0, 120, size=E).astype(np.int32)
    cap_t = torch.from_numpy(cap.copy()).cuda()
    out = fc.limit_by_capacity(torch.from_numpy(ec).cuda(), cap_t, E, W)
    want, left = O.limit_by_capacity(ec, cap, E, W)
    assert np.array_equal(out.cpu().numpy(), want)
    assert np.array_equal(cap_t.cpu().numpy(), left)
    # reference invariants: sum of grants = min(cap, sum of requests), grant <= request
    tot = want.reshape(W, E).sum(0)
    assert np.array_equal(tot, np.minimum(cap, ec.reshape(W, E).sum(0)))


@pytest.mark.parametrize("n,E", [(0, 4), (33, 2), (4096, 16), (32768, 16), (100003, 257)])
@pytest.mark.parametrize("with_skips", [False, True])
def test_prune_gate_by_capacity(fc, n, E, with_skips):
    g = make_gate(n, E, 11 * n + E, frac_skip=0.1 if with_skips else 0.0).reshape(-1, 1)
    rng = np.random.default_rng(n)
    ec = rng.integers(0, max(2, 2 * n // max(E, 1)), size=E).astype(np.int32)
    ec_t = torch.from_numpy(ec.copy()).cuda()
    out = fc.prune_gate_by_capacity(torch.from_numpy(g).cuda(), ec_t, E, 1)
    want, left = O.prune_gate_by_capacity(g, ec)
    assert out.shape == g.shape
    assert np.array_equal(out.cpu().numpy(), want)
    assert np.array_equal(ec_t.cpu().numpy(), left)


def test_capacity_gate_pipeline_single_worker(fc):
    """limit_by_capacity wrapper (count -> limit -> prune) against the oracle, and the
    bound the reference's gate test checks (tests/test_gates.py:55-57)."""
    from fastermoe_b200.gates.utils import limit_by_capacity
    g = make_gate(8192 * 2, 16, 4, frac_skip=0.0).reshape(8192, 2)
    g[:6000, 0] = 3  # one hot expert
    cap = 1500
    new_lec, new_gec, pruned = limit_by_capacity(torch.from_numpy(g).cuda(), 16, 1, cap)
    (w_lec, w_gec, w_pruned), = O.limit_by_capacity_gate([g], 16, 1, cap)
    assert np.array_equal(pruned.cpu().numpy(), w_pruned)
    assert np.array_equal(new_lec.cpu().numpy(), w_lec)
    assert O.expert_count(pruned.cpu().numpy(), 16).max() <= cap
