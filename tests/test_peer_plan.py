"""Host-side plan of the peer-memory token exchange (fmoe_peer_plan) against the oracle's
global_scatter / global_gather: every rank's push and pull segments are applied to numpy buffers
(a dict of landing slots stands in for the peers' memory) and the result must equal the oracle's
layout, with and without shadowed experts.  Runs without a GPU."""
import ctypes

import numpy as np
import pytest

from fastermoe_b200 import _lib
from oracle import moe_oracle as O


def plan(table, stored, rank, E, W, reverse):
    tab = np.ascontiguousarray(table, dtype=np.int64)
    st = np.ascontiguousarray(stored, dtype=np.uint8)
    n_push, n_pull, slot = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int64()
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    rc = _lib.lib.fmoe_peer_plan(p(tab), p(st), rank, E, W, int(reverse), None, ctypes.byref(n_push), None,
                                 ctypes.byref(n_pull), 0, ctypes.byref(slot))
    assert rc == 0, _lib.last_error()
    cap = max(n_push.value, n_pull.value, 1)
    push, pull = (_lib.PeerSeg * cap)(), (_lib.PeerSeg * cap)()
    rc = _lib.lib.fmoe_peer_plan(p(tab), p(st), rank, E, W, int(reverse), push, ctypes.byref(n_push), pull,
                                 ctypes.byref(n_pull), cap, ctypes.byref(slot))
    assert rc == 0, _lib.last_error()
    as_list = lambda arr, n: [(s.dst_rank, s.src_row, s.dst_row, s.rows) for s in arr[:n]]
    return as_list(push, n_push.value), as_list(pull, n_pull.value), slot.value


def exchange(bufs, table, stored, E, W, reverse, out_rows):
    """What the push and consume kernels of all ranks do, in numpy."""
    d = bufs[0].shape[1]
    plans = [plan(table, stored, r, E, W, reverse) for r in range(W)]
    slot_rows = plans[0][2]
    assert all(p[2] == slot_rows for p in plans), "ranks disagree on the slot size"
    landing = [np.full((slot_rows, d), np.nan, dtype=bufs[0].dtype) for _ in range(W)]
    outs = [np.full((out_rows[r], d), np.nan, dtype=bufs[0].dtype) for r in range(W)]
    written = [np.zeros(slot_rows, dtype=np.int32) for _ in range(W)]
    for r in range(W):
        for dst, src_row, dst_row, rows in plans[r][0]:
            assert rows > 0 and src_row + rows <= bufs[r].shape[0]
            if dst == W:
                outs[r][dst_row:dst_row + rows] = bufs[r][src_row:src_row + rows]
            else:
                assert dst != r and dst_row + rows <= slot_rows
                landing[dst][dst_row:dst_row + rows] = bufs[r][src_row:src_row + rows]
                written[dst][dst_row:dst_row + rows] += 1
    for r in range(W):
        assert written[r].max(initial=0) <= 1, "two senders store into the same landing rows"
        for dst, src_row, dst_row, rows in plans[r][1]:
            assert dst == W and (written[r][src_row:src_row + rows] == 1).all(), "consume reads rows nobody stored"
            outs[r][dst_row:dst_row + rows] = landing[r][src_row:src_row + rows]
    return outs, plans


def stored_cases(W, E, rng):
    yield np.zeros(W * E, bool)
    yield np.repeat(np.arange(W) == 0, E)
    yield np.repeat(np.arange(W) == W - 1, E)
    yield rng.random(W * E) < 0.3                   # per-expert shadow flags


@pytest.mark.parametrize("W,E", [(2, 1), (2, 3), (3, 2), (4, 4), (8, 16), (5, 1)])
def test_plan_reproduces_oracle_layout(W, E):
    rng = np.random.default_rng(W * 100 + E)
    for trial in range(3):
        lecs = [rng.integers(0, 9, size=W * E).astype(np.int64) for _ in range(W)]
        if trial == 2:
            lecs[0][:] = 0                                # a rank that sends nothing
            for l in lecs:
                l[(W - 1) * E:] = 0                       # a rank that receives nothing
        table, _, _ = O.expert_exchange(lecs, E, W)
        for stored in stored_cases(W, E, rng):
            bufs = [rng.standard_normal((int(l.sum()), 3)).astype(np.float32) for l in lecs]
            want = O.global_scatter(bufs, lecs, stored, E, W)
            got, plans = exchange(bufs, table, stored, E, W, False, [w.shape[0] for w in want])
            for r in range(W):
                assert np.array_equal(got[r], want[r]), f"scatter layout differs on rank {r}"
            back, _ = exchange(got, table, stored, E, W, True, [b.shape[0] for b in bufs])
            for r in range(W):
                assert np.array_equal(back[r], bufs[r]), f"gather is not the inverse on rank {r}"
            # expert-major, staggered peer order: within one expert round the remote destinations of
            # rank r come in the order r+1, r+2, ...; there are at most E rounds
            for r in range(W):
                dist = [(s[0] - r) % W for s in plans[r][0] if s[0] != W]
                rounds = 1 + sum(1 for a, b in zip(dist, dist[1:]) if b <= a)
                assert rounds <= max(E, 1), "peers are not visited in ring order inside an expert round"


def test_plan_rejects_bad_arguments():
    tab = np.zeros(8, dtype=np.int64)
    tab[3] = -1
    st = np.zeros(4, dtype=np.uint8)
    n1, n2, slot = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int64()
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    rc = _lib.lib.fmoe_peer_plan(p(tab), p(st), 0, 2, 2, 0, None, ctypes.byref(n1), None, ctypes.byref(n2), 0,
                                 ctypes.byref(slot))
    assert rc != 0 and "negative" in _lib.last_error()
    rc = _lib.lib.fmoe_peer_plan(p(np.zeros(8, dtype=np.int64)), p(st), 5, 2, 2, 0, None, ctypes.byref(n1), None,
                                 ctypes.byref(n2), 0, ctypes.byref(slot))
    assert rc != 0
