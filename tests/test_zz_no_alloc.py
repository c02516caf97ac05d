"""fmoe_count_and_pos_static: bucketing for callers that cannot hand the library a scratch
buffer because they may not allocate device memory on this path (a serving process whose
pool owns all free HBM, a plugin host that keeps cudaMalloc off its request path).

The entry point is called through the C ABI with inputs and outputs the test owns, twice in a
row on different inputs (the built-in scratch array keeps the previous call's contents), and
must give exactly what fmoe_count_and_pos gives with caller-provided scratch.  Collected last
on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _both(lib, gate, n_expert):
    n, dev = gate.numel(), gate.device
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = []
    for static in (False, True):
        lec = torch.full((n_expert,), -5, dtype=torch.int64, device=dev)
        off = torch.full((n_expert + 1,), -5, dtype=torch.int64, device=dev)
        pos = torch.full((n,), -5, dtype=torch.int64, device=dev)
        inv = torch.full((n,), -5, dtype=torch.int64, device=dev)
        if static:
            rc = lib.fmoe_count_and_pos_static(_ptr(gate), n, n_expert, _ptr(lec), _ptr(off), _ptr(pos), _ptr(inv),
                                               stream)
        else:
            scratch = torch.empty(lib.fmoe_routing_scratch_bytes(n, n_expert), dtype=torch.uint8, device=dev)
            rc = lib.fmoe_count_and_pos(_ptr(gate), n, n_expert, _ptr(lec), _ptr(off), _ptr(pos), _ptr(inv),
                                        _ptr(scratch), stream)
        assert rc == 0
        torch.cuda.synchronize()
        outs.append((lec, off, pos, inv))
    return outs


def test_static_scratch_matches_caller_scratch_twice():
    from fastermoe_b200 import _lib
    lib = _lib.lib
    assert lib.fmoe_static_scratch_capacity() >= 4 * 1024 * 1024
    rng = np.random.default_rng(0)
    # two calls in a row: a large case first, then a smaller one with other experts, so that the
    # second call runs over whatever the first left in the shared array
    for n, n_expert in ((300000, 64), (32768, 16), (5, 3)):
        g = rng.integers(-1, n_expert, size=n)
        gate = torch.from_numpy(g).cuda()
        ref, got = _both(lib, gate, n_expert)
        for a, b, name in zip(ref, got, ("lec", "offsets", "pos", "inv")):
            assert torch.equal(a, b), f"{name} differs for n={n}, experts={n_expert}"
        assert int(ref[1][-1]) == int((g >= 0).sum())


def test_static_calls_queued_back_to_back_and_edge_sizes():
    """Calls that follow each other on one stream need no host synchronisation between them and
    nothing cleared: calls with different sizes and expert counts (small inputs take the single-launch
    form, large ones the four passes, where more than 256 experts make the tile scan run several
    passes; n = 0 reads nothing) are queued without a sync, then every
    output is compared with fmoe_count_and_pos and with the oracle."""
    from fastermoe_b200 import _lib
    from oracle import moe_oracle as O
    lib = _lib.lib
    rng = np.random.default_rng(1)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    cases = [(200000, 8), (0, 5), (20000, 300), (140000, 300), (777, 1)]
    assert all(lib.fmoe_routing_scratch_bytes(n, e) <= lib.fmoe_static_scratch_capacity() for n, e in cases)
    gates, outs = [], []
    for n, n_expert in cases:                               # queued back to back, no sync in between
        g = rng.integers(-1, n_expert, size=n)
        gate = torch.from_numpy(g).cuda()
        lec = torch.full((n_expert,), -5, dtype=torch.int64, device="cuda")
        off = torch.full((n_expert + 1,), -5, dtype=torch.int64, device="cuda")
        pos = torch.full((max(n, 1),), -5, dtype=torch.int64, device="cuda")
        inv = torch.full((max(n, 1),), -5, dtype=torch.int64, device="cuda")
        assert lib.fmoe_count_and_pos_static(_ptr(gate), n, n_expert, _ptr(lec), _ptr(off), _ptr(pos), _ptr(inv), stream) == 0
        gates.append((g, gate))
        outs.append((lec, off, pos, inv))
    torch.cuda.synchronize()
    for (n, n_expert), (g, gate), (lec, off, pos, inv) in zip(cases, gates, outs):
        cnt = O.expert_count(g, n_expert)
        want_pos = O.assign_pos(g, n_expert)
        assert np.array_equal(lec.cpu().numpy(), cnt), (n, n_expert)
        assert np.array_equal(off.cpu().numpy(), np.concatenate([[0], np.cumsum(cnt)])), (n, n_expert)
        assert np.array_equal(pos.cpu().numpy()[:len(want_pos)], want_pos), (n, n_expert)
        if n:
            assert np.array_equal(inv.cpu().numpy(), O.inverse_pos(want_pos, n)), (n, n_expert)
            ref, _ = _both(lib, gate, n_expert)
            assert torch.equal(ref[2], pos) and torch.equal(ref[3], inv)


def test_static_scratch_rejects_oversized_requests():
    from fastermoe_b200 import _lib
    lib = _lib.lib
    n, n_expert = 1 << 22, 4096           # needs far more than the built-in array holds
    assert lib.fmoe_routing_scratch_bytes(n, n_expert) > lib.fmoe_static_scratch_capacity()
    gate = torch.zeros(16, dtype=torch.int64, device="cuda")   # never read: the size check comes first
    out = torch.zeros(16, dtype=torch.int64, device="cuda")
    rc = lib.fmoe_count_and_pos_static(_ptr(gate), n, n_expert, None, _ptr(out), _ptr(out), None, None)
    assert rc == -4
    assert "built-in" in _lib.last_error() and "fmoe_count_and_pos" in _lib.last_error()
