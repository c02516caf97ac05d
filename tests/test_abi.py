"""C-ABI checks that need no GPU: the library loads, exports every declared symbol,
validates arguments, and its host-only planners agree with the oracle."""
import ctypes
import os
import re

import numpy as np
import pytest

from oracle import moe_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(fmoe_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    from fastermoe_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in include/ but not exported"
    assert set(_lib.EXPORTS) == names
    assert _lib.lib.fmoe_built_for_sm() == 100


def test_argument_validation_reports_errors():
    from fastermoe_b200 import _lib
    lib = _lib.lib
    rc = lib.fmoe_limit_by_capacity(None, None, None, 2, 2, None)
    assert rc == -1 and "null" in _lib.last_error()
    dummy = ctypes.c_void_p(16)  # never dereferenced: the size check fails first
    rc = lib.fmoe_expert_count(dummy, dummy, 10, 0, None)
    assert rc == -1 and "n_expert_total" in _lib.last_error()
    rc = lib.fmoe_expert_count(dummy, dummy, 10, _lib.MAX_EXPERTS + 1, None)
    assert rc == -1
    rc = lib.fmoe_linear_forward(None, None, None, None, None, None, 4, 0, 8, 1, 0, 0, None)
    assert rc == -1 and "bad sizes" in _lib.last_error()
    rc = lib.fmoe_linear_forward(None, None, None, None, None, None, 4, 8, 8, 1, 7, 0, None)
    assert rc == -1 and "dtype" in _lib.last_error()
    with pytest.raises(RuntimeError, match="status -1"):
        _lib.check(rc, "linear_forward")
    assert lib.fmoe_routing_scratch_bytes(1 << 20, 16) > 0


def _plan(lec, gec, stored, rank, E, W):
    from fastermoe_b200 import _lib
    lec = np.ascontiguousarray(lec, dtype=np.int64)
    gec = np.ascontiguousarray(gec, dtype=np.int64)
    st = np.ascontiguousarray(stored, dtype=np.uint8)
    moves = (_lib.Move * (4 * E * W + 8))()
    n, rows = ctypes.c_int32(), ctypes.c_int64()
    rc = _lib.lib.fmoe_plan_global_scatter(lec.ctypes.data, gec.ctypes.data, st.ctypes.data, rank, E, W,
                                           ctypes.cast(moves, ctypes.c_void_p), len(moves), ctypes.byref(n),
                                           ctypes.byref(rows))
    return rc, [moves[i] for i in range(n.value)], rows.value


@pytest.mark.parametrize("shadow", [None, 1, 3])
def test_plan_global_scatter_matches_oracle(shadow):
    rng = np.random.default_rng(3)
    W, E = 4, 3
    lecs = [rng.integers(0, 5, size=W * E) for _ in range(W)]
    stored = np.zeros(W * E, bool)
    if shadow is not None:
        stored[shadow * E:(shadow + 1) * E] = True
    _, _, gecs = O.expert_exchange(lecs, E, W)
    for r in range(W):
        rc, moves, rows = _plan(lecs[r], gecs[r], stored, r, E, W)
        assert rc == 0
        want, want_rows = O.scatter_moves(lecs, stored, r, E, W)
        assert rows == want_rows
        # receives and local copies, in buffer order, must tile the expert-side buffer
        got_recv = sorted((m.dst_row, m.rows, m.peer) for m in moves if (m.local or not m.is_send) and m.rows)
        want_recv = sorted((dst, n, src) for (src, _, dst, n) in want if n)
        assert got_recv == want_recv
        # sends carry the source offsets the oracle expects on the other side
        for m in moves:
            if m.is_send and not m.local:
                w_moves, _ = O.scatter_moves(lecs, stored, m.peer, E, W)
                assert (r, m.src_row) in {(s, sr) for (s, sr, _, n) in w_moves if n == m.rows}


def test_plan_detects_inconsistent_counts():
    from fastermoe_b200 import _lib
    lec = np.array([2, 1, 0, 3]); gec = np.array([5, 1, 0, 3])  # rank 0 keeps 2 rows but expects 5
    rc, _, _ = _plan(lec, gec, np.zeros(4, bool), 0, 2, 2)
    assert rc == -5 and "keeps" in _lib.last_error()


def test_fused_compute_ptrs_matches_oracle():
    from fastermoe_b200 import _lib
    rng = np.random.default_rng(5)
    W, E = 4, 2
    lecs = [rng.integers(0, 7, size=W * E) for _ in range(W)]
    _, _, gecs = O.expert_exchange(lecs, E, W)
    for stored in (np.zeros(W * E, bool), np.repeat(np.array([True, False, False, True]), E)):
        for r in range(W):
            outs = [np.zeros(W * E + 1, dtype=np.int64) for _ in range(3)]
            lec = np.ascontiguousarray(lecs[r], dtype=np.int64)
            gec = np.ascontiguousarray(gecs[r], dtype=np.int64)
            st = stored.astype(np.uint8)
            rc = _lib.lib.fmoe_fused_compute_ptrs(lec.ctypes.data, gec.ctypes.data, st.ctypes.data, r, E, W,
                                                  *[o.ctypes.data for o in outs])
            assert rc == 0
            want = O.fused_compute_ptrs(lec, gec, stored, r, E, W)
            for g, w in zip(outs, want):
                assert np.array_equal(g, w)


def test_product_never_imports_oracle():
    pkg = os.path.join(ROOT, "fastermoe_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                assert "oracle" not in open(os.path.join(base, f)).read().lower().replace("test oracle", ""), f


def test_pool_allocator_without_a_pool():
    """The torch-allocator entry points answer NULL (out of memory) when no receive pool exists,
    and accept a free of memory they do not own."""
    import ctypes
    from fastermoe_b200 import _lib
    assert _lib.lib.fmoe_pool_alloc(1 << 20, 0, None) is None
    _lib.lib.fmoe_pool_free(ctypes.c_void_p(4096), 1 << 20, 0, None)
    assert _lib.lib.fmoe_peer_pool_bytes(None) == 0


def test_struct_mirrors_have_the_library_s_sizes():
    """The ctypes mirrors of the structs that cross the C ABI are as large as the library's own."""
    import ctypes
    from fastermoe_b200 import _lib
    for name, mirror in (("fmoe_move_t", _lib.Move), ("fmoe_peer_seg_t", _lib.PeerSeg), ("fmoe_arrival_t", _lib.Arrival),
                         ("fmoe_mlp_params_t", _lib.MlpParams), ("fmoe_fused_geometry_t", _lib.FusedGeometry)):
        assert _lib.lib.fmoe_abi_sizeof(name.encode()) == ctypes.sizeof(mirror), name
    assert _lib.lib.fmoe_abi_sizeof(b"no_such_struct") == 0
