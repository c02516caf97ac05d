"""This library's operators next to the reference's own CUDA operators (compiled by
oracle/build_ref.py into oracle/_ref) on the same GPU inputs.  Skipped when that build is absent."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import build_ref
    mod = build_ref.load()
    if mod is None:
        pytest.skip("oracle/_ref is not built")
    return mod


@pytest.fixture(scope="module")
def fc():
    from fastermoe_b200 import fmoe_cuda
    return fmoe_cuda


@pytest.mark.parametrize("n,E", [(64, 4), (1000, 7), (32768, 16), (100003, 257)])
def test_count_and_positions(ref, fc, n, E):
    rng = np.random.default_rng(n)
    g = rng.integers(-1, E, size=n)
    gate = torch.from_numpy(g).cuda()
    c_ref = torch.zeros(E, dtype=torch.int32, device="cuda"); ref.expert_count(gate, c_ref)
    c_new = torch.zeros(E, dtype=torch.int32, device="cuda"); fc.expert_count(gate, c_new)
    assert torch.equal(c_ref, c_new)
    cum_r = torch.cumsum(c_ref, 0).int(); cum_n = cum_r.clone()
    total = int(cum_r[-1].item())
    p_ref = torch.empty(total, dtype=torch.int64, device="cuda"); ref.assign_pos(cum_r, gate, p_ref)
    p_new = torch.empty(total, dtype=torch.int64, device="cuda"); fc.assign_pos(cum_n, gate, p_new)
    assert torch.equal(cum_r, cum_n)                       # both leave the exclusive prefix behind
    # the reference's order inside a segment is arbitrary: compare segments as sorted sets
    canon = O.canonical_pos(p_ref.cpu().numpy(), c_ref.cpu().numpy())
    assert np.array_equal(canon, p_new.cpu().numpy())


@pytest.mark.parametrize("W,E", [(1, 4), (8, 2), (4, 16)])
def test_limit_by_capacity(ref, fc, W, E):
    rng = np.random.default_rng(W * 10 + E)
    ec = torch.from_numpy(rng.integers(0, 40, size=W * E)).cuda()
    cap = rng.integers(0, 100, size=E).astype(np.int32)
    cap_r, cap_n = torch.from_numpy(cap.copy()).cuda(), torch.from_numpy(cap.copy()).cuda()
    e_ref = ref.limit_by_capacity(ec, cap_r, E, W)
    e_new = fc.limit_by_capacity(ec, cap_n, E, W)
    assert torch.equal(cap_r, cap_n)
    # per expert the total granted is the same; per source it is when at most one source is cut
    assert torch.equal(e_ref.view(W, E).sum(0), e_new.view(W, E).sum(0))
    assert bool((e_new <= ec).all()) and bool((e_ref <= ec).all())
    if W == 1:
        assert torch.equal(e_ref, e_new)


@pytest.mark.parametrize("n,E", [(256, 4), (4096, 16), (20000, 64)])
def test_prune_gate(ref, fc, n, E):
    rng = np.random.default_rng(n + E)
    g = torch.from_numpy(rng.integers(0, E, size=n)).cuda()     # no -1: the reference does not guard it
    ec = rng.integers(0, 2 * n // E, size=E).astype(np.int32)
    ec_r, ec_n = torch.from_numpy(ec.copy()).cuda(), torch.from_numpy(ec.copy()).cuda()
    p_ref = ref.prune_gate_by_capacity(g, ec_r, E, 1)
    p_new = fc.prune_gate_by_capacity(g, ec_n, E, 1)
    assert torch.equal(ec_r, ec_n)
    kept_r = O.expert_count(p_ref.cpu().numpy(), E)
    kept_n = O.expert_count(p_new.cpu().numpy(), E)
    assert np.array_equal(kept_r, kept_n)                                   # same number kept per expert
    assert bool(((p_ref == g) | (p_ref == -1)).all()) and bool(((p_new == g) | (p_new == -1)).all())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 2e-2)])
def test_linear(ref, fc, dtype, tol):
    torch.manual_seed(0)
    counts, fin, fout = [130, 0, 77, 300], 128, 256
    B = sum(counts)
    x = torch.randn(B, fin, device="cuda").to(dtype)
    w = (torch.randn(len(counts), fout, fin, device="cuda") / 11).to(dtype)
    b = torch.randn(len(counts), fout, device="cuda").to(dtype)
    gy = torch.randn(B, fout, device="cuda").to(dtype)
    cnt = torch.tensor(counts, dtype=torch.int64)
    y_r = ref.linear_forward(x, cnt, w, b)
    gx_r, gw_r, gb_r = ref.linear_backward(gy, x, cnt, w, b)
    y_n = fc.linear_forward(x, cnt, w, b)
    gx_n, gw_n, gb_n = fc.linear_backward(gy, x, cnt, w, b)
    for name, a, b_ in (("y", y_n, y_r), ("gx", gx_n, gx_r), ("gw", gw_n, gw_r), ("gb", gb_n, gb_r)):
        scale = float(b_.float().abs().max())
        torch.testing.assert_close(a.float(), b_.float(), rtol=tol, atol=tol * scale, msg=lambda m, n=name: f"{n}: {m}")
