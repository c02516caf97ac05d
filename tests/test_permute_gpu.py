"""Permutation kernels: byte-exact copies, deterministic sums, gate-score combine."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


@pytest.fixture(scope="module")
def fc():
    from fastermoe_b200 import fmoe_cuda
    return fmoe_cuda


def routing(T, k, E, seed, skip=0.1):
    rng = np.random.default_rng(seed)
    g = rng.integers(0, E, size=(T, k))
    g[rng.random((T, k)) < skip] = -1
    pos = O.assign_pos(g, E)
    return g, pos, O.inverse_pos(pos, T * k)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,k,d", [(12, 2, 6), (257, 2, 1024), (64, 3, 40), (1000, 1, 2050), (33, 2, 7)])
def test_scatter_gather_roundtrip(fc, dtype, T, k, d):
    g, pos, inv = routing(T, k, 5, T + d)
    x = torch.randn(T, d).to(dtype).cuda()
    pos_t, inv_t = torch.from_numpy(pos).cuda(), torch.from_numpy(inv).cuda()
    buf = fc.local_scatter(x, pos_t, pos_div=k)
    assert torch.equal(buf, x[pos_t // k])                              # fmoe/functions.py:72-74
    buf2 = fc.local_scatter(x, (pos_t // k).contiguous())
    assert torch.equal(buf2, buf)
    want = torch.zeros(T * k, d, dtype=dtype, device="cuda")
    want[pos_t] = buf                                                   # index_copy_ semantics
    assert torch.equal(fc.local_gather(buf, pos_t, T * k), want)
    assert torch.equal(fc.local_gather_inv(buf, inv_t), want)


def test_scatter_golden(fc, golden):
    inp = torch.from_numpy(golden["local/inp"]).cuda()
    pos = torch.from_numpy(golden["local/pos"]).cuda()
    buf = fc.local_scatter(inp, pos, pos_div=2)
    assert np.array_equal(buf.cpu().numpy(), golden["local/buf"])
    assert np.array_equal(fc.local_gather(buf, pos, 24).cpu().numpy(), golden["local/back_copy"])
    inv = torch.from_numpy(O.inverse_pos(golden["local/pos"], 24)).cuda()
    add = fc.local_gather_sum(buf, inv, 12, 2)
    np.testing.assert_allclose(add.cpu().numpy(), golden["local/back_add"], rtol=1e-6, atol=1e-7)


def test_scatter_unaligned_rows(fc):
    base = torch.randn(50 * 9 + 1).cuda()
    x = base[1:].view(50, 9)  # 4-byte aligned rows of 36 bytes
    pos = torch.randint(0, 50, (80,)).cuda()
    assert torch.equal(fc.local_scatter(x.contiguous(), pos), x[pos])
    xh = torch.randn(50, 9).half().cuda()
    assert torch.equal(fc.local_scatter(xh, pos), xh[pos])


def test_scatter_marks_empty_slots_zero(fc):
    x = torch.randn(8, 16).cuda()
    pos = torch.tensor([3, -1, 15, 99], device="cuda")
    out = fc.local_scatter(x, pos, pos_div=2)
    assert torch.equal(out[0], x[1]) and torch.equal(out[2], x[7])
    assert out[1].abs().sum() == 0 and out[3].abs().sum() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,k,d", [(64, 2, 128), (257, 3, 1024), (33, 2, 7), (10, 1, 50)])
def test_gather_sum(fc, dtype, T, k, d):
    g, pos, inv = routing(T, k, 4, 3 * T + d)
    buf = torch.randn(len(pos), d).to(dtype).cuda()
    inv_t = torch.from_numpy(inv).cuda()
    got = fc.local_gather_sum(buf, inv_t, T, k)
    want = torch.zeros(T, d, dtype=torch.float32, device="cuda")
    want.index_add_(0, torch.from_numpy(pos // k).cuda(), buf.float())   # fmoe/functions.py:80-81
    tol = dict(rtol=1e-6, atol=1e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got.float(), want, **tol)
    assert torch.equal(got, fc.local_gather_sum(buf, inv_t, T, k))          # fixed summation order


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,k,d", [(64, 2, 128), (257, 3, 1024), (33, 2, 7)])
def test_combine_forward_backward(fc, dtype, T, k, d):
    torch.manual_seed(1000 * T + d)
    g, pos, inv = routing(T, k, 4, 7 * T + d)
    buf = torch.randn(len(pos), d).to(dtype).cuda()
    score = torch.rand(T, k).to(dtype).cuda()
    inv_t, pos_t = torch.from_numpy(inv).cuda(), torch.from_numpy(pos).cuda()

    bufr = buf.float().requires_grad_(True)
    scr = score.float().requires_grad_(True)
    full = torch.zeros(T * k, d, device="cuda").index_copy(0, pos_t, bufr)      # _local_gather
    want = torch.bmm(scr.view(T, 1, k), full.view(T, k, d)).reshape(T, d)      # fmoe/layers.py:321-322
    go = torch.randn(T, d).to(dtype).cuda()
    want.backward(go.float())

    got = fc.combine_forward(buf, inv_t, score)
    gb, gs = fc.combine_backward(go, buf, inv_t, score)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got.float(), want, **tol)
    torch.testing.assert_close(gb.float(), bufr.grad, **tol)
    # the score gradient is a d-term dot product of unit-variance values: two fp32 summation orders differ by
    # a few ulp x sqrt(d) in absolute terms, whatever the size of the (possibly cancelling) result
    gtol = (dict(rtol=1e-5, atol=8 * 2.0 ** -23 * float(np.sqrt(d))) if dtype == torch.float32
            else dict(rtol=3e-2, atol=3e-2 * float(np.sqrt(d))))
    torch.testing.assert_close(gs.float(), scr.grad, **gtol)
    # dense form (no permutation): x [T*k, d]
    xd = torch.randn(T * k, d).to(dtype).cuda()
    got2 = fc.combine_forward(xd, None, score)
    want2 = torch.bmm(score.float().view(T, 1, k), xd.float().view(T, k, d)).reshape(T, d)
    torch.testing.assert_close(got2.float(), want2, **tol)
