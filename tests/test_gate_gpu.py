"""Gate top-k kernels against torch.topk and torch autograd (selection is exact: values are copied)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fc():
    from fastermoe_b200 import fmoe_cuda
    return fmoe_cuda


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n_tok,n_exp,k", [(1, 2, 1), (7, 16, 2), (1000, 16, 2), (333, 33, 4), (64, 100, 8), (5, 4096, 8),
                                           (0, 16, 2), (16384, 16, 2)])
def test_topk_matches_torch(fc, dtype, n_tok, n_exp, k):
    g = torch.Generator().manual_seed(n_tok * 131 + n_exp + k)
    # distinct values per row (a permutation, exactly representable in every dtype), so the order is unique
    base = torch.stack([torch.randperm(n_exp, generator=g) for _ in range(max(n_tok, 1))])[:n_tok]
    logits = ((base.float() - n_exp / 2) * (0.125 if n_exp <= 256 else 1.0)).to(dtype).cuda()
    if dtype != torch.float32 and n_exp > 2048:
        logits = (base.float() % 1024).to(dtype).cuda()       # still exact in 16 bits; ties resolved by index below
    val, idx = fc.gate_topk(logits, k)
    assert val.shape == (n_tok, k) and idx.shape == (n_tok, k) and idx.dtype == torch.int64
    if n_tok == 0:
        return
    f = logits.float().cpu().numpy()
    order = np.lexsort((np.broadcast_to(np.arange(n_exp), f.shape), -f), axis=1)[:, :k]   # value desc, index asc
    assert np.array_equal(idx.cpu().numpy(), order)
    assert torch.equal(val, torch.gather(logits, 1, idx))
    tv, _ = torch.topk(logits.float(), k, dim=-1, largest=True, sorted=True)
    assert torch.equal(val.float(), tv)


def test_topk_ties_and_nan(fc):
    logits = torch.zeros(3, 10, device="cuda")
    logits[1, 7] = float("nan")
    logits[2, 4] = float("inf")
    logits[2, 9] = float("nan")
    val, idx = fc.gate_topk(logits, 3)
    assert idx.tolist() == [[0, 1, 2], [7, 0, 1], [9, 4, 0]]
    assert torch.isnan(val[1, 0]) and torch.isnan(val[2, 0]) and val[2, 1] == float("inf")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_topk_backward_matches_autograd(dtype):
    from fastermoe_b200.functions import gate_topk
    g = torch.Generator().manual_seed(3)
    # distinct values in every row: with ties torch.topk may pick another of the equal entries
    logits = ((torch.stack([torch.randperm(24, generator=g) for _ in range(513)]).float() - 12) * 0.25).to(dtype).cuda()
    a = logits.clone().requires_grad_(True)
    b = logits.clone().requires_grad_(True)
    va, ia = gate_topk(a, 4)
    vb, ib = torch.topk(b, 4, dim=-1, largest=True, sorted=True)
    assert torch.equal(ia, ib) and torch.equal(va, vb)
    torch.manual_seed(4)
    w = torch.randn_like(va)
    (va * w).sum().backward()
    (vb * w).sum().backward()
    assert torch.equal(a.grad, b.grad)
    # leading dimensions are kept
    v3, i3 = gate_topk(logits.view(27, 19, 24), 2)
    assert v3.shape == (27, 19, 2) and i3.shape == (27, 19, 2)


def test_topk_argument_errors(fc):
    with pytest.raises(RuntimeError, match="k="):
        fc.gate_topk(torch.zeros(4, 16, device="cuda"), 9)
    with pytest.raises(RuntimeError, match="k="):
        fc.gate_topk(torch.zeros(4, 2, device="cuda"), 3)
