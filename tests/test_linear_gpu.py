"""Grouped expert GEMM (fmoe_linear) forward/backward against per-expert fp32 matmuls.

Tolerances: fp32 rtol 1e-5 (absolute floor for long sums that cancel); bf16/fp16 rtol 2e-2
against an fp32 reference, with an absolute floor of a few output roundings (2^-9 relative for
bf16) of a typical element, which only matters for entries that cancel to almost nothing."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fc():
    from fastermoe_b200 import fmoe_cuda
    return fmoe_cuda


def reference(x, counts, w, b, gy):
    """cuda/parallel_linear.cuh:55-161 as per-expert fp32 matmuls."""
    x, w, gy = x.float(), w.float(), gy.float()
    y = torch.zeros(x.shape[0], w.shape[1], device=x.device)
    gx = torch.zeros_like(x)
    gw = torch.zeros_like(w)
    gb = torch.zeros(w.shape[0], w.shape[1], device=x.device)
    p = 0
    for e, c in enumerate(counts):
        s = slice(p, p + c)
        y[s] = x[s] @ w[e].t() + (b[e].float() if b is not None else 0)
        gx[s] = gy[s] @ w[e]
        gw[e] = gy[s].t() @ x[s]
        gb[e] = gy[s].sum(0)
        p += c
    return y, gx, gw, gb


def tolerances(dtype, k, want, roundings=1):
    """``roundings``: 16-bit roundings between the inputs and this result (1 for a single product;
    more when intermediate tensors of a chain were stored in 16 bits and the reference kept fp32)."""
    if dtype == torch.float32:
        return dict(rtol=1e-5, atol=1e-5 * float(np.sqrt(k)))
    rms = float(want.float().pow(2).mean().sqrt()) if want.numel() else 0.0
    return dict(rtol=2e-2, atol=4 * roundings * 2.0 ** -9 * rms)


SHAPES = [
    # counts, in_feat, out_feat
    ([4, 0, 3, 5], 16, 32),
    ([1, 1, 1, 1, 1, 1, 1, 1], 32, 16),
    ([130, 0, 77, 300], 128, 256),
    ([0, 0, 0, 9], 24, 40),
    ([257, 511, 64, 128], 1024, 512),
    ([700, 900], 256, 1024),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("counts,fin,fout", SHAPES)
@pytest.mark.parametrize("bias", [True, False])
def test_linear_forward_backward(fc, dtype, counts, fin, fout, bias):
    torch.manual_seed(sum(counts) + fin)
    E, B = len(counts), sum(counts)
    x = torch.randn(B, fin, device="cuda").to(dtype)
    w = ((torch.rand(E, fout, fin, device="cuda") * 2 - 1) / np.sqrt(fin)).to(dtype)
    b = ((torch.rand(E, fout, device="cuda") * 2 - 1) / np.sqrt(fin)).to(dtype) if bias else None
    gy = torch.randn(B, fout, device="cuda").to(dtype)
    cnt = torch.tensor(counts, dtype=torch.int64)                 # CPU tensor, as the reference requires
    y = fc.linear_forward(x, cnt, w, b)
    gx, gw, gb = fc.linear_backward(gy, x, cnt, w, b)
    wy, wgx, wgw, wgb = reference(x, counts, w, b, gy)
    torch.testing.assert_close(y.float(), wy, **tolerances(dtype, fin, wy))
    torch.testing.assert_close(gx.float(), wgx, **tolerances(dtype, fout, wgx))
    torch.testing.assert_close(gw.float(), wgw, **tolerances(dtype, max(counts), wgw))
    torch.testing.assert_close(gb.float(), wgb, **tolerances(dtype, max(counts), wgb))
    # the count vector may also live on the GPU
    y2 = fc.linear_forward(x, cnt.cuda(), w, b)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", ["relu", "gelu"])
def test_fused_mlp_matches_autograd(fc, dtype, act):
    """Linear -> activation -> Linear with fused epilogues against plain autograd in fp32."""
    from fastermoe_b200.functions import FusedExpertMLP
    from fastermoe_b200 import _lib
    torch.manual_seed(3)
    counts, d, h = [100, 0, 157, 31], 64, 256
    E, B = len(counts), sum(counts)
    off = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int64, device="cuda")
    mk = lambda *s, f: (((torch.rand(*s, device="cuda") * 2 - 1) / np.sqrt(f)).to(dtype)).requires_grad_(True)
    x = torch.randn(B, d, device="cuda").to(dtype).requires_grad_(True)
    w1, b1, w2, b2 = mk(E, h, d, f=d), mk(E, h, f=d), mk(E, d, h, f=h), mk(E, d, f=h)
    code = {"relu": _lib.ACT_RELU, "gelu": _lib.ACT_GELU}[act]
    y = FusedExpertMLP.apply(x, off, w1, b1, w2, b2, code)
    gy = torch.randn_like(y)
    y.backward(gy)
    got = [y, x.grad, w1.grad, b1.grad, w2.grad, b2.grad]

    leaves = [t.detach().float().requires_grad_(True) for t in (x, w1, b1, w2, b2)]
    xr, w1r, b1r, w2r, b2r = leaves
    f = torch.relu if act == "relu" else torch.nn.functional.gelu
    outs, p = [], 0
    for e, c in enumerate(counts):
        hmid = f(xr[p:p + c] @ w1r[e].t() + b1r[e])
        outs.append(hmid @ w2r[e].t() + b2r[e])
        p += c
    yr = torch.cat(outs)
    yr.backward(gy.float())
    want = [yr.detach()] + [t.grad for t in leaves]
    # the hidden activations and their gradient are stored in 16 bits on the way, the reference keeps fp32
    for name, g, w_, k, nr in zip(["y", "gx", "gw1", "gb1", "gw2", "gb2"], got, want, [h, h, 157, 157, 157, 157],
                                  [2, 3, 3, 3, 2, 1]):
        torch.testing.assert_close(g.float(), w_, **tolerances(dtype, k, w_, nr), msg=lambda m, n=name: f"{n}: {m}")
