"""The tcgen05 grouped GEMM kernels (bf16/fp16, feature sizes that are multiples of 64 and >= 256)
against fp32 matmuls and against the FFMA kernels on the same inputs."""
import ctypes
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fc():
    from fastermoe_b200 import fmoe_cuda
    return fmoe_cuda


def device_status():
    from fastermoe_b200 import _lib
    v = ctypes.c_int32(-1)
    assert _lib.lib.fmoe_device_status(ctypes.byref(v)) == 0
    return v.value


def reference(x, counts, w, b, gy, act=None):
    x, w, gy = x.float(), w.float(), gy.float()
    y = torch.zeros(x.shape[0], w.shape[1], device=x.device)
    gx, gw = torch.zeros_like(x), torch.zeros_like(w)
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


def close(got, want, k):
    # bf16/fp16 against fp32: rtol 2e-2, absolute floor for sums of k products of O(1) terms
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2 * float(np.sqrt(k)) * float(want.abs().mean() + 1e-3))


CASES = [
    ([128], 256, 256),
    ([1], 256, 256),
    ([100, 0, 0, 29], 256, 320),
    ([300, 0, 77], 512, 256),
    ([257, 511, 64, 128], 1024, 512),
    ([700, 900], 256, 1024),
    ([63, 65, 127, 129, 191, 193, 1, 0], 320, 576),
    ([0, 0, 0, 0], 256, 256),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("counts,fin,fout", CASES)
@pytest.mark.parametrize("bias", [True, False])
def test_tc_against_fp32(fc, dtype, counts, fin, fout, bias):
    torch.manual_seed(sum(counts) + fin + fout)
    E, B = len(counts), sum(counts)
    pad = 5  # rows past the last segment hold NaNs: they must never reach an output
    x = torch.full((B + pad, fin), float("nan"), device="cuda", dtype=dtype)
    gy = torch.full((B + pad, fout), float("nan"), device="cuda", dtype=dtype)
    x[:B] = torch.randn(B, fin, device="cuda").to(dtype)
    gy[:B] = torch.randn(B, fout, device="cuda").to(dtype)
    w = ((torch.rand(E, fout, fin, device="cuda") * 2 - 1) / np.sqrt(fin)).to(dtype)
    b = ((torch.rand(E, fout, device="cuda") * 2 - 1) / np.sqrt(fin)).to(dtype) if bias else None
    cnt = torch.tensor(counts, dtype=torch.int64)
    y = fc.linear_forward(x, cnt, w, b)
    gx, gw, gb = fc.linear_backward(gy, x, cnt, w, b)
    wy, wgx, wgw, wgb = reference(x[:B], counts, w, b, gy[:B])
    assert device_status() == 0
    if B:
        close(y[:B], wy, fin)
        close(gx[:B], wgx, fout)
    close(gw, wgw, max(max(counts), 1))
    close(gb, wgb, max(max(counts), 1))
    assert torch.isfinite(gw.float()).all() and torch.isfinite(gb.float()).all()


@pytest.mark.parametrize("act", ["relu", "gelu"])
def test_tc_fused_epilogues_match_ffma(fc, act, monkeypatch):
    """Bias + activation (forward) and activation backward (input gradient) in the tensor-core
    epilogues against the FFMA kernels, which apply the same formulas in fp32."""
    from fastermoe_b200 import _lib
    torch.manual_seed(1)
    counts, d, h = [300, 0, 157, 431], 256, 512
    E, B = len(counts), sum(counts)
    off = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int64, device="cuda")
    x = torch.randn(B, d, device="cuda").bfloat16()
    w1 = ((torch.rand(E, h, d, device="cuda") * 2 - 1) / np.sqrt(d)).bfloat16()
    b1 = ((torch.rand(E, h, device="cuda") * 2 - 1) / np.sqrt(d)).bfloat16()
    gh = torch.randn(B, h, device="cuda").bfloat16()
    code = {"relu": _lib.ACT_RELU, "gelu": _lib.ACT_GELU}[act]

    def both():
        # the derivative buffer is only written for GELU (ReLU's backward reads the output)
        y, pre = fc.linear_forward_act(x, off, w1, b1, code, want_pre=(act == "gelu"))
        if pre is None:
            pre = torch.zeros(1, device="cuda")
        # backward of a layer whose input came from an activation: a saved buffer of x's shape
        # (ReLU: the activation output, only its sign matters; GELU: the saved derivative)
        pre_in = torch.randn(B, d, device="cuda").bfloat16()
        torch.manual_seed(5)
        gx, gw, gb = fc.linear_backward_act(gh, x, off, w1, pre_in, code)
        return y, pre, gx, gw, gb

    torch.manual_seed(7)
    tc = both()
    monkeypatch.setenv("FMOE_B200_GEMM", "simt")
    torch.manual_seed(7)
    ff = both()
    monkeypatch.delenv("FMOE_B200_GEMM")
    for name, a, b_ in zip(["y", "pre", "gx", "gw", "gb"], tc, ff):
        torch.testing.assert_close(a.float(), b_.float(), rtol=2e-2, atol=2e-2, msg=lambda m, n=name: f"{n}: {m}")
    assert device_status() == 0


def test_tc_accumulate_weight_gradient(fc):
    from fastermoe_b200 import _lib
    torch.manual_seed(2)
    counts, d, h = [200, 312], 256, 256
    off = torch.tensor([0, 200, 512], dtype=torch.int64, device="cuda")
    x = torch.randn(512, d, device="cuda").bfloat16()
    gy = torch.randn(512, h, device="cuda").bfloat16()
    w = torch.randn(2, h, d, device="cuda").bfloat16()
    gw0 = torch.randn(2, h, d, device="cuda").bfloat16()
    gb0 = torch.randn(2, h, device="cuda").bfloat16()
    _, gw, gb = fc.linear_backward_act(gy, x, off, w, None, _lib.ACT_NONE, grad_w=gw0.clone(), grad_b=gb0.clone(),
                                       accumulate=True)
    _, _, wgw, wgb = reference(x, counts, w, None, gy)
    close(gw, wgw + gw0.float(), 312)
    close(gb, wgb + gb0.float(), 312)


def test_full_size_layer_shapes_properties(fc):
    """BASELINE config 2 sizes: linearity of the forward product and agreement of the weight
    gradient with the identity sum(dW * W) = sum(dY * (Y - bias))."""
    torch.manual_seed(3)
    E, d, h, B = 16, 1024, 4096, 32768
    counts = np.random.default_rng(0).multinomial(B, np.ones(E) / E)
    off = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int64, device="cuda")
    x = torch.randn(B, d, device="cuda").bfloat16()
    w = ((torch.rand(E, h, d, device="cuda") * 2 - 1) / np.sqrt(d)).bfloat16()
    from fastermoe_b200 import _lib
    y1, _ = fc.linear_forward_act(x, off, w, None, _lib.ACT_NONE)
    y2, _ = fc.linear_forward_act((2 * x.float()).bfloat16(), off, w, None, _lib.ACT_NONE)
    torch.testing.assert_close(y2.float(), 2 * y1.float(), rtol=1e-2, atol=1e-2)   # exact up to output rounding
    gy = torch.randn(B, h, device="cuda").bfloat16()
    gx, gw, _ = fc.linear_backward_act(gy, x, off, w, None, _lib.ACT_NONE, need_bias=False)
    lhs = (gw.float() * w.float()).sum()
    rhs = (gy.float() * y1.float()).sum()
    assert abs(float(lhs - rhs)) <= 2e-2 * abs(float(rhs)) + 50.0
    # <gx, x> equals the same bilinear form
    mid = (gx.float() * x.float()).sum()
    assert abs(float(mid - rhs)) <= 2e-2 * abs(float(rhs)) + 50.0
    assert device_status() == 0


@pytest.mark.parametrize("form", ["pair", "auto"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_cta_pair_kernels(fc, form, dtype, monkeypatch):
    """The cta_group::2 kernels (256-row tiles, one CTA pair per tile) against fp32 matmuls and,
    bit for bit, against the one-CTA kernels: both accumulate the same products in the same order.
    'pair' forces them for all three products; 'auto' is the default choice at a size where it
    picks pairs for the forward and input-gradient products."""
    from fastermoe_b200 import _lib
    torch.manual_seed(11)
    if form == "pair":
        counts, fin, fout = [2048 + 77, 300, 2600, 0, 1500, 255, 257], 512, 768
        monkeypatch.setenv("FMOE_B200_GEMM", "pair")
    else:
        counts, fin, fout = [9000, 12001, 8191, 10808], 256, 1024      # >= 512 rows per expert, >= 148 pair tiles
        monkeypatch.delenv("FMOE_B200_GEMM", raising=False)
    E, B = len(counts), sum(counts)
    off = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int64, device="cuda")
    x = torch.randn(B, fin, device="cuda").to(dtype)
    gy = torch.randn(B, fout, device="cuda").to(dtype)
    w = ((torch.rand(E, fout, fin, device="cuda") * 2 - 1) / np.sqrt(fin)).to(dtype)
    b = ((torch.rand(E, fout, device="cuda") * 2 - 1) / np.sqrt(fin)).to(dtype)

    def run():
        y, pre = fc.linear_forward_act(x, off, w, b, _lib.ACT_GELU, want_pre=True)
        y0, _ = fc.linear_forward_act(x, off, w, b, _lib.ACT_NONE)
        gx, gw, gb = fc.linear_backward_act(gy, x, off, w, None, _lib.ACT_NONE)
        return y, pre, y0, gx, gw, gb

    got = run()
    monkeypatch.setenv("FMOE_B200_GEMM", "tc1")
    single = run()
    monkeypatch.delenv("FMOE_B200_GEMM")
    assert device_status() == 0
    for name, a_, b_ in zip(["y", "pre", "y0", "gx", "gw", "gb"], got, single):
        assert torch.equal(a_, b_), f"{name}: CTA-pair and one-CTA kernels differ"
    wy, wgx, wgw, wgb = reference(x, counts, w, b, gy)
    close(got[2], wy, fin)
    close(got[3], wgx, fout)
    close(got[4], wgw, max(counts))
    close(got[5], wgb, max(counts))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("form", ["auto", "pair"])
def test_input_gradient_column_sums(fc, dtype, form, monkeypatch):
    """linear_backward_act(want_gx_colsum=True): per-expert column sums of the returned dX (the bias
    gradient of the layer below), from the tensor-core epilogue (16-bit) or the plain kernel (fp32)."""
    from fastermoe_b200 import _lib
    if form == "pair":
        if dtype == torch.float32:
            pytest.skip("fp32 takes the FFMA kernels")
        monkeypatch.setenv("FMOE_B200_GEMM", "pair")
        counts, fin, fout = [2048 + 77, 300, 2600, 0, 1500, 31, 33], 512, 256
    else:
        counts, fin, fout = [100, 0, 0, 29, 257, 32, 1, 511], 320, 256
    torch.manual_seed(5)
    E, B = len(counts), sum(counts)
    off = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int64, device="cuda")
    x = torch.randn(B, fin, device="cuda").to(dtype)
    gy = torch.randn(B, fout, device="cuda").to(dtype)
    w = ((torch.rand(E, fout, fin, device="cuda") * 2 - 1) / np.sqrt(fin)).to(dtype)
    saved = torch.rand(B, fin, device="cuda").to(dtype)          # stands for a saved GELU derivative
    for act_pre, act in ((None, _lib.ACT_NONE), (saved, _lib.ACT_GELU)):
        gx, gw, gb, cs = fc.linear_backward_act(gy, x, off, w, act_pre, act, want_gx_colsum=True)
        gx0, gw0, gb0 = fc.linear_backward_act(gy, x, off, w, act_pre, act)
        assert torch.equal(gx, gx0) and torch.equal(gw, gw0) and torch.equal(gb, gb0)
        want = torch.zeros(E, fin, device="cuda")
        p = 0
        for e, c in enumerate(counts):
            want[e] = gx[p:p + c].float().sum(0)
            p += c
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        torch.testing.assert_close(cs.float(), want, rtol=tol, atol=tol * float(want.abs().max() + 1))
    assert device_status() == 0
