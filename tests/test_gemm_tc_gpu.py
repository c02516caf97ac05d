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


@pytest.fixture(autouse=True)
def _default_form(fc):
    """Every test starts and ends with the library's own choice of GEMM kernels."""
    fc.set_gemm_form("auto")
    yield
    fc.set_gemm_form("auto")


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


def close(got, want):
    """16-bit result against the fp32 product of the same 16-bit inputs.  Accumulation is fp32 on both
    sides, so what separates them is one rounding of the output: relative 2^-9 for bf16.  rtol 2e-2 is
    the bound the layer is specified to; the absolute floor (four such roundings of a typical element)
    only covers entries that cancel to almost nothing."""
    want = want.float()
    rms = float(want.pow(2).mean().sqrt()) if want.numel() else 0.0
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=4 * 2.0 ** -9 * rms)


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
        close(y[:B], wy)
        close(gx[:B], wgx)
    close(gw, wgw)
    close(gb, wgb)
    assert torch.isfinite(gw.float()).all() and torch.isfinite(gb.float()).all()


@pytest.mark.parametrize("act", ["relu", "gelu"])
def test_tc_fused_epilogues_match_ffma(fc, act):
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
    fc.set_gemm_form("simt")
    torch.manual_seed(7)
    ff = both()
    fc.set_gemm_form("auto")
    for name, a, b_ in zip(["y", "pre", "gx", "gw", "gb"], tc, ff):
        # both sides round to bf16: they may differ by one unit in the last place of either
        rms = float(b_.float().pow(2).mean().sqrt())
        torch.testing.assert_close(a.float(), b_.float(), rtol=2e-2, atol=8 * 2.0 ** -9 * rms, msg=lambda m, n=name: f"{n}: {m}")
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
    close(gw, wgw + gw0.float())
    close(gb, wgb + gb0.float())


def test_benchmark_shapes_against_fp32(fc):
    """All six products of the benchmark layer (16384 tokens x top-2 = 32768 rows over 16 experts,
    d_model 1024, d_hidden 4096, bf16; the sizes at which the library picks the CTA-pair kernels)
    against fp32 matmuls of the same bf16 inputs, including the fused bias + GELU epilogue, the
    saved-derivative input gradient and the column sums that give the first layer's bias gradient."""
    from fastermoe_b200 import _lib
    torch.manual_seed(3)
    E, d, h, B = 16, 1024, 4096, 32768
    counts = np.random.default_rng(0).multinomial(B, np.ones(E) / E)
    off = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int64, device="cuda")
    bf = torch.bfloat16
    x = torch.randn(B, d, device="cuda").to(bf)
    w1 = ((torch.rand(E, h, d, device="cuda") * 2 - 1) / np.sqrt(d)).to(bf)
    b1 = ((torch.rand(E, h, device="cuda") * 2 - 1) / np.sqrt(d)).to(bf)
    w2 = ((torch.rand(E, d, h, device="cuda") * 2 - 1) / np.sqrt(h)).to(bf)
    b2 = ((torch.rand(E, d, device="cuda") * 2 - 1) / np.sqrt(h)).to(bf)
    gy = torch.randn(B, d, device="cuda").to(bf)
    hid, deriv = fc.linear_forward_act(x, off, w1, b1, _lib.ACT_GELU, want_pre=True)         # product 1
    y, _ = fc.linear_forward_act(hid, off, w2, b2, _lib.ACT_NONE)                            # product 2
    gh, gw2, gb2, gb1 = fc.linear_backward_act(gy, hid, off, w2, deriv, _lib.ACT_GELU,       # products 3, 4
                                               want_gx_colsum=True)
    gx, gw1, _ = fc.linear_backward_act(gh, x, off, w1, None, _lib.ACT_NONE, need_bias=False)  # products 5, 6
    assert device_status() == 0
    p = 0
    for e, c in enumerate(counts):
        sl = slice(p, p + int(c))
        p += int(c)
        xe, ge = x[sl].float(), gy[sl].float()
        pre = xe @ w1[e].float().t() + b1[e].float()
        close(hid[sl], torch.nn.functional.gelu(pre))
        cdf = 0.5 * (1 + torch.erf(pre * 0.7071067811865476))
        want_deriv = cdf + pre * torch.exp(-0.5 * pre * pre) * 0.3989422804014327
        close(deriv[sl], want_deriv)
        # from here on every product is checked against fp32 math on the kernel's own 16-bit inputs
        he = hid[sl].float()
        close(y[sl], he @ w2[e].float().t() + b2[e].float())
        close(gh[sl], (ge @ w2[e].float()) * deriv[sl].float())
        close(gw2[e], ge.t() @ he)
        close(gb2[e], ge.sum(0))
        ghe = gh[sl].float()
        close(gb1[e], ghe.sum(0))
        close(gx[sl], ghe @ w1[e].float())
        close(gw1[e], ghe.t() @ xe)


def test_offsets_beyond_the_buffer_are_clamped(fc):
    """Segment offsets that live on the device are not seen by the host.  When they overshoot the
    buffers (or run backwards) the kernels clamp them: nothing is read or written past the rows
    given, rows past the clamped end keep their old contents, and status code 8 is raised."""
    from fastermoe_b200 import _lib
    torch.manual_seed(9)
    fin, fout, rows = 256, 512, 700
    for dtype in (torch.bfloat16, torch.float32):
        # counts claim 300 + 900 rows, the buffers hold 700 followed by poisoned padding
        off = torch.tensor([0, 300, 1200], dtype=torch.int64, device="cuda")
        x = torch.full((rows + 600, fin), float("nan"), device="cuda", dtype=dtype)
        gy = torch.full((rows + 600, fout), float("nan"), device="cuda", dtype=dtype)
        x[:rows] = torch.randn(rows, fin, device="cuda").to(dtype)
        gy[:rows] = torch.randn(rows, fout, device="cuda").to(dtype)
        w = ((torch.rand(2, fout, fin, device="cuda") * 2 - 1) / np.sqrt(fin)).to(dtype)
        y = torch.full((rows + 600, fout), 7.0, device="cuda", dtype=dtype)
        gx = torch.full((rows + 600, fin), 7.0, device="cuda", dtype=dtype)
        gw = torch.empty_like(w)
        gb = torch.empty(2, fout, device="cuda", dtype=dtype)
        code = _lib.BF16 if dtype == torch.bfloat16 else _lib.F32
        st = fc._stream()
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        # the library is told the truth about the buffers (700 rows); only the offsets lie
        assert _lib.lib.fmoe_linear_forward(P(x), P(w), None, P(off), P(y), None, rows, fin, fout, 2, code, 0, st) == 0
        scratch = torch.empty(_lib.lib.fmoe_linear_scratch_bytes(rows, fin, fout, 2, code) + 16, dtype=torch.uint8, device="cuda")
        assert _lib.lib.fmoe_linear_backward(P(gy), P(x), P(w), P(off), None, P(gx), P(gw), P(gb), rows, fin, fout, 2,
                                             code, 0, 0, P(scratch), st) == 0
        torch.cuda.synchronize()
        assert (y[rows:] == 7).all() and (gx[rows:] == 7).all(), "rows past the buffer were written"
        wy, wgx, wgw, wgb = reference(x[:rows], [300, 400], w, None, gy[:rows])
        tol = close if dtype == torch.bfloat16 else (lambda a, b: torch.testing.assert_close(a.float(), b, rtol=1e-4, atol=1e-4))
        tol(y[:rows], wy); tol(gx[:rows], wgx); tol(gw, wgw); tol(gb, wgb)
        if dtype == torch.bfloat16:
            assert device_status() == 8
            assert _lib.lib.fmoe_device_status_clear() == 0
    # the reference-named operators take counts on the host and refuse a mismatch before launching
    with pytest.raises(RuntimeError, match="rows"):
        fc.linear_forward(x[:rows].contiguous(), torch.tensor([300, 900]), w)
    assert device_status() == 0


@pytest.mark.parametrize("form", ["pair", "auto"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_cta_pair_kernels(fc, form, dtype):
    """The cta_group::2 kernels (256-row tiles, one CTA pair per tile) against fp32 matmuls and,
    bit for bit, against the one-CTA kernels: both accumulate the same products in the same order.
    'pair' forces them for all three products; 'auto' is the default choice at a size where it
    picks pairs for the forward and input-gradient products."""
    from fastermoe_b200 import _lib
    torch.manual_seed(11)
    if form == "pair":
        counts, fin, fout = [2048 + 77, 300, 2600, 0, 1500, 255, 257], 512, 768
        fc.set_gemm_form("pair")
    else:
        counts, fin, fout = [9000, 12001, 8191, 10808], 256, 1024      # >= 512 rows per expert, >= 148 pair tiles
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
    fc.set_gemm_form("tc1")
    single = run()
    fc.set_gemm_form("auto")
    assert device_status() == 0
    for name, a_, b_ in zip(["y", "pre", "y0", "gx", "gw", "gb"], got, single):
        assert torch.equal(a_, b_), f"{name}: CTA-pair and one-CTA kernels differ"
    wy, wgx, wgw, wgb = reference(x, counts, w, b, gy)
    close(got[2], wy)
    close(got[3], wgx)
    close(got[4], wgw)
    close(got[5], wgb)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("form", ["auto", "pair"])
def test_input_gradient_column_sums(fc, dtype, form):
    """linear_backward_act(want_gx_colsum=True): per-expert column sums of the returned dX (the bias
    gradient of the layer below), from the tensor-core epilogue (16-bit) or the plain kernel (fp32)."""
    from fastermoe_b200 import _lib
    if form == "pair":
        if dtype == torch.float32:
            pytest.skip("fp32 takes the FFMA kernels")
        fc.set_gemm_form("pair")
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
        # fp32 sums of the kernel's own (rounded) dX, rounded once to the output type
        rms = float(want.pow(2).mean().sqrt())
        if dtype == torch.float32:
            torch.testing.assert_close(cs.float(), want, rtol=1e-5, atol=1e-5 * rms)
        else:
            torch.testing.assert_close(cs.float(), want, rtol=2e-2, atol=4 * 2.0 ** -9 * rms)
    assert device_status() == 0
