"""FMoETransformerMLP forward+backward against the reference's recorded outputs and the oracle."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from parity import assert_half_close

pytestmark = pytest.mark.gpu
LAYER_CASES = ["layer_e4_k2_gelu", "layer_e8_k3_gelu", "layer_e4_k2_relu", "layer_e16_k2_gelu"]


def build_layer(E, d, h, k, act, tensors, dtype=torch.float32, bias=True, softmax_scores=False):
    from fastermoe_b200 import FMoETransformerMLP
    fn = {"gelu": torch.nn.GELU(), "relu": torch.nn.ReLU()}[act]
    m = FMoETransformerMLP(num_expert=E, d_model=d, d_hidden=h, world_size=1, activation=fn, top_k=k, bias=bias)
    m.gate.softmax_scores = softmax_scores
    with torch.no_grad():
        m.gate.gate.weight.copy_(tensors["gate_w"])
        m.gate.gate.bias.copy_(tensors["gate_b"])
        m.experts.htoh4.weight.copy_(tensors["w1"])
        m.experts.h4toh.weight.copy_(tensors["w2"])
        if bias:
            m.experts.htoh4.bias.copy_(tensors["b1"])
            m.experts.h4toh.bias.copy_(tensors["b2"])
    return m.to(dtype).cuda()


def grads_of(m, x):
    return {"x": x.grad, "gate_w": m.gate.gate.weight.grad, "gate_b": m.gate.gate.bias.grad,
            "w1": m.experts.htoh4.weight.grad, "b1": m.experts.htoh4.bias.grad,
            "w2": m.experts.h4toh.weight.grad, "b2": m.experts.h4toh.bias.grad}


@pytest.mark.parametrize("tag", LAYER_CASES)
def test_layer_matches_reference_golden(golden, tag):
    z = {k.split("/", 1)[1]: torch.from_numpy(golden[k]) for k in golden.files if k.startswith(tag + "/")}
    T, d, h, E, k, act, seed = z["meta"].tolist()
    act = {2: "gelu", 1: "relu"}[act]
    m = build_layer(E, d, h, k, act, z)
    x = z["x"].cuda().requires_grad_(True)
    out = m(x)
    out.sum().backward()
    # fp32: rtol 1e-5 (absolute floor for sums of O(d_hidden) terms)
    tol = dict(rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(out.cpu(), z["out"], **tol)
    for name, g in grads_of(m, x).items():
        torch.testing.assert_close(g.cpu(), z["grad_" + name], **tol, msg=lambda s, n=name: f"{n}: {s}")


def test_state_dict_keys_match_reference_names():
    m = build_layer(2, 8, 16, 2, "gelu", O.make_layer_inputs(4, 8, 16, 2, 0))
    assert set(m.state_dict()) == {"gate.gate.weight", "gate.gate.bias", "experts.htoh4.weight",
                                   "experts.htoh4.bias", "experts.h4toh.weight", "experts.h4toh.bias"}


def test_cpu_baseline_config_fp32():
    """The CPU-runnable workload: 2048 tokens, d 512, h 2048, 4 experts, top-2, fp32, GELU, seed 0."""
    T, d, h, E, k = 2048, 512, 2048, 4, 2
    tens = O.make_layer_inputs(T, d, h, E, seed=0)
    want = O.moe_layer_fwd_bwd(tens["x"], tens["gate_w"], tens["gate_b"], tens["w1"], tens["b1"], tens["w2"],
                               tens["b2"], k, act="gelu")
    m = build_layer(E, d, h, k, "gelu", tens)
    x = tens["x"].cuda().requires_grad_(True)
    out = m(x)
    out.sum().backward()
    tol = dict(rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(out.cpu(), want["out"], **tol)
    got = grads_of(m, x)
    for name in ("x", "b1", "b2"):
        torch.testing.assert_close(got[name].cpu(), want["grad_" + name], **tol, msg=lambda s, n=name: f"{n}: {s}")
    # gradients that sum over ~1000-4000 tokens: fp32 summation order differs, so the absolute
    # floor scales with the size of the result (2e-5 of its largest entry)
    for name in ("w1", "w2", "gate_w", "gate_b"):
        w_ = want["grad_" + name]
        torch.testing.assert_close(got[name].cpu(), w_, rtol=1e-5, atol=2e-5 * float(w_.abs().max()),
                                   msg=lambda s, n=name: f"{n}: {s}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("softmax_scores", [False, True])
def test_bf16_layer_against_fp32_oracle(dtype, softmax_scores):
    """The benchmark layer scaled down (bf16, near-uniform routing): rtol 2e-2 against fp32."""
    T, d, h, E, k = 1024, 256, 1024, 16, 2
    tens = O.make_layer_inputs(T, d, h, E, seed=1, gate_std=0.02)
    m = build_layer(E, d, h, k, "gelu", tens, dtype=dtype, softmax_scores=softmax_scores)
    x = tens["x"].to(dtype).cuda().requires_grad_(True)
    # the oracle sees the same rounded parameters and the gate decisions of the device run
    with torch.no_grad():
        idx, _ = m.gate(x)
    r = {n: (t.to(dtype).float() if t is not None else None) for n, t in tens.items()}
    want = O.moe_layer_fwd_bwd(r["x"], r["gate_w"], r["gate_b"], r["w1"], r["b1"], r["w2"], r["b2"], k, act="gelu",
                               softmax_scores=softmax_scores, gate_idx=idx.cpu())
    out = m(x)
    out.sum().backward()
    # 16-bit tensors stored between the inputs and each result: hidden, expert output, gate score,
    # combined output (forward); their gradients on the way back
    assert_half_close(out, want["out"], 4, "out")
    got = grads_of(m, x)
    for name, n in (("x", 5), ("b1", 4), ("b2", 2), ("w1", 4), ("w2", 3)):
        assert_half_close(got[name], want["grad_" + name], n, name)


def test_benchmark_layer_against_cpu_oracle():
    """The benchmark's layer at full size (16384 tokens, d_model 1024, d_hidden 4096, 16 experts, top-2,
    bf16, near-uniform gate) against the fp32 CPU oracle given the same bf16-rounded tensors and the
    device's gate decisions."""
    T, d, h, E, k = 16384, 1024, 4096, 16, 2
    tens = O.make_layer_inputs(T, d, h, E, seed=1, gate_std=0.02)
    m = build_layer(E, d, h, k, "gelu", tens, dtype=torch.bfloat16)
    x = tens["x"].bfloat16().cuda().requires_grad_(True)
    with torch.no_grad():
        idx, _ = m.gate(x)
    r = {n: (t.bfloat16().float() if t is not None else None) for n, t in tens.items()}
    torch.set_num_threads(max(torch.get_num_threads(), 1))
    want = O.moe_layer_fwd_bwd(r["x"], r["gate_w"], r["gate_b"], r["w1"], r["b1"], r["w2"], r["b2"], k, act="gelu",
                               gate_idx=idx.cpu())
    out = m(x)
    out.sum().backward()
    assert_half_close(out, want["out"], 4, "out")
    got = grads_of(m, x)
    for name, n in (("x", 5), ("b1", 4), ("b2", 2), ("w1", 4), ("w2", 3)):
        assert_half_close(got[name], want["grad_" + name], n, name)
    from fastermoe_b200 import fmoe_cuda
    assert fmoe_cuda.device_status() == 0


def test_pruned_tokens_give_zero_rows():
    """Gate entries set to -1 (capacity pruning) contribute nothing (fmoe/functions.py:77-84)."""
    from fastermoe_b200.gates import NaiveGate

    class DropGate(NaiveGate):
        def forward(self, inp):
            idx, val = super().forward(inp)
            idx = idx.clone()
            idx[::3, 1] = -1
            idx[5] = -1
            return idx, val

    from fastermoe_b200 import FMoETransformerMLP
    T, d, h, E, k = 96, 32, 64, 4, 2
    tens = O.make_layer_inputs(T, d, h, E, seed=9)
    m = FMoETransformerMLP(num_expert=E, d_model=d, d_hidden=h, top_k=k, gate=DropGate)
    with torch.no_grad():
        m.gate.gate.weight.copy_(tens["gate_w"]); m.gate.gate.bias.copy_(tens["gate_b"])
        m.experts.htoh4.weight.copy_(tens["w1"]); m.experts.htoh4.bias.copy_(tens["b1"])
        m.experts.h4toh.weight.copy_(tens["w2"]); m.experts.h4toh.bias.copy_(tens["b2"])
    m = m.cuda()
    x = tens["x"].cuda().requires_grad_(True)
    idx, _ = m.gate(x)
    out = m(x)
    out.sum().backward()
    want = O.moe_layer_fwd_bwd(tens["x"], tens["gate_w"], tens["gate_b"], tens["w1"], tens["b1"], tens["w2"],
                               tens["b2"], k, gate_idx=idx.cpu())
    tol = dict(rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(out.cpu(), want["out"], **tol)
    torch.testing.assert_close(x.grad.cpu(), want["grad_x"], **tol)
    torch.testing.assert_close(m.experts.htoh4.weight.grad.cpu(), want["grad_w1"], **tol)
    assert out[5].abs().sum() == 0


def test_reference_style_operator_sequence(golden):
    """The reference's own op sequence (count_by_gate -> MOEScatter -> MOELinear x2 -> MOEGather -> bmm)."""
    from fastermoe_b200.functions import count_by_gate, MOEScatter, MOEGather, MOELinear
    z = {k.split("/", 1)[1]: torch.from_numpy(golden[k]) for k in golden.files if k.startswith("layer_e4_k2_relu/")}
    T, d, h, E, k = z["meta"].tolist()[:5]
    x = z["x"].cuda()
    idx = z["idx"].cuda()
    pos, lec, aec, gec, agec = count_by_gate(idx, E, 1)
    assert pos.numel() == T * k
    lec_c, gec_c = lec.cpu(), gec.cpu()
    stored = torch.zeros(E, dtype=torch.bool)
    buf = MOEScatter.apply(x, pos // k, lec_c, gec_c, stored, T * k, 1)
    hmid = torch.relu(MOELinear.apply(buf, gec_c, z["w1"].cuda(), z["b1"].cuda()))
    y = MOELinear.apply(hmid, gec_c, z["w2"].cuda(), z["b2"].cuda())
    full = MOEGather.apply(y, pos, lec_c, gec_c, stored, T * k, 1)
    out = torch.bmm(z["score"].cuda().view(T, 1, k), full.view(T, k, d)).reshape(T, d)
    torch.testing.assert_close(out.cpu(), z["out"], rtol=1e-5, atol=2e-5)
