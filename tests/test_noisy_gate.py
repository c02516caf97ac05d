"""NoisyGate against outputs recorded from the reference's own NoisyGate in training mode with a
prescribed noise sample (tests/golden/make_golden.py): indices exact, scores, loss and gradients to
fp32 accuracy.  Runs on the CPU (torch ops only) and, marked gpu, on the device (library top-k)."""
import numpy as np
import pytest
import torch

CASES = ["e8_k2", "e4_k3", "e2_k2"]


def run_case(golden, tag, device):
    from fastermoe_b200.gates import NoisyGate
    z = {k.split("/", 2)[2]: torch.from_numpy(golden[k]) for k in golden.files if k.startswith(f"noisy/{tag}/")}
    T, d, E, k = (int(v) for v in z["meta"].tolist())
    gate = NoisyGate(d, E, 1, top_k=k)
    with torch.no_grad():
        gate.w_gate.copy_(z["w_gate"])
        gate.w_noise.copy_(z["w_noise"])
    gate = gate.to(device).train()
    x = z["x"].to(device).requires_grad_(True)
    idx, score = gate(x, noise=z["noise"].to(device))
    loss = gate.get_loss()
    (score.sum() * 0.5 + loss).backward()
    assert idx.shape == (T * k,) and score.shape == (T, 1, k)
    assert np.array_equal(idx.cpu().numpy(), z["idx"].numpy())
    tol = dict(rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(score.detach().cpu(), z["score"], **tol)
    torch.testing.assert_close(loss.detach().cpu().reshape(-1), z["loss"].reshape(-1), rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(x.grad.cpu(), z["grad_x"], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gate.w_gate.grad.cpu(), z["grad_w_gate"], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gate.w_noise.grad.cpu(), z["grad_w_noise"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("tag", CASES)
def test_noisy_gate_cpu(golden, tag):
    run_case(golden, tag, "cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("tag", CASES)
def test_noisy_gate_gpu(golden, tag):
    run_case(golden, tag, "cuda")


def test_noisy_gate_eval_mode_is_noise_free():
    from fastermoe_b200.gates import NoisyGate
    torch.manual_seed(0)
    gate = NoisyGate(8, 4, 1, top_k=2).eval()
    x = torch.randn(10, 8)
    a, _ = gate(x)
    b, _ = gate(x)
    assert torch.equal(a, b)
    assert torch.equal(a.view(10, 2), torch.topk(x @ gate.w_gate, 2)[1])
