"""A whole forward+backward step of the layer replayed as one CUDA graph equals the eager step,
also when the routing of the replayed input differs from the captured one."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def make_layer(dtype):
    from fastermoe_b200 import FMoETransformerMLP
    torch.manual_seed(0)
    m = FMoETransformerMLP(num_expert=4, d_model=256, d_hidden=512, top_k=2, activation=torch.nn.GELU())
    with torch.no_grad():
        m.gate.gate.weight.normal_(0, 0.5)
        for lin in (m.experts.htoh4, m.experts.h4toh):
            lin.weight.normal_(0, 0.05)
            lin.bias.normal_(0, 0.05)
    return m.to(dtype).cuda()


def eager_step(m, x):
    m.zero_grad(set_to_none=True)
    xi = x.clone().requires_grad_(True)
    out = m(xi)
    loss = out.sum(dtype=torch.float32)
    loss.backward()
    return out.detach().clone(), loss.detach().clone(), xi.grad.clone(), {n: p.grad.clone() for n, p in m.named_parameters()}


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_graphed_step_equals_eager(dtype):
    from fastermoe_b200 import GraphedStep
    m = make_layer(dtype)
    g = torch.Generator().manual_seed(1)
    xs = [torch.randn(1000, 256, generator=g).to(dtype).cuda() for _ in range(3)]
    want = [eager_step(m, x) for x in xs[1:]]
    step = GraphedStep(m, xs[0], input_grad=True)
    for x, (out, loss, gx, grads) in zip(xs[1:], want):
        got_loss = step(x)
        torch.cuda.synchronize()
        assert torch.equal(step.output, out) and torch.equal(got_loss, loss)
        assert torch.equal(step.input_grad, gx)
        for n, p in m.named_parameters():
            assert torch.equal(p.grad, grads[n]), n
    # a pinned host tensor is accepted as input
    host = xs[2].cpu().pin_memory()
    assert torch.equal(step(host), want[1][1])
