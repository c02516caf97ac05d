r"""Generates tests/golden/reference_cpu.npz by running the reference's own Python code.

Run in the build container, where the reference checkout is mounted:

    python tests/golden/make_golden.py [/path/to/reference]

The reference package imports its CUDA extension at module load
(fmoe/functions.py:9); an in-memory stand-in named ``fmoe_cuda`` is installed
first.  The stand-in only implements what the *recorded* CPU code paths call:
``expert_count`` (a bincount) and ``expert_exchange`` (a prescribed all-gather
table), both needed by HirGate's call of count_by_gate.  Everything that is
recorded is computed by the reference's unmodified Python:

* NaiveGate.forward                      fmoe/gates/naive_gate.py:26-42
* BruteForceMoELinear.forward + autograd tests/moe.py:31-49
* _local_scatter / _local_gather         fmoe/functions.py:72-84
* _gen_policy -> _global_policy          fmoe/transformer.py:33-86
* HirGate.forward                        fmoe/gates/hir_gate.py:36-116
* NoisyGate.forward (+ its loss)         fmoe/gates/noisy_gate.py:108-144
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: first argument, else the directory `reference` beside this repository
REF = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")

stub = types.ModuleType("fmoe_cuda")
_fake_world = {}


def _expert_count(gate_idx, expert_count):
    g = gate_idx.reshape(-1)
    g = g[g >= 0]
    expert_count += torch.bincount(g, minlength=expert_count.numel()).to(expert_count.dtype)


def _expert_exchange(lec, n_expert, n_workers):
    aec = _fake_world["aec"].clone()
    aec[_fake_world["rank"]] = lec.view(n_workers, n_expert)
    agec = aec.transpose(0, 1).contiguous()
    return [aec, agec, agec[_fake_world["rank"]].reshape(-1)]


stub.expert_count = _expert_count
stub.expert_exchange = _expert_exchange
sys.modules["fmoe_cuda"] = stub
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, "tests"))

os.environ["FMOE_ENABLE_DYNREP"] = "1"
torch.set_num_threads(1)

from fmoe.gates.naive_gate import NaiveGate  # noqa: E402
from fmoe.gates.hir_gate import HirGate  # noqa: E402
from fmoe.functions import _local_scatter, _local_gather  # noqa: E402
from fmoe.transformer import _gen_policy  # noqa: E402
from moe import BruteForceMoELinear  # noqa: E402

out = {}


def uniform(shape, fan_in, g):
    b = 1.0 / np.sqrt(fan_in)
    return (torch.rand(shape, generator=g) * 2 - 1) * b


def layer_case(tag, T, d, h, E, k, act_name, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    act = {"gelu": torch.nn.functional.gelu, "relu": torch.relu}[act_name]
    gate = NaiveGate(d, E, 1, top_k=k)
    moe = BruteForceMoELinear(act, num_expert=E, d_model=d, d_hidden=h, world_size=1, top_k=k)
    with torch.no_grad():
        gate.gate.weight.copy_(uniform((E, d), d, g))
        gate.gate.bias.copy_(uniform((E,), d, g))
        moe.weight_htoh4.copy_(uniform((E, h, d), d, g))
        moe.bias_htoh4.copy_(uniform((E, h), d, g))
        moe.weight_h4toh.copy_(uniform((E, d, h), h, g))
        moe.bias_h4toh.copy_(uniform((E, d), h, g))
    gate, moe = gate.to(dtype), moe.to(dtype)
    x = torch.randn(T, d, generator=g).to(dtype).requires_grad_(True)
    idx, score = gate(x)
    y = moe(x, idx, score)
    y.sum().backward()
    rec = dict(x=x, gate_w=gate.gate.weight, gate_b=gate.gate.bias, w1=moe.weight_htoh4, b1=moe.bias_htoh4,
               w2=moe.weight_h4toh, b2=moe.bias_h4toh, idx=idx, score=score, out=y, grad_x=x.grad,
               grad_gate_w=gate.gate.weight.grad, grad_gate_b=gate.gate.bias.grad,
               grad_w1=moe.weight_htoh4.grad, grad_b1=moe.bias_htoh4.grad,
               grad_w2=moe.weight_h4toh.grad, grad_b2=moe.bias_h4toh.grad)
    for name, t in rec.items():
        out[f"{tag}/{name}"] = t.detach().numpy()
    out[f"{tag}/meta"] = np.array([T, d, h, E, k, {"gelu": 2, "relu": 1}[act_name], seed])


# Shapes of the reference's own numerical tests (tests/test_numerical.py:84-95) and a larger one.
layer_case("layer_e4_k2_gelu", 4, 16, 32, 4, 2, "gelu", 42)
layer_case("layer_e8_k3_gelu", 4, 16, 32, 8, 3, "gelu", 43)
layer_case("layer_e4_k2_relu", 64, 32, 64, 4, 2, "relu", 44)
layer_case("layer_e16_k2_gelu", 96, 32, 64, 16, 2, "gelu", 45)

# Local scatter / gather (torch index ops).
g = torch.Generator().manual_seed(7)
inp = torch.randn(12, 6, generator=g)
gate_idx = torch.randint(0, 5, (12, 2), generator=g) - 1  # -1 .. 3, as tests/test_local_exchange.py:20
keep = torch.nonzero(gate_idx.reshape(-1) >= 0).reshape(-1)
pos = keep[torch.argsort(gate_idx.reshape(-1)[keep], stable=True)]
buf = _local_scatter(inp, pos // 2)
back_copy = _local_gather(buf, pos, 24, maybe_overlap=False)
back_add = _local_gather(buf, pos // 2, 12, maybe_overlap=True)
for name, t in dict(inp=inp, gate_idx=gate_idx, pos=pos, buf=buf, back_copy=back_copy, back_add=back_add).items():
    out[f"local/{name}"] = t.numpy()


# Shadowing policy on seeded count tables.
def policy_case(tag, W, E, d_model, alpha, table):
    pol = _gen_policy(alpha)
    aec = torch.from_numpy(table).long()
    agec = aec.transpose(0, 1).contiguous()
    res = pol(aec, agec, E, W, d_model, True)
    out[f"policy/{tag}/aec"] = table
    out[f"policy/{tag}/res"] = res.numpy()
    out[f"policy/{tag}/meta"] = np.array([W, E, d_model, alpha], dtype=np.float64)


rng = np.random.default_rng(4)
W, E, T, k = 8, 2, 8192, 2
# c5-like: 40 % of all assignments to expert 0, rest uniform.
p = np.full(W * E, 0.6 / (W * E - 1))
p[0] = 0.4
tab = np.stack([rng.multinomial(T * k, p).reshape(W, E) for _ in range(W)]).astype(np.int64)
policy_case("skew40", W, E, 1024, 4.0, tab)
# uniform
tab = np.stack([rng.multinomial(T * k, np.full(W * E, 1 / (W * E))).reshape(W, E) for _ in range(W)]).astype(np.int64)
policy_case("uniform", W, E, 1024, 4.0, tab)
# Zipf(1.2) over 32 experts, 4 per worker.
E3 = 4
z = 1.0 / np.arange(1, W * E3 + 1) ** 1.2
z /= z.sum()
tab = np.stack([rng.multinomial(T * k, z).reshape(W, E3) for _ in range(W)]).astype(np.int64)
policy_case("zipf", W, E3, 2048, 4.0, tab)
# small world
tab = np.array([[[50], [2]], [[40], [4]]], dtype=np.int64)
policy_case("w2", 2, 1, 4, 2.0, tab)


# HirGate on one rank of an 8-rank world (2 nodes of 4), with and without the off-node limit biting.
def hir_case(tag, bias_to, seed, policy_on):
    W, E, d, T = 8, 2, 32, 256
    g = torch.Generator().manual_seed(seed)
    rank = 1
    gate = HirGate(d, E, W, node_rank=rank // 4)
    with torch.no_grad():
        gate.gate.weight.copy_(torch.randn(W * E, d, generator=g) * 0.1)
        b = torch.zeros(W * E)
        if bias_to is not None:
            b[bias_to] = 1.0
        gate.gate.bias.copy_(b)
    os.environ["FMOE_ENABLE_DYNREP"] = "1" if policy_on else "0"
    gate.policy_fn = _gen_policy(4.0)
    os.environ["FMOE_ENABLE_DYNREP"] = "1"
    x = torch.randn(T, d, generator=g)
    _fake_world["rank"] = rank
    _fake_world["aec"] = torch.from_numpy(
        np.random.default_rng(seed).multinomial(T * 2, np.full(W * E, 1 / (W * E)), size=W).reshape(W, W, E)).long()
    idx, score = gate(x)
    for name, t in dict(x=x, gate_w=gate.gate.weight, gate_b=gate.gate.bias, aec=_fake_world["aec"], idx=idx,
                        score=score).items():
        out[f"hir/{tag}/{name}"] = t.detach().numpy()
    out[f"hir/{tag}/meta"] = np.array([W, E, d, T, rank, int(policy_on)])


hir_case("few_leaving", 2, 11, False)      # bias towards an on-node expert -> plain top-2
hir_case("many_leaving", 12, 12, False)    # bias towards an off-node expert -> limited
hir_case("uniform", None, 13, True)

# NoisyGate in training mode with a recorded noise sample (fmoe/gates/noisy_gate.py:108-144).
def noisy_case(tag, T, d, E, k, seed):
    from fmoe.gates.noisy_gate import NoisyGate
    g = torch.Generator().manual_seed(seed)
    gate = NoisyGate(d, E, 1, top_k=k)
    with torch.no_grad():
        gate.w_gate.copy_(torch.randn(d, E, generator=g) * 0.3)
        gate.w_noise.copy_(torch.randn(d, E, generator=g) * 0.3)
    gate.train()
    x = torch.randn(T, d, generator=g).requires_grad_(True)
    noise = torch.randn(T, E, generator=g)
    real = torch.randn_like
    torch.randn_like = lambda t, *a, **kw: noise.clone()
    try:
        idx, score = gate(x)
    finally:
        torch.randn_like = real
    loss = gate.get_loss()
    (score.sum() * 0.5 + loss).backward()
    for name, t in dict(x=x, w_gate=gate.w_gate, w_noise=gate.w_noise, noise=noise, idx=idx, score=score, loss=loss,
                        grad_x=x.grad, grad_w_gate=gate.w_gate.grad, grad_w_noise=gate.w_noise.grad).items():
        out[f"noisy/{tag}/{name}"] = t.detach().numpy()
    out[f"noisy/{tag}/meta"] = np.array([T, d, E, k])


noisy_case("e8_k2", 64, 16, 8, 2, 21)
noisy_case("e4_k3", 32, 8, 4, 3, 22)
noisy_case("e2_k2", 16, 8, 2, 2, 23)        # top_k == number of experts: the load is the count of non-zero gates

np.savez_compressed(os.path.join(HERE, "reference_cpu.npz"), **out)
print("wrote", len(out), "arrays")
