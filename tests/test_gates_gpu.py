"""Gate modules on one GPU: HirGate against outputs recorded from the reference's own HirGate
(tests/golden/make_golden.py), GShardGate / SwitchGate against the invariants the reference's
tests state (tests/test_gates.py:44-64, 84-115) and against the oracle's capacity pipeline."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tag", ["few_leaving", "many_leaving", "uniform"])
def test_hir_gate_module_matches_reference_golden(golden, tag, monkeypatch):
    """The recorded run was one rank of an 8-rank world whose count table was prescribed; the same
    table is prescribed here in place of the NCCL all-gather, everything else is the module's own
    path (count kernel, policy, top-k kernels)."""
    import fastermoe_b200.functions as F
    from fastermoe_b200.gates import HirGate
    from fastermoe_b200.transformer import _gen_policy
    z = {k.split("/", 2)[2]: golden[k] for k in golden.files if k.startswith(f"hir/{tag}/")}
    W, E, d, T, rank, policy_on = (int(v) for v in z["meta"].tolist())
    table = torch.from_numpy(z["aec"]).long().cuda()

    def prescribed_exchange(lec, n_expert, n_workers):
        aec = table.clone()
        aec[rank] = lec.view(n_workers, n_expert)
        agec = aec.transpose(0, 1).contiguous()
        return [aec, agec, agec[rank].reshape(-1)]

    monkeypatch.setattr(F.fmoe_cuda, "expert_exchange", prescribed_exchange)
    monkeypatch.setenv("FMOE_ENABLE_DYNREP", "1" if policy_on else "0")
    gate = HirGate(d, E, W, node_rank=rank // 4)
    gate.policy_fn = _gen_policy(4.0, constants="reference")
    with torch.no_grad():
        gate.gate.weight.copy_(torch.from_numpy(z["gate_w"]))
        gate.gate.bias.copy_(torch.from_numpy(z["gate_b"]))
    gate = gate.cuda()
    idx, score = gate(torch.from_numpy(z["x"]).cuda())
    assert np.array_equal(idx.cpu().numpy(), z["idx"])
    np.testing.assert_allclose(score.detach().cpu().numpy(), z["score"], rtol=1e-5, atol=1e-6)
    assert gate.get_loss() is not None
    # and the oracle's restatement gives the same answer for the same policy decision
    stored = np.zeros(W * E, dtype=bool)
    if policy_on:
        aec = z["aec"].copy()
        idx0 = torch.topk(torch.nn.functional.linear(*(torch.from_numpy(z[n]) for n in ("x", "gate_w", "gate_b"))), 2)[1]
        aec[rank] = O.expert_count(idx0.numpy(), W * E).reshape(W, E)
        stored = np.repeat(O.global_policy(aec, aec.transpose(1, 0, 2), E, W, d, True, 4.0).any(1), E)
    o_idx, _ = O.hir_gate(torch.from_numpy(z["x"]), torch.from_numpy(z["gate_w"]), torch.from_numpy(z["gate_b"]), E, W,
                          rank // 4, stored)
    assert np.array_equal(idx.cpu().numpy(), o_idx.numpy())


def test_gen_hir_gate_factory():
    from fastermoe_b200.gates import gen_hir_gate
    gate = gen_hir_gate(rank=5, workers_per_node=4)(16, 2, 8)
    assert gate.node_rank == 1 and gate.ne_per_node == 8 and gate.top_k == 2
    assert gate.mask.tolist() == [False] * 8 + [True] * 8


def _counts(idx, n):
    flat = idx.reshape(-1)
    return torch.bincount(flat[flat >= 0], minlength=n)


@pytest.mark.parametrize("n_expert", [2, 4, 16])
@pytest.mark.parametrize("cap", [0.1, 1.1])
@pytest.mark.parametrize("random_routing", [False, True])
def test_gshard_gate(n_expert, cap, random_routing):
    from fastermoe_b200.gates import GShardGate
    torch.manual_seed(3)
    d_model, batch = 256, 64
    gate = GShardGate(d_model, n_expert, 1, capacity=(cap, cap), random_routing=random_routing).cuda()
    x = torch.rand(batch, d_model, device="cuda")
    idx, val = gate(x)
    real_cap = math.ceil(cap * batch)
    assert int(_counts(idx, n_expert).max()) <= real_cap
    # the returned score of every kept entry is the gate's logit of that expert
    logits = gate.gate(x)
    kept = idx >= 0
    assert torch.equal(val[kept], torch.gather(logits, 1, idx.clamp(min=0))[kept])
    assert gate.get_loss() is not None
    if not random_routing:
        # which entries survive: the lowest flat indices per expert, as the oracle's pipeline prunes
        raw = torch.topk(logits, 2, dim=-1)[1]
        want = O.limit_by_capacity_gate([raw.cpu().numpy()], n_expert, 1, real_cap)[0][2]
        assert np.array_equal(idx.cpu().numpy(), want)
    else:
        # random routing only ever drops second choices
        raw = torch.topk(logits, 2, dim=-1)[1]
        want = torch.from_numpy(O.limit_by_capacity_gate([raw.cpu().numpy()], n_expert, 1, real_cap)[0][2]).cuda()
        assert torch.equal(idx[:, 0], want[:, 0])
        assert bool(((idx[:, 1] == want[:, 1]) | (idx[:, 1] == -1)).all())


@pytest.mark.parametrize("n_expert", [1, 16])
@pytest.mark.parametrize("cap", [0.1, 0.8])
@pytest.mark.parametrize("training", [True, False])
def test_switch_gate(n_expert, cap, training):
    from fastermoe_b200.gates import SwitchGate
    torch.manual_seed(4)
    d_model, batch = 128, 4096
    gate = SwitchGate(d_model, n_expert, 1, capacity=(cap, cap)).cuda()
    gate.train(training)
    x = torch.rand(batch, d_model, device="cuda")
    rng = torch.cuda.get_rng_state()
    idx, val = gate(x)
    assert idx.shape[0] == batch and val.shape[0] == batch
    real_cap = math.ceil(cap * batch)
    assert int(_counts(idx, n_expert).max()) <= real_cap
    score = gate.gate(x)
    if training:
        torch.cuda.set_rng_state(rng)       # the same noise as inside the gate
        noise = torch.rand_like(score)
        score = score + (noise * 2 * gate.switch_eps + 1.0 - gate.switch_eps)
    score = torch.softmax(score.float(), dim=-1)
    kept = idx.reshape(-1) >= 0
    want = torch.gather(score, 1, idx.reshape(-1, 1).clamp(min=0)).reshape(-1)
    assert torch.equal(val.reshape(-1)[kept].float(), want[kept].to(val.dtype).float())
    loss = gate.get_loss()
    assert loss is not None and torch.isfinite(loss)


def test_prepare_forward_matches_oracle():
    """prepare_forward's return tuple (fmoe/functions.py:45-69) at world_size 1."""
    from fastermoe_b200.functions import prepare_forward
    rng = np.random.default_rng(5)
    E = 6
    gate = rng.integers(-1, E, size=(300, 2))
    pos, lec, gec, aec, agec, fwd = prepare_forward(torch.from_numpy(gate).cuda(), E, 1)
    cnt = O.expert_count(gate, E)
    assert np.array_equal(pos.cpu().numpy(), O.assign_pos(gate, E))
    for t in (lec, gec, aec, agec, fwd):
        assert not t.is_cuda and np.array_equal(t.numpy().reshape(-1), cnt)


def test_masked_layer_matches_explicit_computation():
    """mask / mask_dict (fmoe/layers.py:289-317): masked tokens skip the experts; their k expert
    slots are filled from mask_dict before the weighted sum over the gate scores."""
    from fastermoe_b200 import FMoETransformerMLP
    torch.manual_seed(6)
    T, d, h, E, k = 64, 32, 64, 4, 2
    mask = torch.zeros(T, dtype=torch.long)
    mask[::5] = 1
    mask[3::7] = 2
    fill = {1: torch.zeros(d), 2: torch.full((d,), 0.5)}
    tens = O.make_layer_inputs(T, d, h, E, seed=6)
    plain = FMoETransformerMLP(num_expert=E, d_model=d, d_hidden=h, top_k=k)
    with torch.no_grad():
        plain.gate.gate.weight.copy_(tens["gate_w"]); plain.gate.gate.bias.copy_(tens["gate_b"])
        plain.experts.htoh4.weight.copy_(tens["w1"]); plain.experts.htoh4.bias.copy_(tens["b1"])
        plain.experts.h4toh.weight.copy_(tens["w2"]); plain.experts.h4toh.bias.copy_(tens["b2"])
    plain = plain.cuda()
    masked = FMoETransformerMLP(num_expert=E, d_model=d, d_hidden=h, top_k=k, mask=mask.cuda(),
                                mask_dict={key: v.cuda() for key, v in fill.items()})
    masked.load_state_dict(plain.state_dict())
    masked = masked.cuda()
    x = tens["x"].cuda()
    got = masked(x)
    want = plain(x).clone()          # unmasked tokens do not depend on the others
    with torch.no_grad():
        _, score = plain.gate(x)
    for key, v in fill.items():
        sel = mask == key
        want[sel] = score[sel].sum(dim=1, keepdim=True) * v.cuda()
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)


def test_index_add_gather_is_exact_and_ordered():
    """_local_gather(maybe_overlap=True) (fmoe/functions.py:77-81): rows that collide on one output row
    are added in ascending source order in fp32; also with more collisions than the kernel lists."""
    from fastermoe_b200.functions import _local_gather
    torch.manual_seed(8)
    for dtype, d, n_out, mult in ((torch.float32, 40, 50, 2), (torch.bfloat16, 256, 33, 3), (torch.float32, 64, 7, 20)):
        n = n_out * mult - 5
        pos = torch.randint(0, n_out, (n,))
        pos[:4] = -1                                   # skipped entries
        buf = torch.randn(n, d).to(dtype)
        want = torch.zeros(n_out, d)
        for i in range(n):                             # ascending i, fp32
            if pos[i] >= 0:
                want[pos[i]] += buf[i].float()
        got = _local_gather(buf.cuda(), pos.cuda(), n_out)
        assert torch.equal(got.cpu(), want.to(dtype)), (dtype, d, n_out, mult)
