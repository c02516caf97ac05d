"""The Megatron-style plug-in (fastermoe_b200.megatron) without Megatron-LM: a stand-in model with the
attribute layout the adapter walks (model.language_model.transformer.layers[i].mlp), argument and
parallel-state objects bound through megatron.bind, and two simulated data-parallel ranks for the
expert-sharded checkpoint (fmoe/megatron/checkpoint.py:51-386, layers.py:106-258)."""
import argparse
import os
import types

import pytest
import torch
import torch.nn as nn

from fastermoe_b200 import megatron as M


def make_args(**kw):
    a = types.SimpleNamespace(hidden_size=64, num_layers=2, init_method_std=0.02, seq_length=8, micro_batch_size=2,
                              tensor_model_parallel_size=1, data_parallel_size=1, pipeline_model_parallel_size=1,
                              world_size=1, rank=0, balance_strategy=None, balance_loss_weight=1.0, num_experts=None,
                              hidden_hidden_size=None, top_k=None)
    a.__dict__.update(kw)
    return a


class FakeMpu:
    def get_tensor_model_parallel_group(self):
        return None

    def get_data_parallel_group(self):
        return None


class Block(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.attn = nn.Linear(d, d)
        self.mlp = nn.Sequential(nn.Linear(d, 4 * d), nn.GELU(), nn.Linear(4 * d, d))


class FakeMegatronModel(nn.Module):
    def __init__(self, d, n_layers):
        super().__init__()
        self.language_model = nn.Module()
        self.language_model.transformer = nn.Module()
        self.language_model.transformer.layers = nn.ModuleList([Block(d) for _ in range(n_layers)])


@pytest.fixture
def bound():
    args = make_args()
    M.bind(args=args, mpu=FakeMpu())
    yield args
    M.unbind()


def test_arguments_are_added():
    p = M.add_fmoe_args(argparse.ArgumentParser())
    ns = p.parse_args(["--fmoefy", "--num-experts", "8", "--balance-strategy", "gshard"])
    assert ns.fmoefy and ns.num_experts == 8 and ns.top_k == 2 and ns.balance_strategy == "gshard"
    assert ns.hidden_hidden_size is None and ns.balance_loss_weight == 1


def test_unbound_adapter_says_what_is_missing():
    M.unbind()
    with pytest.raises(ImportError, match="bind"):
        M.fmoefy(FakeMegatronModel(64, 1), num_experts=2)


def test_fmoefy_replaces_every_mlp(bound):
    torch.manual_seed(0)
    model = M.fmoefy(FakeMegatronModel(64, 2), num_experts=4, top_k=2)
    layers = model.language_model.transformer.layers
    assert bound.hidden_hidden_size == 256 and bound.top_k == 2 and bound.distributed_experts is True
    for layer in layers:
        mlp = layer.mlp
        assert isinstance(mlp, M.MegatronMLP) and mlp.num_expert == 4 and mlp.top_k == 2 and mlp.world_size == 1
        assert tuple(mlp.experts.htoh4.weight.shape) == (4, 256, 64) and tuple(mlp.experts.h4toh.weight.shape) == (4, 64, 256)
        # expert parameters stay with their rank; the gate is replicated over the MoE group
        assert all(p.dp_comm == "none" for p in mlp.experts.parameters())
        assert all(getattr(p, "dp_comm", None) not in (None, "none") for p in mlp.gate.parameters())
        # Megatron's MLP initialisation: N(0, sigma) in, N(0, sigma / sqrt(2 L)) out, zero biases
        assert abs(float(mlp.experts.htoh4.weight.detach().std()) - 0.02) < 0.002
        assert abs(float(mlp.experts.h4toh.weight.detach().std()) - 0.02 / 2.0) < 0.001
        assert float(mlp.experts.htoh4.bias.detach().abs().max()) == 0.0
    assert isinstance(layers[0].attn, nn.Linear)                      # nothing else is touched
    prof = M.get_balance_profile()
    assert set(prof) == {"coefficient-variation", "Lmax-over-Lmin", "Lmax-over-Lmean"}
    assert all(len(v) == 2 for v in prof.values())


def test_replicated_experts_are_tagged_for_data_parallel(bound):
    model = M.fmoefy(FakeMegatronModel(64, 1), num_experts=2, distributed_experts=False)
    mlp = model.language_model.transformer.layers[0].mlp
    assert mlp.world_size == 1 and all(p.dp_comm == "dp" for p in mlp.experts.parameters())


def test_gate_hook_records_the_imbalance(bound):
    bound.balance_strategy = "gshard"
    M.reset_gate_hook(3)
    hook = M.generate_megatron_gate_hook(1, 4)
    idx = torch.tensor([[0, 1], [0, 2], [0, 3], [0, -1]])          # expert 0 four times, -1 = pruned
    hook(idx, None, None)
    prof = M.get_balance_profile()
    assert "gshard_loss" in prof and len(prof["gshard_loss"]) == 3
    counts = torch.tensor([4.0, 1.0, 1.0, 1.0])
    assert torch.isclose(prof["Lmax-over-Lmean"][1], counts.max() / counts.mean())
    assert torch.isclose(prof["Lmax-over-Lmin"][1], torch.tensor(5.0 / 2.0))
    assert prof["Lmax-over-Lmean"][0] is None and prof["Lmax-over-Lmean"][2] is None


def test_forward_step_gets_the_balance_loss(bound):
    bound.balance_strategy = "gshard"
    bound.balance_loss_weight = 0.5
    model = M.fmoefy(FakeMegatronModel(64, 2), num_experts=2)
    for i, layer in enumerate(model.language_model.transformer.layers):
        layer.mlp.gate.set_loss(torch.tensor(float(i + 1)))            # what the gates would have stored
    step = M.patch_forward_step(lambda it, m: (torch.tensor(10.0), {}), is_pipeline_last_stage=lambda: True)
    loss, stats = step(None, model)
    assert float(loss) == 10.0 + 0.5 * 1.5 and float(stats["gshard_loss"]) == 0.75
    bound.balance_strategy = "naive"                                    # a gate without a loss: untouched
    step = M.patch_forward_step(lambda it, m: (torch.tensor(10.0), {}), is_pipeline_last_stage=lambda: True)
    assert float(step(None, model)[0]) == 10.0


def test_balance_log_and_model_provider(bound):
    bound.balance_strategy, bound.num_experts, bound.top_k = "gshard", 2, 2
    provider = M.patch_model_provider(lambda: FakeMegatronModel(64, 2))
    model = provider()
    mlps = [l.mlp for l in model.language_model.transformer.layers]
    assert all(isinstance(m, M.MegatronMLP) for m in mlps)
    assert mlps[0].experts.htoh4.weight.shape[1] == 4 * 64 // 2           # the dense model's cost per token is kept
    M.generate_megatron_gate_hook(0, 2)(torch.tensor([[0, 1], [0, 0]]), None, None)
    mlps[0].gate.set_loss(torch.tensor(0.25))
    mlps[1].gate.set_loss(torch.tensor(0.75))

    class Writer:
        def __init__(self):
            self.rows = {}

        def add_scalar(self, name, value, iteration):
            self.rows[name] = (value, iteration)

    w = Writer()
    M.add_balance_log(model, w, 5, is_last_rank=True)
    assert w.rows["balance-gshard_loss/layer-0"] == (0.25, 5) and w.rows["balance-gshard_loss/layer-1"] == (0.75, 5)
    assert w.rows["balance-gshard_loss/all"] == (0.5, 5)
    assert w.rows["balance-Lmax-over-Lmean/layer-0"][0] == pytest.approx(1.5)      # counts [3, 1]
    assert "balance-Lmax-over-Lmean/layer-1" not in w.rows                          # layer 1 routed nothing
    assert mlps[0].gate.get_loss() is None                                          # cleared by the log
    quiet = Writer()
    M.add_balance_log(model, quiet, 6, is_last_rank=False)
    assert quiet.rows == {}


def test_checkpoint_names():
    P = M.GridPosition
    assert M.checkpoint_name("/c", 100, P(0, 1, 0, 1)) == "/c/iter_0000100/mp_rank_01/model_optim_rng.pt"
    assert M.checkpoint_name("/c", 100, P(3, 1, 0, 1)) == "/c/iter_0000100/mp_rank_01_dp_rank_0003/model_optim_rng.pt"
    assert M.checkpoint_name("/c", 7, P(3, 0, 2, 4)) == "/c/iter_0000007/mp_rank_00_002_dp_rank_0003/model_optim_rng.pt"
    assert M.checkpoint_name("/c", 7, P(0, 0, 2, 4), release=True) == "/c/release/mp_rank_00_002/model_optim_rng.pt"


class Toy(nn.Module):
    """Two replicated tensors and two expert tensors, nested like Megatron's state dicts."""

    def __init__(self, seed):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.shared = nn.Linear(4, 4)
        self.experts = nn.Linear(4, 4)
        with torch.no_grad():
            for p in self.parameters():
                p.copy_(torch.randn(p.shape, generator=g))
        for p in self.experts.parameters():
            p.dp_comm = "none"
        for p in self.shared.parameters():
            p.dp_comm = "dp"

    def state_dict_for_save_checkpoint(self, keep_vars=False):
        return {"language_model": {"shared": self.shared.state_dict(keep_vars=keep_vars),
                                   "experts": self.experts.state_dict(keep_vars=keep_vars)}}

    def load_state_dict(self, sd, strict=True):
        self.shared.load_state_dict(sd["language_model"]["shared"], strict=strict)
        self.experts.load_state_dict(sd["language_model"]["experts"], strict=strict)


def trained(seed, shared_from=None):
    m = Toy(seed)
    if shared_from is not None:
        m.shared.load_state_dict(shared_from.shared.state_dict())
    opt = torch.optim.Adam(m.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(seed + 100)
    for _ in range(2):
        opt.zero_grad()
        (m.experts(m.shared(torch.randn(3, 4, generator=g))) ** 2).sum().backward()
        opt.step()
    return m, opt


def test_expert_sharded_checkpoint_round_trip(tmp_path):
    root = str(tmp_path)
    m0, o0 = trained(1)
    m1, o1 = trained(2)                       # another data-parallel rank: other experts
    with torch.no_grad():                     # ... and the same replicated tensors (what data parallelism maintains)
        for a, b in zip(m1.shared.parameters(), m0.shared.parameters()):
            a.copy_(b)
    P = M.GridPosition
    f0 = M.save_shard(root, 40, m0, o0, P(0, 0, 0, 1), extra={"checkpoint_version": 3.0})
    f1 = M.save_shard(root, 40, m1, o1, P(1, 0, 0, 1))
    M.write_tracker(root, 40)
    assert os.path.dirname(f1).endswith("mp_rank_00_dp_rank_0001") and os.path.dirname(f0).endswith("mp_rank_00")
    own = torch.load(f1, weights_only=False)
    # the second rank's file holds its experts only: model tensors, optimizer state of parameters 2 and 3
    assert set(own["model"]["language_model"]) == {"experts"} and "iteration" not in own
    assert set(own["optimizer"]["state"]) == {2, 3} and "param_groups" not in own["optimizer"]
    assert M.read_tracker(root) == (40, False)

    fresh, fresh_opt = trained(9)
    blob = M.load_shard(root, fresh, fresh_opt, P(1, 0, 0, 1))
    assert blob["iteration"] == 40 and blob["checkpoint_version"] == 3.0
    for a, b in zip(fresh.shared.parameters(), m0.shared.parameters()):
        assert torch.equal(a, b)
    for a, b in zip(fresh.experts.parameters(), m1.experts.parameters()):
        assert torch.equal(a, b)
    st, st0, st1 = fresh_opt.state_dict()["state"], o0.state_dict()["state"], o1.state_dict()["state"]
    for i in (0, 1):
        assert torch.equal(st[i]["exp_avg"], st0[i]["exp_avg"])           # replicated tensors: rank 0's moments
    for i in (2, 3):
        assert torch.equal(st[i]["exp_avg"], st1[i]["exp_avg"]) and torch.equal(st[i]["exp_avg_sq"], st1[i]["exp_avg_sq"])
    # rank 0 reads its own file alone
    again, again_opt = trained(11)
    M.load_shard(root, again, again_opt, P(0, 0, 0, 1))
    for a, b in zip(again.parameters(), m0.parameters()):
        assert torch.equal(a, b)
    assert M.load_shard(str(tmp_path / "nothing"), again, again_opt, P(0, 0, 0, 1)) is None


def test_fp16_wrapper_state_keeps_expert_master_copies():
    m, opt = trained(3)
    params = list(m.parameters())
    masters = [[p.detach().float().clone() for p in params]]
    for mp, p in zip(masters[0], params):
        if hasattr(p, "dp_comm"):
            mp.dp_comm = p.dp_comm
    wrapped = {"optimizer": opt.state_dict(), "fp32_from_fp16_params": masters, "grad_scaler": {"scale": 2.0}}
    cut = M.expert_optimizer_state(wrapped, params, master_params=masters)
    assert set(cut["optimizer"]["state"]) == {2, 3} and "param_groups" not in cut["optimizer"]
    assert [x is None for x in cut["fp32_from_fp16_params"][0]] == [True, True, False, False]
    assert "param_groups" in opt.state_dict()                             # the optimizer's own dict is untouched
    full = {"model": m.state_dict_for_save_checkpoint(),
            "optimizer": {"optimizer": opt.state_dict(), "fp32_from_fp16_params": [[None] * 4]}}
    merged = M.overlay(full, {"model": {}, "optimizer": cut})
    assert merged["optimizer"]["fp32_from_fp16_params"][0][2] is masters[0][2]
    assert merged["optimizer"]["fp32_from_fp16_params"][0][0] is None


@pytest.mark.gpu
def test_megatron_mlp_runs_and_reports_balance(bound):
    bound.balance_strategy = "naive"
    bound.hidden_size = 256
    model = M.fmoefy(FakeMegatronModel(256, 2), num_experts=4, hidden_hidden_size=512).cuda().bfloat16()
    x = torch.randn(bound.seq_length, bound.micro_batch_size, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out, bias = model.language_model.transformer.layers[1].mlp(x)
    assert out.shape == x.shape and bias.shape == (256,) and float(bias.abs().max()) == 0.0
    out.float().sum().backward()
    assert torch.isfinite(x.grad.float()).all() and x.grad.float().abs().sum() > 0
    prof = M.get_balance_profile()
    assert prof["Lmax-over-Lmean"][1] is not None and float(prof["Lmax-over-Lmean"][1]) >= 1.0
    assert prof["Lmax-over-Lmean"][0] is None                            # layer 0 was not called
