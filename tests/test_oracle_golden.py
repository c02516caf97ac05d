"""The CPU oracle against outputs recorded from the reference's own Python code
(tests/golden/reference_cpu.npz, made by tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

LAYER_CASES = ["layer_e4_k2_gelu", "layer_e8_k3_gelu", "layer_e4_k2_relu", "layer_e16_k2_gelu"]


def t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("tag", LAYER_CASES)
def test_layer_matches_reference(golden, tag):
    z = {k.split("/", 1)[1]: golden[k] for k in golden.files if k.startswith(tag + "/")}
    T, d, h, E, k, act, seed = z["meta"].tolist()
    act = {2: "gelu", 1: "relu"}[act]
    res = O.moe_layer_fwd_bwd(t(z["x"]), t(z["gate_w"]), t(z["gate_b"]), t(z["w1"]), t(z["b1"]), t(z["w2"]),
                              t(z["b2"]), k, act=act)
    assert np.array_equal(res["gate_idx"].numpy(), z["idx"])
    np.testing.assert_allclose(res["gate_score"].numpy(), z["score"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(res["out"].numpy(), z["out"], rtol=1e-5, atol=1e-6)
    for name in ("x", "gate_w", "gate_b", "w1", "b1", "w2", "b2"):
        np.testing.assert_allclose(res["grad_" + name].numpy(), z["grad_" + name], rtol=1e-5, atol=1e-6,
                                   err_msg=name)


def test_gate_returns_raw_logits(golden):
    z = golden
    idx, score, logits = O.naive_gate(t(z["layer_e4_k2_gelu/x"]), t(z["layer_e4_k2_gelu/gate_w"]),
                                      t(z["layer_e4_k2_gelu/gate_b"]), 2)
    assert np.array_equal(idx.numpy(), z["layer_e4_k2_gelu/idx"])
    # not a softmax: rows do not sum to one
    assert not np.allclose(z["layer_e4_k2_gelu/score"].sum(1), 1.0)
    np.testing.assert_allclose(torch.gather(logits, 1, idx).numpy(), z["layer_e4_k2_gelu/score"], rtol=1e-6)


def test_local_scatter_gather(golden):
    inp, gate, pos = golden["local/inp"], golden["local/gate_idx"], golden["local/pos"]
    assert np.array_equal(O.assign_pos(gate, 4), pos)
    buf = inp[pos // 2]
    assert np.array_equal(buf, golden["local/buf"])
    back = np.zeros((24, inp.shape[1]), dtype=inp.dtype)
    back[pos] = buf
    assert np.array_equal(back, golden["local/back_copy"])
    inv = O.inverse_pos(pos, 24)
    add = np.zeros_like(inp)
    for tok in range(12):
        for j in range(2):
            if inv[tok * 2 + j] >= 0:
                add[tok] += buf[inv[tok * 2 + j]]
    np.testing.assert_allclose(add, golden["local/back_add"], rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("tag", ["skew40", "uniform", "zipf", "w2"])
def test_policy(golden, tag):
    aec = golden[f"policy/{tag}/aec"]
    W, E, d_model, alpha = golden[f"policy/{tag}/meta"].tolist()
    W, E, d_model = int(W), int(E), int(d_model)
    agec = aec.transpose(1, 0, 2)
    want = golden[f"policy/{tag}/res"]
    got = O.global_policy(aec, agec, E, W, d_model, True, alpha)
    assert np.array_equal(got, want)
    # the product's host-side policy (same constants) must agree as well
    os.environ["FMOE_ENABLE_DYNREP"] = "1"
    try:
        from fastermoe_b200.transformer import _gen_policy
        pol = _gen_policy(alpha, constants="reference")
    finally:
        os.environ["FMOE_ENABLE_DYNREP"] = "0"
    res = pol(t(aec).long(), t(agec.copy()).long(), E, W, d_model, True)
    assert np.array_equal(res.numpy(), want)


@pytest.mark.parametrize("tag", ["few_leaving", "many_leaving", "uniform"])
def test_hir_gate(golden, tag):
    z = {k.split("/", 2)[2]: golden[k] for k in golden.files if k.startswith(f"hir/{tag}/")}
    W, E, d, T, rank, policy_on = z["meta"].tolist()
    aec = z["aec"].copy()
    stored = np.zeros(W * E, dtype=bool)
    if policy_on:
        # the recorded run replaced row `rank` of the table by the rank's own counts
        idx0 = torch.topk(torch.nn.functional.linear(t(z["x"]), t(z["gate_w"]), t(z["gate_b"])), 2)[1]
        aec[rank] = O.expert_count(idx0.numpy(), W * E).reshape(W, E)
        st = O.global_policy(aec, aec.transpose(1, 0, 2), E, W, d, True, 4.0)
        stored = np.repeat(st.any(1), E)
    idx, score = O.hir_gate(t(z["x"]), t(z["gate_w"]), t(z["gate_b"]), E, W, rank // 4, stored)
    assert np.array_equal(idx.numpy(), z["idx"])
    np.testing.assert_allclose(score.numpy(), z["score"], rtol=1e-6, atol=1e-7)


def test_routing_oracle_invariants():
    rng = np.random.default_rng(0)
    for n, E in [(0, 4), (1, 1), (257, 3), (4096, 64)]:
        gate = rng.integers(-1, E, size=n)
        cnt = O.expert_count(gate, E)
        pos = O.assign_pos(gate, E)
        assert cnt.sum() == (gate >= 0).sum() == len(pos)
        assert np.array_equal(gate[pos], np.repeat(np.arange(E), cnt))
        cap = rng.integers(0, max(1, n // max(E, 1)) + 2, size=E)
        pruned, left = O.prune_gate_by_capacity(gate, cap)
        kept = O.expert_count(pruned, E)
        assert np.array_equal(kept, np.minimum(cnt, cap))
        assert np.array_equal(left, cap - cnt)
        assert np.all((pruned == gate) | (pruned == -1))


def test_exchange_oracle_roundtrip():
    rng = np.random.default_rng(1)
    W, E, d = 4, 3, 5
    lecs = [rng.integers(0, 6, size=W * E) for _ in range(W)]
    for stored in (np.zeros(W * E, bool), np.repeat(np.array([False, True, False, False]), E)):
        bufs = [rng.standard_normal((int(l.sum()), d)).astype(np.float32) for l in lecs]
        g = O.global_scatter(bufs, lecs, stored, E, W)
        _, _, gecs = O.expert_exchange(lecs, E, W)
        for r in range(W):
            assert g[r].shape[0] == O.generate_cached_count(lecs[r], gecs[r], stored, r, E, W).sum()
        back = O.global_gather(g, lecs, stored, E, W)
        for r in range(W):
            assert np.array_equal(back[r], bufs[r])


# ---- the reference's own CUDA routing kernels, recorded on a B200 (tests/golden/make_routing_golden.py)

@pytest.fixture(scope="module")
def routing_golden():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "routing_ref_gpu.npz"))


@pytest.mark.parametrize("case", range(5))
def test_oracle_matches_reference_count_and_positions(routing_golden, case):
    z = routing_golden
    n, E = z[f"route{case}/meta"].tolist()
    gate, cnt = z[f"route{case}/gate"], z[f"route{case}/count"]
    assert np.array_equal(O.expert_count(gate, E), cnt)
    # the reference fills a segment in atomic arrival order: compare segments as sorted sets
    assert np.array_equal(O.canonical_pos(z[f"route{case}/pos"], cnt), O.assign_pos(gate, E))
    assert np.array_equal(z[f"route{case}/cum_after"], np.cumsum(cnt) - cnt)


@pytest.mark.parametrize("case", range(3))
def test_oracle_matches_reference_limit_by_capacity(routing_golden, case):
    z = routing_golden
    W, E = z[f"limit{case}/meta"].tolist()
    ec, cap = z[f"limit{case}/ec"], z[f"limit{case}/cap"]
    got, left = O.limit_by_capacity(ec, cap, E, W)
    ref = z[f"limit{case}/eca"]
    assert np.array_equal(left, z[f"limit{case}/cap_after"])
    assert np.array_equal(got.reshape(W, E).sum(0), ref.reshape(W, E).sum(0))   # order-independent part
    assert np.all(ref <= ec)
    if W == 1:
        assert np.array_equal(got, ref)


@pytest.mark.parametrize("case", range(3))
def test_oracle_matches_reference_prune(routing_golden, case):
    z = routing_golden
    n, E = z[f"prune{case}/meta"].tolist()
    gate, ec, ref = z[f"prune{case}/gate"], z[f"prune{case}/ec"], z[f"prune{case}/pruned"]
    got, left = O.prune_gate_by_capacity(gate, ec)
    assert np.array_equal(left, z[f"prune{case}/ec_after"])
    assert np.array_equal(O.expert_count(got, E), O.expert_count(ref, E))      # kept per expert
    assert np.all((ref == gate) | (ref == -1))


def test_oracle_matches_reference_linear(routing_golden):
    z = routing_golden
    counts = z["linear/counts"].tolist()
    x, w, b, gy = (t(z["linear/" + k]) for k in ("x", "w", "b", "gy"))
    p = 0
    for e, c in enumerate(counts):
        sl = slice(p, p + c)
        np.testing.assert_allclose((x[sl] @ w[e].t() + b[e]).numpy(), z["linear/y"][sl], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose((gy[sl] @ w[e]).numpy(), z["linear/gx"][sl], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose((gy[sl].t() @ x[sl]).numpy(), z["linear/gw"][e], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(gy[sl].sum(0).numpy(), z["linear/gb"][e], rtol=1e-5, atol=1e-5)
        p += c


def test_policy_matches_the_reference_implementation_on_random_tables():
    """The product's host-side policy against the reference's own _gen_policy (the staged copy of its
    Python package), on random count tables: balanced, skewed, tiny and large worlds."""
    import types
    from oracle import stage_reference
    if stage_reference.staged() is None and stage_reference.stage() is None:
        pytest.skip("no staged copy of the reference's Python package")
    import sys
    saved = {n: m for n, m in sys.modules.items() if n == "fmoe_cuda" or n == "fmoe" or n.startswith("fmoe.")}
    os.environ["FMOE_ENABLE_DYNREP"] = "1"
    try:
        stage_reference.import_reference(types.ModuleType("fmoe_cuda"))
        from fmoe.transformer import _gen_policy as ref_gen
        from fastermoe_b200.transformer import _gen_policy
        rng = np.random.default_rng(11)
        n_shadow = 0
        for trial in range(300):
            W = int(rng.choice([2, 3, 4, 8, 16]))
            E = int(rng.choice([1, 2, 4]))
            d_model = int(rng.choice([64, 256, 1024, 4096]))
            alpha = float(rng.choice([2.0, 4.0]))
            p = rng.dirichlet(np.full(W * E, float(rng.choice([0.05, 0.3, 5.0]))))
            table = np.stack([rng.multinomial(int(rng.choice([64, 4096, 65536])), p).reshape(W, E) for _ in range(W)]).astype(np.int64)
            aec = t(table).long()
            agec = aec.transpose(0, 1).contiguous()
            want = ref_gen(alpha)(aec.clone(), agec.clone(), E, W, d_model, True)
            got = _gen_policy(alpha, constants="reference")(aec, agec, E, W, d_model, True)
            assert torch.equal(got, want), (trial, W, E, d_model, alpha, table.tolist())
            n_shadow += int(want.any())
        assert 20 < n_shadow < 280, n_shadow           # both outcomes are exercised
    finally:
        os.environ["FMOE_ENABLE_DYNREP"] = "0"
        for n in [n for n in sys.modules if n == "fmoe_cuda" or n == "fmoe" or n.startswith("fmoe.")]:
            del sys.modules[n]
        sys.modules.update(saved)
