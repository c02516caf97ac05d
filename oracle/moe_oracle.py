r"""CPU restatement of the FasterMoE MoE-layer hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product (the ``fastermoe_b200`` package) imports this file; it is
the checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.

Each function restates one piece of the reference (paths are relative to the
reference repository) in plain numpy / CPU PyTorch:

* integer routing work in numpy, bit-exact by construction;
* floating-point work (gate, expert MLP, combine) in CPU PyTorch, the same
  arithmetic the reference's own brute-force test oracle uses (tests/moe.py:6-49).

Parity pins: the floating-point functions and the shadowing policy are checked
against outputs of the reference's own Python code (tests/golden/*.npz, made by
tests/golden/make_golden.py by importing the reference).  The reference's
routing kernels are CUDA-only and order-nondeterministic inside a segment
(atomics, cuda/local_exchange.cuh:12-13, cuda/balancing.cuh:12,39); they are
pinned by tests/golden/routing_ref_gpu.npz, recorded from the reference's
kernels compiled by oracle/build_ref.py and run on a B200, and compared in the
canonical forms documented on each function below.
"""
import math

import numpy as np
import torch

# ---------------------------------------------------------------------------
# Routing (integers)
# ---------------------------------------------------------------------------


def expert_count(gate_idx, n_expert_total):
    """cuda/local_exchange.cuh:32-61 (and the CPU loop of cuda/tests/counting.cu:17-22):
    histogram of gate entries, -1 skipped.  int32 result."""
    g = np.asarray(gate_idx).reshape(-1)
    g = g[(g >= 0) & (g < n_expert_total)]
    return np.bincount(g, minlength=n_expert_total).astype(np.int32)


def assign_pos(gate_idx, n_expert_total):
    """cuda/local_exchange.cuh:5-16 with fmoe/functions.py:38-41.

    Segment e of the result, [cum[e-1], cum[e]), holds the flat indices whose gate
    is e.  The reference fills a segment in atomic arrival order; the canonical
    form used for comparison is ascending flat index (a stable counting sort),
    which is one of the orders the reference can produce."""
    g = np.asarray(gate_idx).reshape(-1)
    keep = np.nonzero((g >= 0) & (g < n_expert_total))[0]
    order = np.argsort(g[keep], kind="stable")
    return keep[order].astype(np.int64)


def canonical_pos(pos, counts):
    """Sorts every expert segment of a reference-produced ``pos`` ascending."""
    out = np.array(pos, dtype=np.int64, copy=True)
    start = 0
    for c in counts:
        out[start:start + c] = np.sort(out[start:start + c])
        start += int(c)
    return out


def inverse_pos(pos, n_entries):
    inv = np.full(n_entries, -1, dtype=np.int64)
    inv[np.asarray(pos)] = np.arange(len(pos), dtype=np.int64)
    return inv


def limit_by_capacity(ec, cap, n_expert, n_worker):
    """cuda/balancing.cuh:5-21.  ``ec`` is [W*E] laid out w*E+e; each expert serves
    its sources in ascending w (the canonical order of the reference's atomics):
    grant = clamp(capacity left, 0, request).  Returns (granted [W*E] int64,
    capacity after = cap - sum of requests, as the atomicSub leaves it)."""
    ec = np.asarray(ec, dtype=np.int64).reshape(n_worker, n_expert)
    left = np.asarray(cap, dtype=np.int64).copy()
    out = np.zeros_like(ec)
    for w in range(n_worker):
        prop = ec[w]
        out[w] = np.where(left >= prop, prop, np.where(left >= 0, left, 0))
        left = left - prop
    return out.reshape(-1), left.astype(np.int32)


def prune_gate_by_capacity(gate_idx, ec):
    """cuda/balancing.cuh:33-46.  An entry keeps its expert while the expert's
    allowance ``ec[e]`` lasts; canonical order = ascending flat index.  -1 stays -1.
    Returns (new gate, ec after = ec - number of entries per expert)."""
    g = np.asarray(gate_idx, dtype=np.int64)
    flat = g.reshape(-1)
    left = np.asarray(ec, dtype=np.int64).copy()
    out = flat.copy()
    for i, e in enumerate(flat):
        if e < 0:
            continue
        if left[e] <= 0:
            out[i] = -1
        left[e] -= 1
    return out.reshape(g.shape), left.astype(np.int32)


def limit_by_capacity_gate(topk_idx_per_rank, n_expert, n_worker, capacity):
    """Intended behaviour of fmoe/gates/utils.py:9-26 over all ranks at once:
    count -> exchange -> limit -> exchange back -> prune.  Returns per-rank
    (new_lec, new_gec, pruned gate)."""
    lecs = [expert_count(g, n_expert * n_worker).astype(np.int64) for g in topk_idx_per_rank]
    _, _, gecs = expert_exchange(lecs, n_expert, n_worker)
    new_gecs = [limit_by_capacity(gecs[r], np.full(n_expert, capacity), n_expert, n_worker)[0]
                for r in range(n_worker)]
    _, _, new_lecs = expert_exchange(new_gecs, n_expert, n_worker)
    out = []
    for r in range(n_worker):
        pruned, _ = prune_gate_by_capacity(topk_idx_per_rank[r], new_lecs[r])
        out.append((new_lecs[r], new_gecs[r], pruned))
    return out


# ---------------------------------------------------------------------------
# Exchange layouts (multi-rank, simulated in one process)
# ---------------------------------------------------------------------------


def expert_exchange(lec_per_rank, n_expert, n_worker):
    """cuda/global_exchange.cuh:8-58.  aec[src][dst][e] = all-gather of the local
    counts; agec[dst][src][e] its transpose; gec of rank r = agec[r].  Returns
    (aec, agec, [gec_r])."""
    aec = np.stack([np.asarray(l, dtype=np.int64).reshape(n_worker, n_expert) for l in lec_per_rank])
    agec = aec.transpose(1, 0, 2).copy()
    return aec, agec, [agec[r].reshape(-1) for r in range(n_worker)]


def scatter_moves(lecs, stored, rank, n_expert, n_worker):
    """Row map of global_scatter's output on ``rank`` (cuda/global_exchange.cuh:60-144).

    Returns ([(src_rank, src_row, dst_row, rows)], total rows): rows
    [src_row, +rows) of src_rank's token-side buffer land at dst_row of rank's
    expert-side buffer.  Order: rows kept local for shadowed workers j < rank, then
    received rows expert-major and source-minor, then rows kept local for shadowed
    workers j > rank."""
    st = np.asarray(stored).astype(bool).reshape(-1)
    eptrs = [np.concatenate([[0], np.cumsum(np.asarray(l, dtype=np.int64))]) for l in lecs]
    lec = np.asarray(lecs[rank], dtype=np.int64)
    out, rp = [], 0

    def local_block(j):
        nonlocal rp
        for i in range(n_expert):
            idx = i + j * n_expert
            if st[idx]:
                out.append((rank, int(eptrs[rank][idx]), rp, int(lec[idx])))
                rp += int(lec[idx])

    for j in range(rank):
        local_block(j)
    for i in range(n_expert):
        for j in range(n_worker):
            # rows that worker j routed to (rank, expert i)
            sidx = i + rank * n_expert
            n = int(lecs[j][sidx])
            if n and (not st[rank * n_expert + i] or j == rank):
                out.append((j, int(eptrs[j][sidx]), rp, n))
                rp += n
    for j in range(rank + 1, n_worker):
        local_block(j)
    return out, rp


def global_scatter(local_bufs, lecs, stored, n_expert, n_worker):
    """Simulates global_scatter on every rank.  local_bufs[r]: [A_r, d] array whose
    rows are ordered by (destination worker, expert).  Returns the expert-side
    buffers [B_r, d]."""
    outs = []
    for r in range(n_worker):
        moves, rows = scatter_moves(lecs, stored, r, n_expert, n_worker)
        buf = np.zeros((rows, local_bufs[r].shape[1]), dtype=local_bufs[r].dtype)
        for (src, src_row, dst_row, n) in moves:
            buf[dst_row:dst_row + n] = local_bufs[src][src_row:src_row + n]
        outs.append(buf)
    return outs


def global_gather(global_bufs, lecs, stored, n_expert, n_worker):
    """Inverse of global_scatter (cuda/global_exchange.cuh:146-230): returns the
    token-side buffers [A_r, d]."""
    outs = [np.zeros((int(np.sum(lecs[r])), global_bufs[r].shape[1]), dtype=global_bufs[r].dtype)
            for r in range(n_worker)]
    for r in range(n_worker):
        moves, _ = scatter_moves(lecs, stored, r, n_expert, n_worker)
        for (src, src_row, dst_row, n) in moves:
            outs[src][src_row:src_row + n] = global_bufs[r][dst_row:dst_row + n]
    return outs


def generate_cached_count(lec, gec, stored, rank, n_expert, n_worker):
    """cuda/global_exchange.cu:189-195."""
    lec = np.asarray(lec, dtype=np.int64).reshape(n_worker, n_expert)
    gec = np.asarray(gec, dtype=np.int64).reshape(n_worker, n_expert)
    st = np.asarray(stored).astype(bool).reshape(n_worker, n_expert)
    out = lec * st
    out[rank] = out[rank] + (gec * (~st[rank])).sum(0)
    return out.reshape(-1)


def fused_compute_ptrs(lec, gec, stored, rank, n_expert, n_worker):
    """cuda/fused_compute.cuh:216-248."""
    n = n_expert * n_worker
    st = np.asarray(stored).astype(bool).reshape(-1)
    local_ptr = np.zeros(n + 1, dtype=np.int64)
    global_ptr = np.zeros(n + 1, dtype=np.int64)
    lg_ptr = np.zeros(n + 1, dtype=np.int64)
    for i in range(n):
        local_ptr[i + 1] = local_ptr[i] + lec[i]
        lg_ptr[i + 1] = lg_ptr[i] + (lec[i] if st[i] else 0)
        e, w = i % n_expert, i // n_expert
        global_ptr[e * n_worker + w + 1] = 0 if st[rank * n_expert + e] else gec[i]
    global_ptr = np.concatenate([[0], np.cumsum(global_ptr[1:])]).astype(np.int64)
    return local_ptr, global_ptr, lg_ptr


# ---------------------------------------------------------------------------
# Shadowing policy
# ---------------------------------------------------------------------------


def global_policy(aec, agec, num_expert, world_size, d_model, fused, alpha,
                  bw_net=50 * 1e9 / 8, bw_mm=11.5e12, data_size=4):
    """fmoe/transformer.py:34-74, restated with explicit loops.  aec/agec: int64
    arrays [W, W, E].  Returns bool [W, E]."""
    agec = np.asarray(agec, dtype=np.int64)
    if fused:
        agec = agec.sum(-1).reshape(world_size, world_size, 1)
    load = agec.sum(1).astype(np.float64)  # [W, E']
    assert load.shape[1] == 1, "the reference policy only works at whole-worker granularity"
    # torch.sort(descending=True) is not stable; ties are broken here by the order
    # torch produces, which the golden test pins.
    order = torch.from_numpy(load.copy()).sort(0, descending=True)[1].numpy()[:, 0]
    unit = alpha * d_model ** 2 * data_size
    busiest = load.max()
    lat_plain = 3 * 4 * busiest * unit / bw_mm + 4 * busiest * d_model * data_size / bw_net
    model_cost = 2 * unit * num_expert / bw_net * 2
    comp_time = 12 * unit / bw_mm
    best, i = math.inf, 0
    for i, w in enumerate(order):
        load[w] = 0
        load += agec[w].reshape(world_size, -1)
        lat = load.max() * comp_time + (i + 1) * model_cost
        if lat < best:
            best = lat
        elif lat > best:
            break
    res = np.zeros((world_size, num_expert), dtype=bool)
    if lat_plain > best:
        res[order[:i]] = True
    return res


# ---------------------------------------------------------------------------
# Floating point: gate, experts, layer
# ---------------------------------------------------------------------------


def naive_gate(x, weight, bias, top_k, softmax_scores=False):
    """fmoe/gates/naive_gate.py:26-42: logits = x W^T + b, top-k (unsorted), scores =
    the raw top-k logits (the reference discards its softmax)."""
    logits = torch.nn.functional.linear(x, weight, bias)
    val, idx = torch.topk(logits, k=top_k, dim=-1, largest=True, sorted=False)
    val = val.view(-1, top_k)
    if softmax_scores:
        val = torch.softmax(val, dim=-1)
    return idx, val, logits


def activation(name):
    return {"gelu": torch.nn.functional.gelu, "relu": torch.relu, "none": (lambda v: v)}[name]


def expert_mlp(x, gate_flat, w1, b1, w2, b2, act):
    """tests/moe.py:31-44: per expert, rows with that gate: (x W1^T + b1) -> act -> W2^T + b2.
    Rows whose gate is -1 produce zeros."""
    out = torch.zeros(x.shape[0], w2.shape[1], dtype=x.dtype)
    f = activation(act)
    for e in range(w1.shape[0]):
        sel = gate_flat == e
        if not bool(sel.any()):
            continue
        h = x[sel] @ w1[e].t()
        if b1 is not None:
            h = h + b1[e]
        h = f(h)
        y = h @ w2[e].t()
        if b2 is not None:
            y = y + b2[e]
        out[sel] = y
    return out


def moe_layer(x, gate_idx, gate_score, w1, b1, w2, b2, act="gelu"):
    """tests/moe.py:31-49 (BruteForceMoELinear.forward): repeat each token top_k
    times, run its expert, weight by the gate score and sum over k."""
    top_k = gate_idx.shape[1]
    xr = x.repeat_interleave(top_k, dim=0)
    o = expert_mlp(xr, gate_idx.reshape(-1), w1, b1, w2, b2, act)
    return torch.bmm(gate_score.unsqueeze(1).to(o.dtype), o.view(-1, top_k, o.shape[1])).reshape(-1, o.shape[1])


def moe_layer_fwd_bwd(x, gate_w, gate_b, w1, b1, w2, b2, top_k, act="gelu", softmax_scores=False,
                      gate_idx=None, grad_out=None, score_idx=None, grads_for=None):
    """Forward + backward of gate -> experts -> combine on the CPU.  Returns a dict
    with the output and the gradients of every input that requires grad.  The loss is
    ``sum(out * grad_out)`` (``grad_out`` None = ones = out.sum()).  ``gate_idx`` prescribes the
    experts (-1 = pruned entry); ``score_idx`` (default: gate_idx) the experts whose logits give
    the scores, for gates that compute scores before a capacity limit prunes entries.  ``grads_for``: names of
    the inputs whose gradients are wanted (default: all); the others are used as they are, without a copy."""
    leaves = {}
    for name, t in (("x", x), ("gate_w", gate_w), ("gate_b", gate_b), ("w1", w1), ("b1", b1), ("w2", w2), ("b2", b2)):
        if t is None:
            leaves[name] = None
        elif grads_for is None or name in grads_for:
            leaves[name] = t.detach().clone().requires_grad_(True)
        else:
            leaves[name] = t.detach()
    idx, score, _ = naive_gate(leaves["x"], leaves["gate_w"], leaves["gate_b"], top_k, softmax_scores)
    if gate_idx is not None:
        # Use prescribed indices (e.g. after capacity pruning); scores follow the indices.
        logits = torch.nn.functional.linear(leaves["x"], leaves["gate_w"], leaves["gate_b"])
        idx = gate_idx
        score = torch.gather(logits, 1, (gate_idx if score_idx is None else score_idx).clamp(min=0))
        if softmax_scores:
            score = torch.softmax(score, dim=-1)
    out = moe_layer(leaves["x"], idx, score, leaves["w1"], leaves["b1"], leaves["w2"], leaves["b2"], act)
    loss = out.sum() if grad_out is None else (out * grad_out).sum()
    loss.backward()
    res = {"out": out.detach(), "gate_idx": idx.detach(), "gate_score": score.detach()}
    for name, t in leaves.items():
        if t is not None and t.requires_grad:
            res["grad_" + name] = t.grad
    return res


def hir_gate(x, weight, bias, n_expert, world_size, node_rank, stored, nw_per_node=4, ogn_ratio=0.14):
    """fmoe/gates/hir_gate.py:36-116 for one rank, given the policy's answer ``stored``
    (bool [W*E]).  Returns (idx [T,2], score [T,2])."""
    logits = torch.nn.functional.linear(x, weight, bias)
    tot = n_expert * world_size
    on_node = (torch.arange(tot) // (nw_per_node * n_expert)) == node_rank
    limited = (~on_node) & ~torch.as_tensor(stored).reshape(-1).bool()
    top2_val, top2_idx = torch.topk(logits, k=2, dim=-1)
    top1_idx, top1_val = top2_idx[:, 0], top2_val[:, 0].clone()
    leaving = limited[top1_idx]
    thres = int(x.shape[0] * ogn_ratio)
    if int(leaving.sum()) < thres:
        return top2_idx, torch.softmax(top2_val, dim=-1)
    top1_val[~leaving] = float("-inf")
    _, keep = torch.topk(top1_val, k=thres)
    cand = logits.clone()
    cand[:, limited] = float("-inf")
    _, idx = torch.topk(cand, k=2)
    idx[keep, 1] = top1_idx[keep]
    val = torch.gather(logits, 1, idx)
    return idx, torch.softmax(val, dim=-1)


# ---------------------------------------------------------------------------
# Synthetic workloads
# ---------------------------------------------------------------------------


def uniform_fan_in(shape, fan_in, gen):
    b = 1.0 / math.sqrt(fan_in)
    return (torch.rand(shape, generator=gen) * 2 - 1) * b


def make_layer_inputs(tokens, d_model, d_hidden, n_expert_total, seed, gate_std=None, gate_bias=None):
    """Seeded synthetic tensors with the benchmark workloads' value distributions: x ~ N(0,1);
    expert weights/biases U(+-1/sqrt(fan_in)); gate weight U(+-1/sqrt(d)) or
    N(0, gate_std) with zero (or given) bias."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, d_model, generator=g)
    if gate_std is None:
        gw = uniform_fan_in((n_expert_total, d_model), d_model, g)
        gb = uniform_fan_in((n_expert_total,), d_model, g)
    else:
        gw = torch.randn(n_expert_total, d_model, generator=g) * gate_std
        gb = torch.zeros(n_expert_total) if gate_bias is None else gate_bias.clone()
    w1 = uniform_fan_in((n_expert_total, d_hidden, d_model), d_model, g)
    b1 = uniform_fan_in((n_expert_total, d_hidden), d_model, g)
    w2 = uniform_fan_in((n_expert_total, d_model, d_hidden), d_hidden, g)
    b2 = uniform_fan_in((n_expert_total, d_model), d_hidden, g)
    return dict(x=x, gate_w=gw, gate_b=gb, w1=w1, b1=b1, w2=w2, b2=b2)
