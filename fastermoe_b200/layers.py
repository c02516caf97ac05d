r"""MoE layer (mirrors the public classes of fmoe/layers.py)."""
import math
import os

import torch
import torch.nn as nn

from . import fmoe_cuda
from .functions import (AllGather, Exchange, ExpertCounts, MOECache, MOEGatherCombine, MOELinear,
                        MOEScatterFused, PlannedExchange, Slice, cached_count_host, ensure_comm, route)
from .gates import NaiveGate


class FMoELinear(nn.Module):
    r"""One linear layer per expert, evaluated for all experts of a worker in a
    single grouped GEMM (fmoe/layers.py:16-67).  ``weight`` is [E, out, in],
    ``bias`` [E, out]."""

    def __init__(self, num_expert, in_feat, out_feat, bias=True, rank=0):
        super().__init__()
        self.num_expert, self.in_feat, self.out_feat, self.rank = num_expert, in_feat, out_feat, rank
        self.weight = nn.Parameter(torch.empty(num_expert, out_feat, in_feat))
        if bias:
            self.bias = nn.Parameter(torch.zeros(num_expert, out_feat))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def forward(self, inp, fwd_expert_count):
        """``fwd_expert_count``: rows per expert, as a CPU/CUDA int64 tensor or ExpertCounts."""
        return MOELinear.apply(inp, fwd_expert_count, self.weight, self.bias)

    def extra_repr(self):
        return "num_expert={}, in_features={}, out_features={}, bias={}, rank={}".format(
            self.num_expert, self.in_feat, self.out_feat, self.bias is not None, self.rank)

    def reset_parameters(self):
        # Same call as the reference (fmoe/layers.py:62-67): the fan-in is taken
        # over the 3-D tensor, so the default scale is small; callers that care
        # set the weights explicitly.
        torch.nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))


def mark_module_parallel_comm(module, comm):
    """Tags every parameter of ``module`` with the data-parallel group name ``comm``
    ('world', 'dp', 'moe' or 'none'), read by DistributedGroupedDataParallel."""
    for p in module.parameters():
        setattr(p, "dp_comm", comm)


_no_shadow = {}


def _no_shadow_flags(world_size, num_expert):
    key = (world_size, num_expert)
    if key not in _no_shadow:
        _no_shadow[key] = torch.zeros(world_size, num_expert, dtype=torch.bool)
    return _no_shadow[key]


def _shadow_plan(policy_fn, routing, experts, num_expert, world_size, d_model, fused, shadows):
    """Runs the shadowing policy on the count tables and makes sure a module exists
    for every shadowed worker.  Returns (stored [W,E] bool CPU, stored_workers [W])."""
    stored = policy_fn(routing.aec.view(world_size, world_size, num_expert),
                       routing.agec.view(world_size, world_size, num_expert),
                       num_expert, world_size, d_model, fused).cpu()
    workers = stored.any(dim=1)
    if fused:
        # Whole-worker granularity: all experts of a shadowed worker travel together.
        stored = workers.view(world_size, 1).repeat(1, num_expert)
    if bool(workers.any()):
        import copy
        for j in range(world_size):
            if bool(workers[j]) and j != routing.rank and j not in shadows:
                m = copy.deepcopy(experts)
                for p in m.parameters():
                    p.grad = None
                shadows[j] = m
    return stored, workers


def _fmoe_general_global_forward(inp, gate, expert_fn, policy_fn, experts, num_expert, world_size,
                                 fused, enable_fuse=False, gate_score=None, shadows=None):
    r"""Routes ``inp`` to the experts chosen in ``gate`` and back.

    Steps (same as fmoe/layers.py:79-149): count tokens per expert, bucket them so
    that each expert's rows are contiguous, exchange rows between workers,
    run ``expert_fn``, and undo the exchange and the bucketing.

    With ``gate_score`` the weighted sum over the top-k outputs is fused into
    the final gather and a [T, d] tensor is returned; without it the result is
    the [T*k, d] tensor the reference returns.  Also returns ``stored_models``.
    """
    top_k = gate.shape[1] if gate.dim() == 2 else 1
    n_tokens = inp.shape[0]
    early = None
    cap_rows = 0
    no_policy = policy_fn is None or getattr(policy_fn, "never_shadows", False)
    # The smart schedule's aim -- rows travelling while the experts compute (cuda/fused_compute.cuh:289-349)
    # -- is met on the device-planned path by the GEMMs themselves (outputs stored straight into their
    # owners' buffers; optionally the scatter's push beside the first product), so the flag selects that path
    # whenever nothing is shadowed.  FMOE_B200_SMART=nccl keeps the reference's shape: one NCCL group per
    # pipeline step on a side stream, the step's GEMMs on the compute stream (csrc/fused.cu), which is also
    # what runs when experts are shadowed.
    if enable_fuse and no_policy and fused and os.environ.get("FMOE_B200_SMART", "peer") != "nccl":
        enable_fuse = False
    if world_size > 1 and not enable_fuse:
        # Nothing has to come back to the host when no shadowing policy wants to see the counts, the
        # experts are one fused module (it reads its segment offsets on the device) and the rows
        # travel through peer memory: buffers are then sized for the worst case the pool can hold.
        if no_policy and fused and os.environ.get("FMOE_B200_NOSYNC", "1") != "0":
            cap_rows = fmoe_cuda.nosync_capacity(n_tokens * top_k, inp.shape[1] * inp.element_size(), world_size,
                                                 inp.device)
        if cap_rows == 0:
            # the local scatter needs the positions only: queue it before the host waits for the counts
            def early(r, inp=inp):
                with torch.no_grad():
                    return fmoe_cuda.local_scatter(inp.detach().contiguous(), r.pos, pos_div=top_k, n_rows=r.pos.numel())
    routing = route(gate, num_expert, world_size, before_wait=early, cap_rows=cap_rows)

    if world_size == 1:
        # No exchange, no host copies: buffers have one row per gate entry; rows past
        # the kept count are never touched by the grouped GEMMs.
        stored = torch.zeros(1, num_expert, dtype=torch.bool)
        x = MOEScatterFused.apply(inp, routing.pos, routing.inv, top_k, routing.n_rows, None)
        counts = ExpertCounts(routing.offsets_dev)
        x = expert_fn(x, [[experts] if fused else experts], counts, num_expert)
        exch = None
        n_rows = routing.n_rows
    elif routing.plan is not None:
        # No host copy of the counts: plan, offsets and row counts stay on the device.
        stored = _no_shadow_flags(world_size, num_expert)
        # the push of the scatter runs beside the experts' first GEMM (and, in the backward pass, beside
        # the input-gradient GEMM of the second layer) when the experts module can wait for rows tile by tile
        overlap, fused_gather = 0, False
        if getattr(experts, "consumes_arrival", None) is not None and experts.consumes_arrival(inp):
            overlap = int(os.environ.get("FMOE_B200_OVERLAP_SMS", "0"))
            # the experts' last GEMM (and the input-gradient GEMM of their first layer) stores its rows
            # straight into the token-side buffers of their owners: no gather pass afterwards
            # (not when someone else may look at the experts' raw output: a hook on the module, or a subclass
            # with its own expert_fn -- that tensor is never written in this form)
            plain_call = getattr(expert_fn, "__func__", None) is FMoE.expert_fn
            hooked = bool(experts._forward_hooks) or bool(getattr(experts, "_forward_hooks_with_kwargs", None))
            fused_gather = plain_call and not hooked and os.environ.get("FMOE_B200_FUSED_GATHER", "1") == "1"
        # the scatters' pushes pick (forward) or pick and scale (backward) their rows themselves
        fused_scatter = overlap == 0 and os.environ.get("FMOE_B200_FUSED_SCATTER", "1") == "1"
        # ... and the experts' first GEMM (backward: the second layer's input-gradient GEMM) moves them itself
        fused_push = fused_gather and fused_scatter and os.environ.get("FMOE_B200_FUSED_PUSH", "0") == "1"
        exch = PlannedExchange(routing.plan, routing.n_recv, world_size, overlap_sms=overlap, token_rows=routing.n_rows,
                               fused_gather=fused_gather, fused_scatter=fused_scatter, fused_push=fused_push)
        n_rows = routing.n_rows
        x = MOEScatterFused.apply(inp, routing.pos, routing.inv, top_k, n_rows, exch)
        x = expert_fn(x, [[experts]], ExpertCounts(routing.own_offsets_dev, exchange=exch), num_expert)
    else:
        shadows = {} if shadows is None else shadows
        if no_policy:
            # No shadowing: every row goes to its expert's owner; nothing else to plan on the host.
            stored, any_shadow = _no_shadow_flags(world_size, num_expert), False
            if fused:
                fwd_count = ExpertCounts(routing.own_offsets_dev, routing.own_counts)
            else:
                fwd_count = torch.zeros(world_size, num_expert, dtype=torch.int64)
                fwd_count[routing.rank] = routing.own_counts
                fwd_count = fwd_count.reshape(-1)
            fwd_batch_size = routing.n_recv
            models = [[] for _ in range(world_size)]
            models[routing.rank] = [experts] if fused else experts
        else:
            stored, workers = _shadow_plan(policy_fn, routing, experts, num_expert, world_size,
                                           inp.shape[1], fused, shadows)
            any_shadow = bool(workers.any())
            fwd_count = cached_count_host(routing.lec.clone(), routing.gec.clone(), stored, routing.rank,
                                          num_expert, world_size)
            fwd_batch_size = int(fwd_count.sum())
            models = [[] for _ in range(world_size)]
            for j in range(world_size):
                if j == routing.rank:
                    models[j] = [experts] if fused else experts
                elif bool(workers[j]):
                    models[j] = [shadows[j]] if fused else shadows[j]
        if any_shadow:
            inp = MOECache.apply(inp, workers, experts, shadows, world_size, routing.rank)
        exch = Exchange(routing.lec, routing.gec, stored.reshape(-1), fwd_batch_size, world_size,
                        table=routing.aec)
        n_rows = routing.n_rows
        if enable_fuse:
            from .fused_functions import MOEForward, fused_activation
            flat = [p for node in models if node for p in node[0].parameters()]
            x = MOEForward.apply(inp, models, routing, top_k, exch, n_rows, fused_activation(experts), *flat)
            exch = None
        else:
            x = MOEScatterFused.apply(inp, routing.pos, routing.inv, top_k, n_rows, exch, routing.early)
            x = expert_fn(x, models, fwd_count, num_expert)

    if gate_score is not None:
        pos = routing.pos if getattr(exch, "fused_scatter", False) else None
        out = MOEGatherCombine.apply(x, routing.inv, gate_score.reshape(n_tokens, top_k), n_rows, exch, pos)
    else:
        ones = torch.ones(n_tokens * top_k, 1, dtype=x.dtype, device=x.device)
        out = MOEGatherCombine.apply(x, routing.inv, ones, n_rows, exch)
    return out, stored


class FMoE(nn.Module):
    r"""General MoE layer (fmoe/layers.py:151-326).

    * ``num_expert``: experts on **each** worker; ``world_size``: workers holding
      different experts.
    * ``mp_group``: group whose members hold identical input; the input is sliced
      across it and the output all-gathered.
    * ``top_k``: experts per token; ``gate``: a gate class of ``fastermoe_b200.gates``.
    * ``expert``: a module class (or list of classes) instantiated per expert;
      when None the subclass provides one fused ``self.experts`` module.
    * ``policy_fn``: shadowing policy (see transformer._gen_policy).
    * ``enable_fuse`` / env ``FMOE_ENABLE_FUSE=1``: smart schedule.
    """

    def __init__(self, num_expert=32, d_model=1024, world_size=1, mp_group=None, moe_group=None, top_k=2,
                 gate=NaiveGate, expert=None, gate_hook=None, policy_fn=None, mask=None, mask_dict=None,
                 enable_fuse=False):
        super().__init__()
        self.num_expert, self.d_model, self.world_size = num_expert, d_model, world_size
        self.mp_group = mp_group
        if mp_group is None:
            self.mp_size, self.mp_rank = 1, 0
        else:
            self.mp_size, self.mp_rank = mp_group.size(), mp_group.rank()
        self.top_k = top_k
        if isinstance(expert, list):
            self.experts = nn.ModuleList([e(d_model) for e in expert])
            self.experts_fused = False
            self.num_expert = num_expert = len(expert)
        elif expert is not None:
            self.experts = nn.ModuleList([expert(d_model) for _ in range(num_expert)])
            self.experts_fused = False
        else:
            self.experts_fused = True
        self.gate = gate(d_model, num_expert, world_size, top_k)
        if hasattr(self.gate, "stored_models"):
            self.gate.policy_fn = policy_fn
        self.gate_hook, self.mask, self.mask_dict, self.moe_group = gate_hook, mask, mask_dict, moe_group
        if os.environ.get("FMOE_ENABLE_FUSE", "0") == "1":
            enable_fuse = True
        self.enable_fuse = enable_fuse
        if enable_fuse:
            assert self.experts_fused
        self.policy_fn = policy_fn
        self._shadows = {}

    def expert_fn(self, inp, models, fwd_expert_count, num_expert):
        r"""Runs the experts over a buffer laid out worker by worker, expert by expert
        (fmoe/layers.py:222-255).  ``models[j]`` holds worker j's experts (own or
        shadowed) or is empty."""
        if isinstance(fwd_expert_count, ExpertCounts) and self.experts_fused:
            present = [m for m in models if m]
            if len(present) == 1:
                return present[0][0](inp, fwd_expert_count)
        counts_all = (fwd_expert_count.host_counts() if isinstance(fwd_expert_count, ExpertCounts)
                      else fwd_expert_count.cpu()).view(-1, num_expert)
        res, ptr = [], 0
        for j in range(counts_all.shape[0]):
            counts = counts_all[j]
            size = int(counts.sum())
            node_inp = inp[ptr:ptr + size]
            ptr += size
            experts = models[j]
            if not experts:
                if size:
                    raise ValueError(f"worker {j} has no experts here but {size} rows were routed to it")
                continue
            if self.experts_fused:
                if size:
                    res.append(experts[0](node_inp, counts))
                continue
            base = 0
            for i in range(self.num_expert):
                n = int(counts[i])
                res.append(experts[i](node_inp[base:base + n]))
                base += n
        if ptr < inp.shape[0]:
            # Rows past the routed ones exist only at world_size 1 (one slot per gate entry).
            res.append(inp.new_zeros((inp.shape[0] - ptr, res[0].shape[1] if res else inp.shape[1])))
        return torch.cat(res, dim=0) if res else inp.new_zeros((0, inp.shape[1]))

    def mark_parallel_comm(self, expert_dp_comm="none"):
        """Tags expert parameters with ``expert_dp_comm`` and gate parameters with 'moe'."""
        if self.experts is not None:
            if isinstance(self.experts, list):
                for e in self.experts:
                    mark_module_parallel_comm(e, expert_dp_comm)
            else:
                mark_module_parallel_comm(self.experts, expert_dp_comm)
        mark_module_parallel_comm(self.gate, "moe")

    def check_status(self, device=None):
        """Raises RuntimeError when a kernel of the library reported trouble on ``device`` since the last
        check: a bounded wait that expired (a peer did not deliver: that step's results are incomplete),
        more rows routed to a GPU than its buffers hold, or clamped segment offsets.  Waits for the
        queued work; call it where the training loop synchronises anyway (e.g. after reading the loss).
        With FMOE_B200_CHECK_STATUS=1 every forward starts with this check (of the previous step)."""
        fmoe_cuda.check_status(device)

    def forward(self, inp):
        r"""gate -> route -> experts -> weighted sum of the top-k expert outputs."""
        if os.environ.get("FMOE_B200_CHECK_STATUS", "0") == "1" and inp.is_cuda:
            self.check_status(inp.device)
        if self.world_size > 1:
            ensure_comm(inp, self.moe_group)
        if self.mp_size > 1:
            inp = Slice.apply(inp, self.mp_rank, self.mp_size, self.mp_group)

        gate_top_k_idx, gate_score = self.gate(inp)
        if self.gate_hook is not None:
            self.gate_hook(gate_top_k_idx, gate_score, None)

        masked = self.mask is not None and self.mask_dict is not None
        if masked:
            mask = self.mask.view(-1)
            inp = inp[mask == 0, :]
            gate_top_k_idx = gate_top_k_idx[mask == 0, :]

        fwd, _ = _fmoe_general_global_forward(
            inp, gate_top_k_idx.contiguous(), self.expert_fn, self.policy_fn, self.experts,
            self.num_expert, self.world_size, self.experts_fused, self.enable_fuse,
            gate_score=None if masked else gate_score, shadows=self._shadows)

        if masked:
            fwd = fwd.view(-1, self.top_k, self.d_model)
            x = torch.zeros(mask.shape[0], self.top_k, self.d_model, device=fwd.device, dtype=fwd.dtype)
            x[mask == 0] = fwd
            for k, v in self.mask_dict.items():
                x[mask == k] = v
            gate_score = gate_score.view(x.shape[0], 1, self.top_k)
            x = torch.bmm(gate_score, x).reshape(-1, self.d_model)
        else:
            x = fwd

        if self.mp_size > 1:
            x = AllGather.apply(x, self.mp_rank, self.mp_size, self.mp_group)
        return x
