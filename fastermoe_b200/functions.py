r"""Autograd glue between the MoE layer and the CUDA operators.

Mirrors the public names of the reference's ``fmoe/functions.py`` (count_by_gate,
prepare_forward, ensure_comm, MOECache, MOEScatter, MOELinear, MOEGather,
AllGather, Slice) and adds the fused forms the layer uses on its fast path.

Where the reference copies five count vectors to the host per forward
(fmoe/functions.py:64-68), this module needs none at world_size 1 and one
(the all-gathered count table, a few KB) otherwise.
"""
import numpy as np
import torch
from torch.autograd import Function

from . import fmoe_cuda
from . import _lib
from .utils import get_torch_default_comm


class ExpertCounts:
    """Rows per expert for a grouped expert call.

    ``offsets`` is a device int64 [E+1] exclusive prefix sum; ``counts_cpu`` the
    per-expert counts on the host when they are known there (multi-GPU runs),
    else ``None``.  Accepted wherever the reference passes ``fwd_expert_count``.
    """

    def __init__(self, offsets, counts_cpu=None, exchange=None):
        self.offsets = offsets
        self.counts_cpu = counts_cpu
        self.exchange = exchange     # PlannedExchange whose scatter fills the rows (may still be arriving)

    @staticmethod
    def wrap(counts, device):
        if isinstance(counts, ExpertCounts):
            return counts
        cpu = counts if not counts.is_cuda else None
        return ExpertCounts(fmoe_cuda.offsets_from_counts(counts, device), cpu)

    def host_counts(self):
        """Counts as a CPU tensor (copies from the device, with a sync, if unknown)."""
        if self.counts_cpu is None:
            off = self.offsets.cpu()
            self.counts_cpu = off[1:] - off[:-1]
        return self.counts_cpu


def ensure_comm(t, comm):
    """Creates the expert-parallel NCCL communicator of t's device (fmoe/functions.py:14-17)."""
    if comm is None:
        comm = get_torch_default_comm()
    fmoe_cuda.ensure_nccl(comm, t)


def count_by_gate(gate, num_expert, world_size, require_pos=True):
    """Same contract as fmoe/functions.py:19-42.

    Returns ``(pos, local_expert_count, all_expert_count, global_expert_count,
    all_global_expert_count)`` as device tensors; ``pos`` has exactly as many
    entries as gate entries that are not -1 (which costs one host read, as in
    the reference).
    """
    with torch.no_grad():
        n_tot = num_expert * world_size
        if require_pos:
            lec, off, pos_full, _ = fmoe_cuda.count_and_pos(gate.reshape(-1), n_tot, want_inv=False)
        else:
            lec32 = torch.zeros(n_tot, device=gate.device, dtype=torch.int32)
            fmoe_cuda.expert_count(gate.reshape(-1), lec32)
            lec = lec32.long()
        if world_size > 1:
            aec, agec, gec = fmoe_cuda.expert_exchange(lec, num_expert, world_size)
        else:
            gec = lec
            aec = lec
            agec = gec
        pos = None
        if require_pos:
            pos = pos_full[: int(off[-1].item())]
    return pos, lec, aec, gec, agec


class Routing:
    """Everything the layer derives from the gate indices for one forward."""
    __slots__ = ("pos", "inv", "lec_dev", "offsets_dev", "own_offsets_dev", "n_rows", "n_recv", "lec", "gec",
                 "own_counts", "_aec", "_agec", "rank", "early", "plan")

    @property
    def aec(self):
        """all_expert_count [W, W, E] on the host: [source worker, destination worker, expert]."""
        return self._aec

    @property
    def agec(self):
        """all_global_expert_count [W, W, E] on the host (built on first use: only a shadowing policy reads it)."""
        if self._agec is None and self._aec is not None:
            self._agec = self._aec.transpose(0, 1).contiguous()
        return self._agec


def route(gate, num_expert, world_size, before_wait=None, cap_rows=0):
    """Bucketing + count exchange with at most one device-to-host copy, and none at all with
    ``cap_rows`` > 0: the counts are then swapped through peer memory and the exchange plan is built
    on the device (``routing.plan``); the expert-side buffers get ``cap_rows`` rows, the offsets of
    this worker's experts stay on the device (``own_offsets_dev``), and ``lec``/``gec``/``aec`` are
    not available on the host.

    ``before_wait(routing)``, if given, is called right before the host waits for
    the count table (world_size > 1 only) with ``pos``/``inv`` already queued; what
    it returns is kept in ``routing.early``.  The layer uses it to queue the local
    scatter, which needs no counts, so that the GPU works through the wait.

    Everything that needs only device data (the positions, the offsets of this
    worker's experts in the received buffer) is queued before the host waits for
    the count table, and the host-side slicing after the wait is a few numpy
    views, so the GPU idles as briefly as possible around the one sync."""
    r = Routing()
    r._aec = r._agec = r.early = r.plan = None
    with torch.no_grad():
        flat = gate.reshape(-1)
        n_tot = num_expert * world_size
        r.lec_dev, r.offsets_dev, r.pos, r.inv = fmoe_cuda.count_and_pos(flat, n_tot)
        if world_size == 1:
            r.n_rows = flat.numel()
            r.lec = r.gec = r.own_offsets_dev = r.own_counts = None
            r.rank = 0
            return r
        if cap_rows > 0:
            r.plan = fmoe_cuda.peer_plan_exchange(r.lec_dev, None, cap_rows, num_expert)
        if r.plan is not None:
            r.rank, _ = fmoe_cuda.comm_rank(gate.device)
            r.own_offsets_dev = r.plan.own_offsets
            r.n_rows, r.n_recv = flat.numel(), int(cap_rows)
            r.lec = r.gec = r.own_counts = None
            return r
        aec, _, _ = fmoe_cuda.expert_exchange(r.lec_dev, num_expert, world_size)
        r.rank, _ = fmoe_cuda.comm_rank(gate.device)
        # rows of this worker's expert e sit together in the received buffer (all sources)
        own = aec[:, r.rank, :].sum(dim=0)
        r.own_offsets_dev = torch.zeros(num_expert + 1, dtype=torch.int64, device=gate.device)
        torch.cumsum(own, 0, out=r.own_offsets_dev[1:])
        if before_wait is not None:
            r.early = before_wait(r)
        r._aec = aec.cpu()                      # the one sync of the forward pass
        table = r._aec.numpy()
        lec = table[r.rank].reshape(-1)
        gec = np.ascontiguousarray(table[:, r.rank, :]).reshape(-1)
        r.n_rows = int(lec.sum())
        r.n_recv = int(gec.sum())
        r.lec = torch.from_numpy(lec)
        r.gec = torch.from_numpy(gec)
        r.own_counts = torch.from_numpy(gec.reshape(world_size, num_expert).sum(axis=0))
    return r


def prepare_forward(gate, num_expert, world_size):
    """Same return tuple as fmoe/functions.py:45-69 (count tensors on the CPU)."""
    r = route(gate, num_expert, world_size)
    if world_size == 1:
        lec = r.lec_dev.cpu()
        n = int(lec.sum())
        return r.pos[:n], lec, lec, lec, lec, lec.view(1, num_expert).sum(dim=0)
    fwd = r.gec.view(world_size, num_expert).sum(dim=0)
    return r.pos[: r.n_rows], r.lec, r.gec, r.aec.reshape(-1), r.agec.reshape(-1), fwd


def _local_scatter(inp, pos):
    """out[i] = inp[pos[i]] (fmoe/functions.py:72-74)."""
    return fmoe_cuda.local_scatter(inp.contiguous(), pos.contiguous())


def _local_gather(inp, pos, out_batch_size, maybe_overlap=True):
    """zeros(out_batch_size, d) then index_add_/index_copy_ at pos (fmoe/functions.py:77-84)."""
    if maybe_overlap:
        return fmoe_cuda.local_gather_add(inp.contiguous(), pos.contiguous(), out_batch_size)
    return fmoe_cuda.local_gather(inp.contiguous(), pos.contiguous(), out_batch_size)


def cached_count_host(lec, gec, stored, rank, num_expert, world_size):
    """Host mirror of generate_cached_count (cuda/global_exchange.cu:189-195)."""
    lec = lec.view(world_size, num_expert)
    gec = gec.view(world_size, num_expert)
    stored = stored.view(world_size, num_expert)
    out = lec * stored.to(lec.dtype)
    out[rank] += (gec * (~stored[rank]).to(gec.dtype)).sum(dim=0)
    return out.reshape(-1)


class MOECache(Function):
    """Dynamic shadowing: fetch the parameters of overloaded workers' experts so
    that their tokens are computed locally (fmoe/functions.py:121-194).

    ``shadows`` maps worker index -> module that holds the fetched copy.  The
    modules persist between calls (the reference deep-copies the experts every
    forward); parameters and gradients are exchanged tensor by tensor, so no
    flattened copies are made.
    """

    @staticmethod
    def forward(ctx, inp, stored_workers, experts, shadows, world_size, rank):
        ctx.stored_workers = stored_workers
        ctx.experts, ctx.shadows, ctx.world_size, ctx.rank = experts, shadows, world_size, rank
        flags = stored_workers.to(torch.bool)
        with torch.no_grad():
            local = list(experts.parameters())
            for k, p in enumerate(local):
                remote = [[list(shadows[j].parameters())[k].data] if (bool(flags[j]) and j != rank) else []
                          for j in range(world_size)]
                fmoe_cuda.model_exchange(flags, [p.data], remote, 1, world_size)
        return inp.view_as(inp)

    @staticmethod
    def backward(ctx, grad_inp):
        flags = ctx.stored_workers.to(torch.bool)
        world_size, rank = ctx.world_size, ctx.rank
        local = list(ctx.experts.parameters())
        for k, p in enumerate(local):
            if bool(flags[rank]) and p.grad is None:
                p.grad = torch.zeros_like(p)
            remote = []
            for j in range(world_size):
                if bool(flags[j]) and j != rank:
                    q = list(ctx.shadows[j].parameters())[k]
                    if q.grad is None:
                        q.grad = torch.zeros_like(q)
                    remote.append([q.grad])
                else:
                    remote.append([])
            fmoe_cuda.gradient_exchange(flags, [p.grad] if bool(flags[rank]) else [p.data], remote, 1,
                                        world_size)
        for j in range(world_size):
            if bool(flags[j]) and j != rank:
                for q in ctx.shadows[j].parameters():
                    q.grad = None
        return grad_inp, None, None, None, None, None


class MOEScatter(Function):
    """Local scatter followed by the all-to-all-v (fmoe/functions.py:196-248).

    ``pos`` holds row indices into ``inp`` (the caller divides by top_k, as the
    reference's callers do).  The backward sums the k gradient rows of a token
    with ``index_add_``-equivalent semantics.
    """

    @staticmethod
    def forward(ctx, inp, pos, local_expert_count, global_expert_count, stored_models, fwd_batch_size,
                world_size):
        local_input_buf = _local_scatter(inp, pos)
        if world_size > 1:
            global_input_buf = fmoe_cuda.global_scatter(local_input_buf, local_expert_count,
                                                        global_expert_count, stored_models,
                                                        fwd_batch_size, world_size)
        else:
            global_input_buf = local_input_buf
        ctx.moe_args = inp.shape[0], pos.shape[0], world_size
        ctx.save_for_backward(pos, local_expert_count, global_expert_count, stored_models)
        return global_input_buf

    @staticmethod
    def backward(ctx, global_grad_in):
        pos, lec, gec, stored = ctx.saved_tensors
        inp_batch_size, buf_batch_size, world_size = ctx.moe_args
        global_grad_in = global_grad_in.contiguous()
        if world_size > 1:
            local_grad_in = fmoe_cuda.global_gather(global_grad_in, lec, gec, stored, buf_batch_size,
                                                    world_size)
        else:
            local_grad_in = global_grad_in
        grad_in = _local_gather(local_grad_in, pos, inp_batch_size)
        return grad_in, None, None, None, None, None, None


class MOEGather(Function):
    """All-to-all-v back followed by the local gather (fmoe/functions.py:278-330)."""

    @staticmethod
    def forward(ctx, global_output_buf, pos, local_expert_count, global_expert_count, stored_models,
                local_batch_size, world_size):
        global_output_buf = global_output_buf.contiguous()
        if world_size > 1:
            local_output_buf = fmoe_cuda.global_gather(global_output_buf, local_expert_count,
                                                       global_expert_count, stored_models, pos.shape[0],
                                                       world_size)
        else:
            local_output_buf = global_output_buf
        output = _local_gather(local_output_buf, pos, local_batch_size, maybe_overlap=False)
        ctx.moe_args = (global_output_buf.shape[0], world_size)
        ctx.save_for_backward(pos, local_expert_count, global_expert_count, stored_models)
        return output

    @staticmethod
    def backward(ctx, grad_out):
        pos, lec, gec, stored = ctx.saved_tensors
        fwd_batch_size, world_size = ctx.moe_args
        grad_out_buf = _local_scatter(grad_out.contiguous(), pos)
        if world_size > 1:
            global_grad_out_buf = fmoe_cuda.global_scatter(grad_out_buf, lec, gec, stored, fwd_batch_size,
                                                           world_size)
        else:
            global_grad_out_buf = grad_out_buf
        return global_grad_out_buf, None, None, None, None, None, None


class MOELinear(Function):
    """Grouped expert linear layer (fmoe/functions.py:251-275)."""

    @staticmethod
    def forward(ctx, global_input_buf, fwd_expert_count, weight, bias=None):
        counts = ExpertCounts.wrap(fwd_expert_count, global_input_buf.device)
        x = global_input_buf.contiguous()
        y, _ = fmoe_cuda.linear_forward_act(x, counts.offsets, weight.contiguous(), bias, _lib.ACT_NONE)
        ctx.save_for_backward(x, counts.offsets, weight, bias)
        return y

    @staticmethod
    def backward(ctx, grad_out):
        x, offsets, weight, bias = ctx.saved_tensors
        gx, gw, gb = fmoe_cuda.linear_backward_act(grad_out.contiguous(), x, offsets, weight.contiguous(),
                                                   None, _lib.ACT_NONE, need_bias=bias is not None,
                                                   need_input_grad=ctx.needs_input_grad[0])
        return gx, None, gw, gb


# ---------------------------------------------------------------------------
# Fused forms used by the layer's fast path
# ---------------------------------------------------------------------------

class MOEScatterFused(Function):
    """Scatter with the division by top_k and the k-way gradient sum done in the
    kernels: forward ``buf[i] = inp[pos[i] // k]``, backward
    ``grad_inp[t] = sum_j grad_buf[inv[t*k+j]]`` in a fixed order.  With
    world_size > 1 the all-to-all-v follows / precedes."""

    @staticmethod
    def forward(ctx, inp, pos, inv, top_k, n_rows, exch, scattered=None):
        inp = inp.contiguous()
        ctx.exch, ctx.top_k, ctx.n_tokens, ctx.n_rows = exch, top_k, inp.shape[0], n_rows
        ctx.save_for_backward(inv)
        if scattered is None and exch is not None and hasattr(exch, "scatter_rows"):
            # the exchange's push reads inp[pos[i] // k] itself: no token-side copy in between
            buf = exch.scatter_rows(inp, pos, top_k, None, exch.fwd_batch_size)
            if buf is not None:
                return buf
        # `scattered`: the same local scatter, queued earlier by the caller (at least n_rows rows)
        buf = scattered if scattered is not None else fmoe_cuda.local_scatter(inp, pos, pos_div=top_k, n_rows=n_rows)
        if exch is not None:
            buf = exch.scatter(buf, exch.fwd_batch_size)
        return buf

    @staticmethod
    def backward(ctx, grad_buf):
        (inv,) = ctx.saved_tensors
        grad_buf = grad_buf.contiguous()
        exch = ctx.exch
        if exch is not None:
            grad_buf = exch.gather(grad_buf, ctx.n_rows)
        grad_inp = fmoe_cuda.local_gather_sum(grad_buf, inv, ctx.n_tokens, ctx.top_k)
        return grad_inp, None, None, None, None, None, None


class MOEGatherCombine(Function):
    """Gather fused with the gate-score combine (fmoe/layers.py:319-322):
    ``out[t] = sum_j score[t,j] * buf[inv[t*k+j]]``; rows of pruned entries
    contribute zero, as the zero rows of the reference's ``_local_gather`` do."""

    @staticmethod
    def forward(ctx, buf, inv, score, n_rows, exch, pos=None):
        """``pos`` (the inverse of ``inv``: pos[i] = flat gate entry of token-side row i), when given,
        lets the backward's exchange produce its rows on the way."""
        buf = buf.contiguous()
        ctx.exch, ctx.global_rows = exch, buf.shape[0]
        if exch is not None:
            buf = exch.gather(buf, n_rows)
        score_c = score.contiguous().to(buf.dtype)
        ctx.save_for_backward(buf, inv, score_c, pos)
        ctx.score_dtype = score.dtype
        return fmoe_cuda.combine_forward(buf, inv, score_c)

    @staticmethod
    def backward(ctx, grad_out):
        buf, inv, score, pos = ctx.saved_tensors
        exch = ctx.exch
        grad_out = grad_out.contiguous()
        grad_buf = None
        if pos is not None and exch is not None and hasattr(exch, "scatter_rows"):
            # grad_buf[i] = score[pos[i]] * grad_out[pos[i] // k] is formed by the push itself
            grad_buf = exch.scatter_rows(grad_out, pos, score.shape[1], score, ctx.global_rows)
        if grad_buf is not None:
            _, grad_score = fmoe_cuda.combine_backward(grad_out, buf, inv, score, need_score_grad=ctx.needs_input_grad[2],
                                                       need_buf_grad=False)
        else:
            grad_buf, grad_score = fmoe_cuda.combine_backward(grad_out, buf, inv, score,
                                                              need_score_grad=ctx.needs_input_grad[2])
            if exch is not None:
                grad_buf = exch.scatter(grad_buf, ctx.global_rows)
        if grad_score is not None:
            grad_score = grad_score.to(ctx.score_dtype)
        return grad_buf, None, grad_score, None, None, None


class Exchange:
    """Host-side description of one layer call's all-to-all-v.

    ``table`` is the all-gathered count table [W, W, E] on the host (or None); with
    it the rows travel by direct stores into the peers' memory when the library
    has that form enabled, else over NCCL."""
    __slots__ = ("lec", "gec", "stored", "fwd_batch_size", "world_size", "table", "num_expert")

    def __init__(self, lec, gec, stored, fwd_batch_size, world_size, table=None):
        self.lec, self.gec, self.stored = lec, gec, stored
        self.fwd_batch_size, self.world_size = fwd_batch_size, world_size
        self.table = table.reshape(-1) if table is not None else None
        self.num_expert = lec.numel() // world_size

    def scatter(self, buf, out_rows):
        """Token-side rows -> expert-side rows on the experts' owners."""
        if self.table is not None:
            out = fmoe_cuda.peer_global_scatter(buf, self.table, self.stored, out_rows, self.num_expert,
                                                self.world_size)
            if out is not None:
                return out
        return fmoe_cuda.global_scatter(buf, self.lec, self.gec, self.stored, out_rows, self.world_size)

    def gather(self, buf, out_rows):
        """Expert-side rows -> token-side rows on the tokens' owners."""
        if self.table is not None:
            out = fmoe_cuda.peer_global_gather(buf, self.table, self.stored, out_rows, self.num_expert,
                                               self.world_size)
            if out is not None:
                return out
        return fmoe_cuda.global_gather(buf, self.lec, self.gec, self.stored, out_rows, self.world_size)


_phase_hook = None


def set_phase_hook(fn):
    """``fn(name)`` is called on the host at points of a layer call that other traffic may want to
    avoid or to follow.  So far: ``"scatter_done"`` right after a scatter of the device-planned
    exchange has been queued on the current stream (its kernels store into the peers' memory; a
    host-to-device copy that runs beside them slows them down, so an input pipeline can record an
    event here -- an ``external`` one inside a CUDA graph capture -- and start its copy of the next
    batch behind it).  ``None`` removes the hook."""
    global _phase_hook
    _phase_hook = fn


def _phase(name):
    if _phase_hook is not None:
        _phase_hook(name)


class PlannedExchange:
    """One layer call's all-to-all-v driven by a plan that lives on the device (fmoe_cuda.PeerPlan):
    the host knows neither the counts nor how many rows arrive; ``fwd_batch_size`` is the capacity
    of the expert-side buffers."""
    __slots__ = ("plan", "fwd_batch_size", "world_size", "num_expert", "overlap_sms", "pending", "token_rows", "early",
                 "fused_gather", "fused_scatter", "fused_push")

    def __init__(self, plan, cap_rows, world_size, overlap_sms=0, token_rows=0, fused_gather=False, fused_scatter=False,
                 fused_push=False):
        self.plan, self.fwd_batch_size, self.world_size = plan, int(cap_rows), world_size
        self.num_expert = plan.n_expert
        # > 0: the pushes run on that many SMs beside the grouped GEMMs that read (scatter) or write
        # (gather) their rows; FusedExpertMLP takes part; the caller sets it only when that module follows
        self.overlap_sms, self.pending = int(overlap_sms), None
        self.token_rows = int(token_rows)       # rows of this rank's token-side buffers
        self.early = None                       # (expert-side tensor, token-side result, pending, fused into the GEMM) of a gather started early
        # the GEMM before a gather stores its rows straight into their owners' token-side buffers;
        # FusedExpertMLP takes part; its expert-side outputs are then placeholders nobody may read
        self.fused_gather = bool(fused_gather)
        # the push of a scatter picks (and scales) its rows itself instead of reading a token-side buffer
        # that a local scatter / the combine's backward would have to write first
        self.fused_scatter = bool(fused_scatter)
        # ... and the GEMM that consumes those rows is the kernel that moves them (its spare warps push while its
        # tensor-core warps work on the experts whose rows are complete); FusedExpertMLP takes part
        self.fused_push = bool(fused_push) and self.fused_scatter

    def flush(self):
        """Closes a scatter whose rows nobody waited for tile by tile, and a gather that was started early."""
        if self.pending is not None:
            self.pending.finish()
            self.pending = None
        if self.early is not None:
            self.early[2].finish()

    def begin_gather(self, buf, use):
        """Called right before the GEMM that writes ``buf`` (expert side): starts the gather that
        forwards its rows as experts complete.  Returns the handle for that GEMM, or None."""
        self.flush()
        self.early = None
        if self.fused_gather and self.token_rows > 0 and buf.dtype in (torch.bfloat16, torch.float16):
            out, pend = fmoe_cuda.peer_gather_fused_begin(buf, self.plan, self.token_rows)
            if pend is not None:
                self.early = (buf, out, pend, True)
                return pend
        if self.overlap_sms <= 0 or self.token_rows <= 0:
            return None
        out, pend = fmoe_cuda.peer_gather_planned_async(buf, self.plan, self.token_rows, self.overlap_sms, use)
        if pend is None:
            return None
        self.early = (buf, out, pend, False)
        return pend

    def take_pending(self):
        p, self.pending = self.pending, None
        return p

    def scatter(self, buf, out_rows):
        self.flush()
        if self.overlap_sms > 0:
            out, self.pending = fmoe_cuda.peer_scatter_planned_async(buf, self.plan, out_rows, self.overlap_sms)
            return out
        out = fmoe_cuda.peer_scatter_planned(buf, self.plan, out_rows)
        _phase("scatter_done")
        return out

    def scatter_rows(self, src, row_of, row_div, scale, out_rows):
        """scatter of the rows ``[scale[row_of[i]] *] src[row_of[i] // row_div]`` without storing them on
        the token side first; None when this exchange does not take that form."""
        if not self.fused_scatter or self.overlap_sms > 0:
            return None
        self.flush()
        if self.fused_push and src.dtype in (torch.bfloat16, torch.float16):
            out, pend = fmoe_cuda.peer_scatter_fused_begin(src, row_of, row_div, scale, self.plan, out_rows)
            if pend is not None:
                self.pending = pend          # the next grouped GEMM takes it (or flush() runs the exchange)
                return out
        out = fmoe_cuda.peer_scatter_planned_rows(src, row_of, row_div, scale, self.plan, out_rows)
        _phase("scatter_done")
        return out

    def gather(self, buf, out_rows):
        early, self.early = self.early, None
        if early is not None:
            early[2].finish()
            if early[0].data_ptr() == buf.data_ptr() and early[1].shape[0] == out_rows:
                return early[1]                 # the rows are already here
            if early[3]:
                raise RuntimeError("the expert-side output of this exchange was never stored (its GEMM sent the rows "
                                   "to their owners): gather the tensor that GEMM returned, or set FMOE_B200_FUSED_GATHER=0")
        self.flush()
        return fmoe_cuda.peer_gather_planned(buf, self.plan, out_rows)


_ACT_CODES = {"none": _lib.ACT_NONE, "relu": _lib.ACT_RELU, "gelu": _lib.ACT_GELU}


def activation_code(fn):
    """Maps a torch activation callable to the code of an activation the GEMM
    epilogue can apply, or None when it must run as a separate torch op."""
    import torch.nn.functional as F
    if fn is None:
        return _lib.ACT_NONE
    if isinstance(fn, torch.nn.ReLU) or fn in (F.relu, torch.relu):
        return _lib.ACT_RELU
    if isinstance(fn, torch.nn.GELU):
        return _lib.ACT_GELU if getattr(fn, "approximate", "none") == "none" else None
    if fn is F.gelu:
        return _lib.ACT_GELU
    return None


class FusedExpertMLP(Function):
    """Linear -> activation -> Linear over all experts of a worker, with bias and
    activation applied in the first GEMM's epilogue and the activation's backward
    applied in the epilogue of the second layer's input-gradient GEMM."""

    @staticmethod
    def forward(ctx, x, offsets, w1, b1, w2, b2, act, exch=None):
        """``exch``: the PlannedExchange whose scatter produced ``x`` (and whose scatter of the output
        gradient will produce ``grad_y``); a pending arrival of it is waited for tile by tile."""
        x = x.contiguous()
        want_pre = act == _lib.ACT_GELU and (x.requires_grad or w1.requires_grad)
        arrival = exch.take_pending() if exch is not None else None
        h, pre = fmoe_cuda.linear_forward_act(x, offsets, w1, b1, act, want_pre=want_pre, arrival=arrival)
        y = x.new_empty((x.shape[0], w2.shape[1]))
        # the gather that follows the experts starts now and forwards y expert by expert
        departure = exch.begin_gather(y, 0) if exch is not None and hasattr(exch, "begin_gather") else None
        fmoe_cuda.linear_forward_act(h, offsets, w2, b2, _lib.ACT_NONE, departure=departure, out=y)
        ctx.act, ctx.exch = act, exch
        ctx.has_bias = (b1 is not None, b2 is not None)
        ctx.save_for_backward(x, offsets, w1, w2, h, pre)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, offsets, w1, w2, h, pre = ctx.saved_tensors
        act = ctx.act
        arrival = ctx.exch.take_pending() if ctx.exch is not None else None
        act_pre = None
        if act == _lib.ACT_RELU:
            act_pre = h
        elif act == _lib.ACT_GELU:
            act_pre = pre
        # The first layer's bias gradient is the column sum of gh: the input-gradient kernel of the
        # second layer returns it, so the first layer's backward does not read gh once more for it.
        if ctx.has_bias[0]:
            gh, gw2, gb2, gb1 = fmoe_cuda.linear_backward_act(grad_y.contiguous(), h, offsets, w2, act_pre, act,
                                                              need_bias=ctx.has_bias[1], want_gx_colsum=True,
                                                              arrival=arrival)
        else:
            gh, gw2, gb2 = fmoe_cuda.linear_backward_act(grad_y.contiguous(), h, offsets, w2, act_pre, act,
                                                         need_bias=ctx.has_bias[1], arrival=arrival)
            gb1 = None
        gx, departure = None, None
        if ctx.needs_input_grad[0] and ctx.exch is not None and hasattr(ctx.exch, "begin_gather"):
            gx = x.new_empty(x.shape)
            departure = ctx.exch.begin_gather(gx, 1)        # the input gradient travels back as it is produced
        gx, gw1, _ = fmoe_cuda.linear_backward_act(gh, x, offsets, w1, None, _lib.ACT_NONE, need_bias=False,
                                                   need_input_grad=ctx.needs_input_grad[0], departure=departure,
                                                   grad_x=gx)
        return gx, None, gw1, gb1, gw2, gb2, None, None


class AllGather(Function):
    """All-gather along dim 0 over ``group`` with a slicing backward (fmoe/functions.py:333-352)."""

    @staticmethod
    def forward(ctx, inp, rank, world_size, group):
        tensor_list = [torch.empty_like(inp) for _ in range(world_size)]
        torch.distributed.all_gather(tensor_list, inp.contiguous(), group=group)
        ctx.args = rank, inp.shape[0]
        return torch.cat(tensor_list, dim=0)

    @staticmethod
    def backward(ctx, grad_out):
        rank, dim0 = ctx.args
        return grad_out[rank * dim0: (rank + 1) * dim0], None, None, None


class GateTopK(Function):
    """torch.topk(logits, k, largest=True) on the last dimension of a 2-D CUDA tensor with the
    library's kernels (fmoe/gates/naive_gate.py:31-34): returns (values, indices), descending."""

    @staticmethod
    def forward(ctx, logits, k):
        val, idx = fmoe_cuda.gate_topk(logits, k)
        ctx.n_expert = logits.shape[1]
        ctx.save_for_backward(idx)
        ctx.mark_non_differentiable(idx)
        return val, idx

    @staticmethod
    def backward(ctx, grad_val, _grad_idx):
        (idx,) = ctx.saved_tensors
        return fmoe_cuda.gate_topk_backward(grad_val, idx, ctx.n_expert), None


def gate_topk(logits, k):
    """Top-k over the last dimension with the library's kernel (CUDA tensors; k <= 8).  A CPU
    tensor, which no GPU code path produces, is answered by torch.topk.  Returns (values, indices)."""
    if logits.is_cuda:
        if k > 8 or logits.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise RuntimeError(f"gate_topk: k={k}, dtype={logits.dtype} is outside what the kernel takes "
                               "(k <= 8; float32, float16, bfloat16)")
        lead = logits.shape[:-1]
        val, idx = GateTopK.apply(logits.reshape(-1, logits.shape[-1]), k)
        return val.reshape(*lead, k), idx.reshape(*lead, k)
    return torch.topk(logits, k=k, dim=-1, largest=True, sorted=True)       # CPU tensors: module set-up and tests only


class Slice(Function):
    """Keeps this rank's slice of dim 0; backward all-gathers (fmoe/functions.py:355-375)."""

    @staticmethod
    def forward(ctx, inp, rank, world_size, group):
        local = inp.shape[0] // world_size
        start = local * rank
        ctx.args = world_size, group
        return inp[start: min(start + local, inp.shape[0])]

    @staticmethod
    def backward(ctx, grad_out):
        world_size, group = ctx.args
        tensor_list = [torch.empty_like(grad_out) for _ in range(world_size)]
        torch.distributed.all_gather(tensor_list, grad_out.contiguous(), group=group)
        return torch.cat(tensor_list, dim=0), None, None, None
