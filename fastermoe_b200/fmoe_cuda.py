r"""Drop-in module for the reference's ``fmoe_cuda`` extension.

Every function registered by the reference's pybind11 module
(cuda/fmoe_cuda.cpp:105-130) exists here under the same name, with the same
positional arguments, in-place side effects and return values, and forwards to
``libfmoe_b200.so`` through its C ABI (include/fmoe_b200.h).  Outputs are
allocated with torch, work is queued on torch's current stream, and a failure
raises ``RuntimeError`` (the reference exits the process).

Two deliberate differences from the reference: operators do not block the
host, and ``linear_forward`` / ``linear_backward`` accept the expert-count
vector on either the CPU (as the reference requires) or the GPU.

Functions past the "extended operators" marker have no counterpart in the
reference's extension; they are the fused forms the layer in this package uses
(bucketing in one call, permutation kernels, gate-score combine, activation
fused into the expert GEMMs).
"""
import ctypes
import os
import threading

import torch

from . import _lib
from ._lib import lib, check

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


# Kernel launches issued by one call of each C entry point (for launch accounting).
_KERNELS = {"expert_count": 1, "assign_pos": 4, "count_and_pos": 4, "limit_by_capacity": 1,
            "prune_gate_by_capacity": 4, "local_scatter": 1, "local_gather": 3, "local_gather_inv": 1,
            "local_gather_sum": 1, "local_gather_add": 3, "combine_forward": 1, "combine_backward": 1, "linear_forward": 1,
            "linear_backward": 3, "expert_exchange": 2, "generate_cached_count": 1,
            "peer_scatter": 2, "peer_gather": 2, "peer_plan": 1}


class Profile:
    """Optional per-call accounting: number of library calls / kernel launches and,
    when ``timing`` is set, CUDA-event durations of each call on the current stream."""

    def __init__(self, timing=False):
        self.timing = timing
        self.calls = {}
        self.launches = 0
        self.events = []

    def durations_ms(self):
        """{op name: [ms per call]}; synchronises the device."""
        torch.cuda.synchronize()
        out = {}
        for name, a, b in self.events:
            out.setdefault(name, []).append(a.elapsed_time(b))
        return out


_profile = None


def set_profile(p):
    """Installs (or with None removes) a Profile that every operator call reports to."""
    global _profile
    _profile = p


def _check_or_unavailable(status, name):
    if status == _lib.PEER_UNAVAILABLE:
        return False
    check(status, name)
    return True


def _run(name, fn, *args, soft=False):
    """Calls the library; with ``soft`` a positive FMOE_PEER_UNAVAILABLE is returned as False."""
    chk = _check_or_unavailable if soft else check
    p = _profile
    if p is None:
        return chk(fn(*args), name)
    p.calls[name] = p.calls.get(name, 0) + 1
    p.launches += _KERNELS.get(name, 1)
    if p.timing:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        ok = chk(fn(*args), name)
        b.record()
        p.events.append((name, a, b))
        return ok
    return chk(fn(*args), name)


def set_gemm_form(name):
    """Forces the kernels of the grouped expert GEMM: "auto", "pair", "tc1" or "simt"."""
    check(lib.fmoe_gemm_set_form(_lib.GEMM_FORMS[name]), "gemm_set_form")


def set_gemm_sm_limit(n_sms):
    """Upper bound on the SMs the tensor-core GEMM grids occupy (0: all of them)."""
    check(lib.fmoe_gemm_set_sm_limit(int(n_sms)), "gemm_set_sm_limit")


def device_status(device=None):
    """The status word of ``device`` (0: no bounded wait expired, no offsets were clamped).
    Waits for the work queued on the device."""
    st = ctypes.c_int32(0)
    with torch.cuda.device(device):
        check(lib.fmoe_device_status(ctypes.byref(st)), "device_status")
    return st.value


def check_status(device=None):
    """Raises RuntimeError when a kernel of this library reported trouble since the last clear:
    an expired bounded wait (results of that step are incomplete) or clamped segment offsets."""
    v = device_status(device)
    if v:
        with torch.cuda.device(device):
            lib.fmoe_device_status_clear()
        what = []
        if v & 15:
            what.append({8: "segment offsets overshot the buffer and were clamped",
                         7: "misaligned shared memory"}.get(v & 15, f"tensor-core kernel wait {v & 15} expired"))
        if v & 16:
            what.append("a peer never announced where it receives rows")
        if v & 32:
            what.append("rows from a peer did not arrive in time")
        if v & 64:
            what.append("more rows were routed to a GPU than its expert-side buffers hold")
        raise RuntimeError(f"fastermoe_b200: device status {v}: " + "; ".join(what))


def _dtype_code(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise RuntimeError(f"fmoe_cuda: unsupported dtype {t.dtype} (float32, float16, bfloat16)") from None


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(device=None):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _check_cuda(*tensors):
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("fmoe_cuda: expected a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError("fmoe_cuda: expected a contiguous tensor")


def _scratch(nbytes, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


def _routing_scratch(n, n_expert, device):
    return _scratch(lib.fmoe_routing_scratch_bytes(n, n_expert), device)


# ---------------------------------------------------------------------------
# local_exchange: cuda/fmoe_cuda.cpp:48-54
# ---------------------------------------------------------------------------

def expert_count(gate_idx, expert_count):
    """Adds the histogram of ``gate_idx`` (int64, -1 ignored) into ``expert_count`` (int32)."""
    _check_cuda(gate_idx, expert_count)
    assert gate_idx.dtype == torch.int64 and expert_count.dtype == torch.int32
    with torch.cuda.device(gate_idx.device):
        _run("expert_count", lib.fmoe_expert_count, _ptr(gate_idx), _ptr(expert_count), gate_idx.numel(),
                                    expert_count.numel(), _stream())


def assign_pos(cum_count, gate, pos):
    """Fills ``pos`` with flat gate indices bucketed by expert; consumes ``cum_count``."""
    _check_cuda(cum_count, gate, pos)
    assert cum_count.dtype == torch.int32 and gate.dtype == torch.int64 and pos.dtype == torch.int64
    n, e = gate.numel(), cum_count.numel()
    with torch.cuda.device(gate.device):
        scratch = _routing_scratch(n, e, gate.device)
        _run("assign_pos", lib.fmoe_assign_pos, _ptr(cum_count), _ptr(gate), _ptr(pos), n, e, _ptr(scratch),
                                  _stream())


# ---------------------------------------------------------------------------
# balancing: cuda/fmoe_cuda.cpp:72-77
# ---------------------------------------------------------------------------

def limit_by_capacity(expert_count, capacity, n_expert, n_worker):
    """Returns the granted counts [W*E] int64; decrements ``capacity`` (int32 [E])."""
    _check_cuda(expert_count, capacity)
    assert expert_count.dtype == torch.int64 and capacity.dtype == torch.int32
    assert expert_count.numel() == n_expert * n_worker and capacity.numel() == n_expert
    out = torch.empty_like(expert_count)
    with torch.cuda.device(expert_count.device):
        _run("limit_by_capacity", lib.fmoe_limit_by_capacity, _ptr(expert_count), _ptr(capacity), _ptr(out), n_expert,
                                         n_worker, _stream())
    return out


def prune_gate_by_capacity(gate_idx, expert_count, n_expert, n_worker):
    """Returns a new gate tensor with entries beyond each expert's allowance set to -1."""
    _check_cuda(gate_idx, expert_count)
    assert gate_idx.dtype == torch.int64 and expert_count.dtype == torch.int32
    assert expert_count.numel() == n_expert * n_worker
    out = torch.empty_like(gate_idx)
    n, e = gate_idx.numel(), expert_count.numel()
    with torch.cuda.device(gate_idx.device):
        scratch = _routing_scratch(n, e, gate_idx.device)
        _run("prune_gate_by_capacity", lib.fmoe_prune_gate_by_capacity, _ptr(gate_idx), _ptr(out), _ptr(expert_count), n, e,
                                              _ptr(scratch), _stream())
    return out


# ---------------------------------------------------------------------------
# parallel_linear: cuda/fmoe_cuda.cpp:57-69
# ---------------------------------------------------------------------------

_offset_cache = {}
_offset_lock = threading.Lock()


def offsets_from_counts(expert_count, device):
    """Exclusive prefix sum (int64 [E+1], on ``device``) of a CPU or CUDA count vector."""
    if expert_count.is_cuda:
        off = torch.zeros(expert_count.numel() + 1, dtype=torch.int64, device=device)
        torch.cumsum(expert_count.reshape(-1).to(torch.int64), 0, out=off[1:])
        return off
    key = id(expert_count)
    with _offset_lock:
        hit = _offset_cache.get(key)
        if hit is not None and hit[0]() is expert_count and hit[1] == expert_count._version \
                and hit[2].device == device:
            return hit[2]
    ec = expert_count.reshape(-1).to(torch.int64)
    off = torch.zeros(ec.numel() + 1, dtype=torch.int64)
    torch.cumsum(ec, 0, out=off[1:])
    dev = off.to(device)
    import weakref
    with _offset_lock:
        if len(_offset_cache) > 64:
            _offset_cache.clear()
        _offset_cache[key] = (weakref.ref(expert_count), expert_count._version, dev)
    return dev


def _check_host_counts(expert_count, n_rows, what):
    """Counts that live on the host are checked against the buffer before anything is queued
    (counts on the device cannot be: the kernels clamp them instead and raise status code 8)."""
    if not expert_count.is_cuda:
        total = int(expert_count.sum())
        if total > n_rows or bool((expert_count < 0).any()):
            raise RuntimeError(f"{what}: expert_count sums to {total} but the buffer has only {n_rows} rows "
                               "(or a count is negative)")


def linear_forward(input_buf, expert_count, weight, bias=None):
    """Y[seg_e] = X[seg_e] @ W_e^T + b_e for every expert (cuda/parallel_linear.cu:5-49)."""
    _check_host_counts(expert_count, input_buf.shape[0], "linear_forward")
    off = offsets_from_counts(expert_count, input_buf.device)
    return linear_forward_act(input_buf, off, weight, bias, _lib.ACT_NONE)[0]


def linear_backward(grad_output_buf, input_buf, expert_count, weight, bias=None):
    """Returns [dX, dW, db] (cuda/parallel_linear.cu:52-94); db is returned even without bias."""
    _check_host_counts(expert_count, input_buf.shape[0], "linear_backward")
    off = offsets_from_counts(expert_count, input_buf.device)
    gx, gw, gb = linear_backward_act(grad_output_buf, input_buf, off, weight, None, _lib.ACT_NONE,
                                     need_bias=True)
    return [gx, gw, gb]


# ---------------------------------------------------------------------------
# global_exchange: cuda/fmoe_cuda.cpp:8-44
# ---------------------------------------------------------------------------

_comms = {}
_comm_lock = threading.Lock()


def _comm(device):
    c = _comms.get(device.index if device.index is not None else torch.cuda.current_device())
    if c is None:
        raise RuntimeError("fmoe_cuda: no communicator on this device; call ensure_nccl first")
    return c


def ensure_nccl(group, t):
    """Creates this device's expert-parallel communicator once (cuda/global_exchange.cu:107-119).

    ``group`` is a ``torch.distributed`` process group (``None`` = default group);
    it is only used to broadcast the 128-byte NCCL unique id from its rank 0.
    """
    import torch.distributed as dist
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    with _comm_lock:
        if dev in _comms:
            return
        rank = dist.get_rank(group)
        world = dist.get_world_size(group)
        ident = (ctypes.c_uint8 * 128)()
        if rank == 0:
            _run("comm_unique_id", lib.fmoe_comm_unique_id, ident)
        box = [bytes(ident)]
        src = dist.get_global_rank(group, 0) if group is not None else 0
        dist.broadcast_object_list(box, src=src, group=group)
        ident = (ctypes.c_uint8 * 128).from_buffer_copy(box[0])
        handle = ctypes.c_void_p()
        _run("comm_init", lib.fmoe_comm_init, ident, rank, world, dev, ctypes.byref(handle))
        _comms[dev] = handle
        # Token rows travel by direct stores into the peers' memory where the GPUs allow it
        # (FMOE_B200_PEER=0 keeps NCCL send/receive; FMOE_B200_PEER_SLOT_MB sizes the landing slots).
        if world > 1 and os.environ.get("FMOE_B200_PEER", "1") != "0":
            slot = int(os.environ.get("FMOE_B200_PEER_SLOT_MB", "256")) << 20
            pool = int(os.environ.get("FMOE_B200_PEER_POOL_MB", "2048")) << 20
            with torch.cuda.device(dev):
                _run("peer_enable", lib.fmoe_peer_enable, handle, slot, pool, _stream())


def peer_slot_bytes(device):
    """Bytes of one landing slot of the peer-memory exchange on ``device`` (0: the form is off)."""
    c = _comms.get(device.index if device.index is not None else torch.cuda.current_device())
    return int(lib.fmoe_peer_slot_bytes(c)) if c is not None else 0


def comm_rank(device):
    r, w = ctypes.c_int32(), ctypes.c_int32()
    _run("comm_rank", lib.fmoe_comm_rank, _comm(device), ctypes.byref(r), ctypes.byref(w))
    return r.value, w.value


def destroy_comms():
    """Destroys every communicator created by ensure_nccl (for orderly shutdown).  Tensors that were
    allocated from a receive pool must not be used afterwards: the pool's memory goes with it."""
    _recv_pools.clear()
    with _comm_lock:
        for h in _comms.values():
            lib.fmoe_comm_destroy(h)
        _comms.clear()


def expert_exchange(local_expert_count, n_expert, n_workers):
    """Returns [all_expert_count[W,W,E], all_global_expert_count[W,W,E], global_expert_count[W*E]]."""
    _check_cuda(local_expert_count)
    assert local_expert_count.dtype == torch.int64 and local_expert_count.numel() == n_expert * n_workers
    dev = local_expert_count.device
    aec = local_expert_count.new_empty((n_workers, n_workers, n_expert))
    agec = local_expert_count.new_empty((n_workers, n_workers, n_expert))
    gec = torch.empty_like(local_expert_count)
    with torch.cuda.device(dev):
        _run("expert_exchange", lib.fmoe_expert_exchange, _comm(dev), _ptr(local_expert_count), _ptr(aec), _ptr(agec),
                                       _ptr(gec), n_expert, n_workers, _stream())
    return [aec, agec, gec]


def _host_i64(t):
    if t.dtype == torch.int64 and not t.is_cuda and t.dim() == 1 and t.is_contiguous():
        return t
    t = t.detach()
    if t.is_cuda:
        t = t.cpu()
    return t.reshape(-1).to(torch.int64).contiguous()


def _host_flags(t):
    if t.dtype == torch.bool and not t.is_cuda and t.is_contiguous():
        # same bytes as uint8
        return t.view(torch.uint8).reshape(-1)
    t = t.detach()
    if t.is_cuda:
        t = t.cpu()
    return t.reshape(-1).to(torch.uint8).contiguous()


def _global_move(fn, name, buf, local_expert_count, global_expert_count, stored_models, batch_size,
                 n_workers):
    _check_cuda(buf)
    lec, gec, st = _host_i64(local_expert_count), _host_i64(global_expert_count), _host_flags(stored_models)
    n_expert = lec.numel() // n_workers
    out = buf.new_empty((batch_size, buf.shape[1]))
    row_bytes = buf.shape[1] * buf.element_size()
    # staging of the expert-side size: one send/receive per peer instead of one per (expert, peer)
    expert_rows = batch_size if name == "global_scatter" else buf.shape[0]
    # (allocated on every rank, also one that receives nothing: all ranks must use the same form)
    staging = (buf.new_empty((max(int(expert_rows), 1), buf.shape[1]))
               if os.environ.get("FMOE_B200_EXCHANGE") != "split" else None)
    with torch.cuda.device(buf.device):
        _run(name, fn, _comm(buf.device), _ptr(buf), _ptr(out), _ptr(lec), _ptr(gec), _ptr(st), buf.shape[0],
             batch_size, row_bytes, n_expert, n_workers, _ptr(staging), _stream())
    return out


def global_scatter(input_buf, local_expert_count, global_expert_count, stored_models, batch_size,
                   n_workers):
    """All-to-all-v of token rows to the experts' owners (cuda/global_exchange.cu:26-52)."""
    return _global_move(lib.fmoe_global_scatter, "global_scatter", input_buf, local_expert_count,
                        global_expert_count, stored_models, batch_size, n_workers)


def global_gather(output_buf, local_expert_count, global_expert_count, stored_models, batch_size,
                  n_workers):
    """Inverse of global_scatter (cuda/global_exchange.cu:54-80)."""
    return _global_move(lib.fmoe_global_gather, "global_gather", output_buf, local_expert_count,
                        global_expert_count, stored_models, batch_size, n_workers)


_recv_pools = {}


def _recv_pool(device):
    """torch memory pool over this device's peer-mapped receive pool (None: there is none).  Exchange
    outputs allocated from it are written by the peers directly; torch's caching allocator keeps
    managing their lifetime (it obtains its segments from fmoe_pool_alloc)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _recv_pools:
        pool = None
        c = _comms.get(idx)
        if c is not None and int(lib.fmoe_peer_pool_bytes(c)) > 0 and hasattr(torch.cuda, "MemPool"):
            alloc = torch.cuda.memory.CUDAPluggableAllocator(_lib.LIB_PATH, "fmoe_pool_alloc", "fmoe_pool_free")
            pool = (torch.cuda.MemPool(alloc.allocator()), alloc)      # the allocator object must stay alive
        _recv_pools[idx] = pool
    return _recv_pools[idx]


_pool_backoff = {}


class ReceiveArena:
    """Exchange outputs that are handed out again, in the same order, step after step: what a step
    that is captured in a CUDA graph needs (no allocation inside the capture, the same addresses at
    every replay).  The i-th request of a step gets the i-th buffer; buffers are created (from the
    receive pool when it has room) the first time a request is seen, which must happen outside a
    capture.  Only one step may be in flight: a buffer is reused as soon as the next step asks for it."""

    def __init__(self):
        self.bufs, self.next = [], 0

    def begin_step(self):
        self.next = 0

    def get(self, like, rows):
        i = self.next
        self.next += 1
        if i < len(self.bufs):
            b = self.bufs[i]
            if b.shape == (rows, like.shape[1]) and b.dtype == like.dtype and b.device == like.device:
                return b
            raise RuntimeError("ReceiveArena: the sequence of exchange buffers changed between steps "
                               f"(request {i}: {tuple(b.shape)} {b.dtype} before, {(rows, like.shape[1])} {like.dtype} now)")
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("ReceiveArena: a new exchange buffer was requested during graph capture; run the step "
                               "once before capturing")
        b = _recv_empty(like, rows, arena=False)
        self.bufs.append(b)
        return b


_arena = None


def set_receive_arena(arena):
    """Installs (None: removes) the ReceiveArena that serves the exchange outputs from now on."""
    global _arena
    _arena = arena


def _recv_empty(like, rows, arena=True):
    """Output buffer of a peer exchange: from the receive pool when there is one and it has room
    (after a refusal the pool is left alone for the next 64 requests: a failed request is slow)."""
    if arena and _arena is not None:
        return _arena.get(like, rows)
    pool = _recv_pool(like.device)
    if pool is not None:
        idx = like.device.index
        if _pool_backoff.get(idx, 0) > 0:
            _pool_backoff[idx] -= 1
        else:
            try:
                with torch.cuda.use_mem_pool(pool[0], device=like.device):
                    return like.new_empty((rows, like.shape[1]))
            except torch.OutOfMemoryError:
                _pool_backoff[idx] = 64
    return like.new_empty((rows, like.shape[1]))


def _peer_move(fn, name, buf, table, stored_models, batch_size, n_expert, n_workers):
    _check_cuda(buf)
    tab, st = _host_i64(table.reshape(-1)), _host_flags(stored_models)
    assert tab.numel() == n_workers * n_workers * n_expert
    out = _recv_empty(buf, batch_size)
    with torch.cuda.device(buf.device):
        ok = _run(name, fn, _comm(buf.device), _ptr(buf), _ptr(out), _ptr(tab), _ptr(st), buf.shape[0], batch_size,
                  buf.shape[1] * buf.element_size(), n_expert, n_workers, _stream(), soft=True)
    return out if ok else None


def peer_global_scatter(input_buf, all_expert_count, stored_models, batch_size, n_expert, n_workers):
    """global_scatter by direct stores into the peers' memory; ``all_expert_count`` is the host table
    [W, W, E] of expert_exchange.  Returns None (nothing queued, on every rank alike) when that form
    cannot serve the call; the caller then uses global_scatter."""
    return _peer_move(lib.fmoe_peer_global_scatter, "peer_scatter", input_buf, all_expert_count, stored_models,
                      batch_size, n_expert, n_workers)


def peer_global_gather(output_buf, all_expert_count, stored_models, batch_size, n_expert, n_workers):
    """Inverse of peer_global_scatter; same contract."""
    return _peer_move(lib.fmoe_peer_global_gather, "peer_gather", output_buf, all_expert_count, stored_models,
                      batch_size, n_expert, n_workers)


class PeerPlan:
    """Plan of a layer call's exchanges as the device built it (fmoe_peer_plan_exchange /
    fmoe_peer_plan_from_table).  ``own_offsets`` (int64 [E+1]) and ``table`` (int64 [W, W, E]) are
    views into the plan buffer on the device; nothing is copied to the host."""
    __slots__ = ("buf", "n_expert", "n_workers", "own_offsets", "table")

    def __init__(self, buf, n_expert, n_workers):
        self.buf, self.n_expert, self.n_workers = buf, n_expert, n_workers
        at = int(lib.fmoe_peer_plan_offsets_at(n_expert, n_workers))
        self.own_offsets = buf[at: at + 8 * (n_expert + 1)].view(torch.int64)
        at = int(lib.fmoe_peer_plan_table_at(n_expert, n_workers))
        n = n_workers * n_workers * n_expert
        self.table = buf[at: at + 8 * n].view(torch.int64).view(n_workers, n_workers, n_expert)

    def read(self, which):
        """Decodes list ``which`` (0 push/1 pull of global_scatter, 2/3 of global_gather) on the host:
        (segments [(dst_rank, src_row, dst_row, rows)], expert_rows, token_rows, overflow).  Synchronises."""
        host = self.buf.cpu().numpy()
        d = lib.fmoe_peer_plan_bytes(self.n_expert, self.n_workers)
        cap = (2 * self.n_workers - 1) * self.n_expert
        segs = (_lib.PeerSeg * cap)()
        n, er, tr, ov = ctypes.c_int32(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int32()
        check(lib.fmoe_peer_plan_read(host.ctypes.data, self.n_expert, self.n_workers, which,
                                      ctypes.cast(segs, ctypes.c_void_p), cap, ctypes.byref(n), ctypes.byref(er),
                                      ctypes.byref(tr), ctypes.byref(ov)), "peer_plan_read")
        assert d == host.size
        return ([(segs[i].dst_rank, segs[i].src_row, segs[i].dst_row, segs[i].rows) for i in range(n.value)],
                er.value, tr.value, ov.value)


def _plan_buffer(n_expert, n_workers, device):
    return torch.empty(int(lib.fmoe_peer_plan_bytes(n_expert, n_workers)), dtype=torch.uint8, device=device)


def peer_plan_exchange(local_expert_count, stored_models, cap_rows, n_expert):
    """Swaps the local expert counts (int64 [W*E], CUDA) with all peers through peer memory and builds
    the exchange plan on the device; nothing comes back to the host.  ``stored_models``: bool/uint8
    [W*E] CUDA tensor or None; ``cap_rows``: rows of this rank's expert-side buffers.  Returns a
    PeerPlan, or None when the peer-memory form is off."""
    _check_cuda(local_expert_count, stored_models)
    dev = local_expert_count.device
    assert local_expert_count.dtype == torch.int64
    rank, world = comm_rank(dev)
    assert local_expert_count.numel() == n_expert * world
    plan = _plan_buffer(n_expert, world, dev)
    st = stored_models.view(torch.uint8) if stored_models is not None and stored_models.dtype == torch.bool else stored_models
    with torch.cuda.device(dev):
        ok = _run("peer_plan", lib.fmoe_peer_plan_exchange, _comm(dev), _ptr(local_expert_count), _ptr(st), int(cap_rows),
                  _ptr(plan), n_expert, _stream(), soft=True)
    return PeerPlan(plan, n_expert, world) if ok else None


def peer_plan_from_table(all_expert_count, stored_models, rank, n_expert, n_workers, caps=None):
    """The same plan for ``rank`` from a full count table [W, W, E] that is already on the device."""
    _check_cuda(all_expert_count, stored_models, caps)
    dev = all_expert_count.device
    assert all_expert_count.dtype == torch.int64 and all_expert_count.numel() == n_workers * n_workers * n_expert
    plan = _plan_buffer(n_expert, n_workers, dev)
    st = stored_models.view(torch.uint8) if stored_models is not None and stored_models.dtype == torch.bool else stored_models
    with torch.cuda.device(dev):
        _run("peer_plan", lib.fmoe_peer_plan_from_table, _ptr(all_expert_count), _ptr(st), _ptr(caps), rank, n_expert,
             n_workers, _ptr(plan), _stream())
    return PeerPlan(plan, n_expert, n_workers)


def _planned_move(fn, name, buf, plan, out_rows):
    _check_cuda(buf)
    out = _recv_empty(buf, out_rows)
    with torch.cuda.device(buf.device):
        _run(name, fn, _comm(buf.device), _ptr(buf), _ptr(out), _ptr(plan.buf), buf.shape[0], out_rows,
             buf.shape[1] * buf.element_size(), plan.n_expert, _stream())
    return out


def peer_scatter_planned(input_buf, plan, out_rows):
    """global_scatter driven by a PeerPlan: [A, d] token-side rows -> [out_rows, d] expert-side buffer
    (out_rows may exceed the rows that arrive; the rest is left untouched)."""
    return _planned_move(lib.fmoe_peer_scatter_planned, "peer_scatter", input_buf, plan, out_rows)


def peer_scatter_planned_rows(src, row_of, row_div, scale, plan, out_rows):
    """peer_scatter_planned of rows that are produced on the way: token-side row i is
    ``src[row_of[i] // row_div]``, times ``scale.flatten()[row_of[i]]`` when ``scale`` is given (rounded
    once to the rows' dtype).  ``row_of``: int64, one entry per token-side row (more entries are ignored)."""
    _check_cuda(src, row_of)
    assert row_of.dtype == torch.int64 and src.dim() == 2 and src.is_contiguous() and row_of.is_contiguous()
    if scale is not None:
        _check_cuda(scale)
        assert scale.dtype == src.dtype and scale.is_contiguous()
    out = _recv_empty(src, out_rows)
    with torch.cuda.device(src.device):
        _run("peer_scatter", lib.fmoe_peer_scatter_planned_rows, _comm(src.device), _ptr(src), src.shape[0], _ptr(row_of),
             int(row_div), _ptr(scale), _dtype_code(src), _ptr(out), _ptr(plan.buf), row_of.numel(), out_rows,
             src.shape[1] * src.element_size(), plan.n_expert, _stream())
    return out


def peer_scatter_fused_begin(src, row_of, row_div, scale, plan, out_rows):
    """Prepares a peer_scatter_planned_rows that the grouped GEMM consuming its rows performs itself: give the
    returned PendingArrival to ``linear_forward_act`` / ``linear_backward_act`` as ``arrival``; that product
    moves the rows with its spare warps while it computes, and closes the exchange.  Returns (out, pending), or
    (None, None) when the exchange cannot take this form (nothing was queued).  ``finish()`` on a handle that no
    product took runs the exchange as a call of its own."""
    _check_cuda(src, row_of)
    assert row_of.dtype == torch.int64 and src.dim() == 2 and src.is_contiguous() and row_of.is_contiguous()
    if scale is not None:
        _check_cuda(scale)
        assert scale.dtype == src.dtype and scale.is_contiguous()
    out = _recv_empty(src, out_rows)
    h = _lib.Arrival()
    with torch.cuda.device(src.device):
        _run("peer_scatter", lib.fmoe_peer_scatter_fused_begin, _comm(src.device), _ptr(src), src.shape[0], _ptr(row_of),
             int(row_div), _ptr(scale), _dtype_code(src), _ptr(out), _ptr(plan.buf), row_of.numel(), out_rows,
             src.shape[1] * src.element_size(), plan.n_expert, _stream(), ctypes.byref(h))
    if not h.comm:
        return None, None
    return out, PendingArrival(h, (out, src, row_of, scale, plan.buf))


class PendingArrival:
    """Rows of a global_scatter that are still on their way (fmoe_arrival_t): give it to the grouped
    GEMM that reads them (``linear_forward_act`` / ``linear_backward_act``), which closes the exchange,
    or call ``finish()``.  Holds the buffers the exchange uses."""

    def __init__(self, handle, keep):
        self.handle, self.keep, self.open = handle, keep, bool(handle.comm)

    def finish(self):
        if self.open:
            self.open = False
            dev = self.keep[0].device
            with torch.cuda.device(dev):
                _run("peer_arrival_finish", lib.fmoe_peer_arrival_finish, ctypes.byref(self.handle), _stream())


def peer_scatter_planned_async(input_buf, plan, out_rows, overlap_sms):
    """peer_scatter_planned whose push runs beside the caller's stream on ``overlap_sms`` SMs.  Returns
    (out, PendingArrival); ``out`` may only be read by the GEMM the pending object is given to, or after
    ``finish()``.  Falls back to the plain exchange (pending object already closed) when it cannot overlap."""
    _check_cuda(input_buf)
    out = _recv_empty(input_buf, out_rows)
    h = _lib.Arrival()
    with torch.cuda.device(input_buf.device):
        _run("peer_scatter", lib.fmoe_peer_scatter_planned_async, _comm(input_buf.device), _ptr(input_buf), _ptr(out),
             _ptr(plan.buf), input_buf.shape[0], out_rows, input_buf.shape[1] * input_buf.element_size(), plan.n_expert,
             int(overlap_sms), _stream(), ctypes.byref(h))
    return out, PendingArrival(h, (input_buf, out, plan.buf))


def peer_gather_planned_async(output_buf, plan, out_rows, overlap_sms, use):
    """Starts a peer_gather_planned whose rows a grouped GEMM, queued next with the returned handle as
    ``departure``, is about to write into ``output_buf``.  Returns (out, PendingArrival) -- close it
    with ``finish()`` after that GEMM -- or (None, None) when it cannot overlap (nothing was queued)."""
    _check_cuda(output_buf)
    out = _recv_empty(output_buf, out_rows)
    h = _lib.Arrival()
    with torch.cuda.device(output_buf.device):
        _run("peer_gather", lib.fmoe_peer_gather_planned_async, _comm(output_buf.device), _ptr(output_buf), _ptr(out),
             _ptr(plan.buf), output_buf.shape[0], out_rows, output_buf.shape[1] * output_buf.element_size(),
             plan.n_expert, int(overlap_sms), int(use), _stream(), ctypes.byref(h))
    if not h.comm:
        return None, None
    return out, PendingArrival(h, (output_buf, out, plan.buf))


def peer_gather_fused_begin(like, plan, out_rows):
    """Prepares a global_gather that the next grouped GEMM performs itself: given the returned handle as
    ``departure``, that GEMM stores its output rows into the token-side buffers of their owners and
    writes no expert-side output.  ``like``: a tensor with the rows' width, dtype and device.  Returns
    (out [out_rows, d], PendingArrival) -- ``finish()`` after the GEMM makes ``out`` readable -- or
    (None, None) when the receive pool cannot hold ``out`` (nothing was queued)."""
    _check_cuda(like)
    out = _recv_empty(like, out_rows)
    h = _lib.Arrival()
    with torch.cuda.device(like.device):
        _run("peer_gather", lib.fmoe_peer_gather_fused_begin, _comm(like.device), _ptr(out), _ptr(plan.buf), out_rows,
             like.shape[1] * like.element_size(), plan.n_expert, _stream(), ctypes.byref(h))
    if not h.comm:
        return None, None
    return out, PendingArrival(h, (out, plan.buf))


def peer_gather_planned(output_buf, plan, out_rows):
    """global_gather driven by a PeerPlan: expert-side rows -> [out_rows, d] token-side buffer."""
    return _planned_move(lib.fmoe_peer_gather_planned, "peer_gather", output_buf, plan, out_rows)


def nosync_capacity(token_rows, row_bytes, n_workers, device):
    """Rows to give the expert-side buffers of a forward that does not read the counts back: the worst
    case (every rank routes everything here) when the receive pool can hold two such buffers beside
    the two token-side ones, else what the pool does hold; 0 when that leaves less than 1.5 x the
    balanced load (the caller then reads the counts as before)."""
    c = _comms.get(device.index if device.index is not None else torch.cuda.current_device())
    if c is None or int(lib.fmoe_peer_slot_bytes(c)) == 0:
        return 0
    pool = int(lib.fmoe_peer_pool_bytes(c))
    worst = n_workers * token_rows
    fits = int((0.9 * pool - 2 * token_rows * row_bytes) // (2 * row_bytes)) if row_bytes else 0
    cap = min(worst, fits)
    return cap if cap >= int(1.5 * token_rows) else 0


def exchange_cache_info(sent_models, num_expert, world_size):
    """All-gathers the per-rank shadow flags; returns [sent_models, stored_models[W,E]]."""
    _check_cuda(sent_models)
    assert sent_models.dtype == torch.bool and sent_models.numel() == num_expert
    stored = sent_models.new_zeros((world_size, num_expert))
    with torch.cuda.device(sent_models.device):
        _run("exchange_cache_info", lib.fmoe_exchange_cache_info, _comm(sent_models.device), _ptr(sent_models), _ptr(stored),
                                           num_expert, world_size, _stream())
    return [sent_models, stored]


def model_exchange(stored_models, local_params, params, num_expert, world_size):
    """Broadcasts each shadowed (worker j, slot i) parameter buffer from its owner.

    ``local_params[i]`` is this rank's flat buffer, ``params[j][i]`` the buffer that
    receives worker j's copy (cuda/global_exchange.cuh:251-282).  Returns this rank.
    """
    flags = _host_flags(stored_models)
    dev = local_params[0].device
    rank, world = comm_rank(dev)
    assert world == world_size
    with torch.cuda.device(dev):
        for i in range(num_expert):
            for j in range(world_size):
                if not flags[i + j * num_expert]:
                    continue
                buf = local_params[i] if j == rank else params[j][i]
                _check_cuda(buf)
                _run("model_exchange", lib.fmoe_model_broadcast, _comm(dev), _ptr(buf), buf.numel() * buf.element_size(),
                                               j, _stream())
    return rank


def generate_cached_count(local_expert_count, global_expert_count, stored_models, num_expert, world_size):
    """fwd_expert_count [W*E] once shadowed experts run locally (cuda/global_exchange.cu:175-196)."""
    _check_cuda(local_expert_count, global_expert_count, stored_models)
    dev = local_expert_count.device
    rank, _ = comm_rank(dev)
    lec = local_expert_count.reshape(-1).to(torch.int64).contiguous()
    gec = global_expert_count.reshape(-1).to(torch.int64).contiguous()
    st = stored_models.reshape(-1).to(torch.uint8).contiguous()
    out = torch.empty_like(lec)
    with torch.cuda.device(dev):
        _run("generate_cached_count", lib.fmoe_generate_cached_count, _ptr(lec), _ptr(gec), _ptr(st), _ptr(out), rank, num_expert,
                                             world_size, _stream())
    return out


def gradient_exchange(stored_models, local_grads, grads, num_expert, world_size):
    """Sum-reduces shadow gradients to the owning rank, in place (cuda/global_exchange.cuh:322-348)."""
    flags = _host_flags(stored_models)
    dev = local_grads[0].device
    rank, _ = comm_rank(dev)
    with torch.cuda.device(dev):
        for i in range(num_expert):
            for j in range(world_size):
                if not flags[i + j * num_expert]:
                    continue
                buf = local_grads[i] if j == rank else grads[j][i]
                _check_cuda(buf)
                _run("gradient_exchange", lib.fmoe_gradient_reduce, _comm(dev), _ptr(buf), buf.numel(), _dtype_code(buf), j,
                                               _stream())


# ---------------------------------------------------------------------------
# Extended operators (no counterpart in the reference's extension)
# ---------------------------------------------------------------------------

def gate_topk(logits, k):
    """(values [T,k], indices [T,k] int64): the k largest logits per row (torch.topk, largest=True), in
    descending order, ties by ascending index (fmoe/gates/naive_gate.py:31-34)."""
    _check_cuda(logits)
    logits = logits.contiguous()
    n_tok, n_exp = logits.shape
    val = logits.new_empty((n_tok, k))
    idx = torch.empty((n_tok, k), dtype=torch.int64, device=logits.device)
    with torch.cuda.device(logits.device):
        _run("gate_topk", lib.fmoe_gate_topk, _ptr(logits), n_tok, n_exp, k, _dtype_code(logits), _ptr(val), _ptr(idx),
             _stream())
    return val, idx


def gate_topk_backward(grad_values, indices, n_expert_total):
    """Gradient of gate_topk with respect to the logits ([T, n_expert_total])."""
    _check_cuda(grad_values, indices)
    grad_values = grad_values.contiguous()
    n_tok, k = indices.shape
    out = grad_values.new_empty((n_tok, n_expert_total))
    with torch.cuda.device(grad_values.device):
        _run("gate_topk_backward", lib.fmoe_gate_topk_backward, _ptr(grad_values), _ptr(indices), n_tok, n_expert_total, k,
             _dtype_code(grad_values), _ptr(out), _stream())
    return out


def count_and_pos(gate, n_expert_total, want_inv=True):
    """One-call form of count_by_gate's bucketing (fmoe/functions.py:19-41).

    Returns ``(lec int64[E_tot], offsets int64[E_tot+1], pos int64[n], inv int64[n] or None)``.
    ``pos`` has one slot per gate entry; slots past ``offsets[-1]`` hold -1.
    Nothing is copied to the host.
    """
    _check_cuda(gate)
    assert gate.dtype == torch.int64
    n, dev = gate.numel(), gate.device
    lec = torch.empty(n_expert_total, dtype=torch.int64, device=dev)
    off = torch.empty(n_expert_total + 1, dtype=torch.int64, device=dev)
    pos = torch.empty(n, dtype=torch.int64, device=dev)
    inv = torch.empty(n, dtype=torch.int64, device=dev) if want_inv else None
    with torch.cuda.device(dev):
        scratch = _routing_scratch(n, n_expert_total, dev)
        _run("count_and_pos", lib.fmoe_count_and_pos, _ptr(gate), n, n_expert_total, _ptr(lec), _ptr(off), _ptr(pos),
                                     _ptr(inv), _ptr(scratch), _stream())
    return lec, off, pos, inv


def local_scatter(inp, pos, pos_div=1, n_rows=None):
    """out[i] = inp[pos[i] // pos_div]; rows with pos[i] < 0 are zero."""
    _check_cuda(inp, pos)
    n = pos.numel() if n_rows is None else n_rows
    out = inp.new_empty((n, inp.shape[1]))
    with torch.cuda.device(inp.device):
        _run("local_scatter", lib.fmoe_local_scatter, _ptr(inp), _ptr(pos), _ptr(out), n, inp.shape[0],
                                     inp.shape[1] * inp.element_size(), pos_div, _stream())
    return out


def local_gather(buf, pos, out_rows):
    """zeros(out_rows, d) with out[pos[i]] = buf[i] (index_copy_ semantics)."""
    _check_cuda(buf, pos)
    out = buf.new_empty((out_rows, buf.shape[1]))
    with torch.cuda.device(buf.device):
        inv = torch.empty(out_rows, dtype=torch.int64, device=buf.device)
        _run("local_gather", lib.fmoe_local_gather, _ptr(buf), _ptr(pos), _ptr(out), pos.numel(), out_rows,
                                    buf.shape[1] * buf.element_size(), _ptr(inv), _stream())
    return out


def local_gather_inv(buf, inv):
    """out[r] = buf[inv[r]] (zero row where inv[r] < 0)."""
    _check_cuda(buf, inv)
    out = buf.new_empty((inv.numel(), buf.shape[1]))
    with torch.cuda.device(buf.device):
        _run("local_gather_inv", lib.fmoe_local_gather_inv, _ptr(buf), _ptr(inv), _ptr(out), inv.numel(),
                                        buf.shape[1] * buf.element_size(), _stream())
    return out


def local_gather_sum(buf, inv, n_tokens, top_k):
    """out[t] = sum_j buf[inv[t*top_k+j]] over valid slots (deterministic index_add_)."""
    _check_cuda(buf, inv)
    out = buf.new_empty((n_tokens, buf.shape[1]))
    with torch.cuda.device(buf.device):
        _run("local_gather_sum", lib.fmoe_local_gather_sum, _ptr(buf), _ptr(inv), _ptr(out), n_tokens, top_k, buf.shape[1],
                                        _dtype_code(buf), _stream())
    return out


def local_gather_add(buf, pos, out_rows):
    """zeros(out_rows, d) with out[pos[i]] += buf[i] (index_add_ semantics), rows that collide added
    in ascending i (fmoe/functions.py:77-81)."""
    _check_cuda(buf, pos)
    out = buf.new_empty((out_rows, buf.shape[1]))
    with torch.cuda.device(buf.device):
        scratch = _scratch(lib.fmoe_local_gather_add_scratch_bytes(out_rows), buf.device)
        _run("local_gather_add", lib.fmoe_local_gather_add, _ptr(buf), _ptr(pos), _ptr(out), pos.numel(), out_rows,
             buf.shape[1], _dtype_code(buf), _ptr(scratch), _stream())
    return out


def combine_forward(buf, inv, score):
    """out[t] = sum_j score[t,j] * buf[inv[t*k+j]] (inv None: buf is already [T*k, d])."""
    _check_cuda(buf, inv, score)
    n_tokens, top_k = score.shape
    assert score.dtype == buf.dtype
    out = buf.new_empty((n_tokens, buf.shape[1]))
    with torch.cuda.device(buf.device):
        _run("combine_forward", lib.fmoe_combine_forward, _ptr(buf), _ptr(inv), _ptr(score), _ptr(out), n_tokens, top_k,
                                       buf.shape[1], _dtype_code(buf), _stream())
    return out


def combine_backward(grad_out, buf, inv, score, need_score_grad=True, need_buf_grad=True):
    """Returns (grad_buf, grad_score) of combine_forward.  Rows of grad_buf that no
    slot maps to are left unwritten.  ``need_buf_grad=False``: only the score gradient (grad_buf None)."""
    _check_cuda(grad_out, buf, inv, score)
    n_tokens, top_k = score.shape
    if not (need_score_grad or need_buf_grad):
        return None, None
    grad_buf = torch.empty_like(buf) if need_buf_grad else None
    grad_score = torch.empty_like(score) if need_score_grad else None
    with torch.cuda.device(buf.device):
        _run("combine_backward", lib.fmoe_combine_backward, _ptr(grad_out), _ptr(buf), _ptr(inv), _ptr(score), _ptr(grad_buf),
                                        _ptr(grad_score), n_tokens, top_k, buf.shape[1], _dtype_code(buf),
                                        _stream())
    return grad_buf, grad_score


def linear_forward_act(x, seg_offsets, weight, bias, activation, want_pre=False, arrival=None, departure=None, out=None):
    """Grouped GEMM with fused bias and activation.  Returns (y, act_deriv or None);
    ``act_deriv`` (with ``want_pre`` and GELU) holds gelu'(pre-activation), the factor
    that linear_backward_act multiplies into the input gradient.  ``arrival``: a PendingArrival
    whose exchange is still filling ``x``; the call closes it.  ``departure``: a PendingArrival of
    peer_gather_planned_async that forwards ``out`` (the preallocated y) while the product runs; the
    caller closes it."""
    _check_cuda(x, seg_offsets, weight, bias)
    n_expert, out_feat, in_feat = weight.shape
    assert x.shape[1] == in_feat and x.dtype == weight.dtype
    assert seg_offsets.dtype == torch.int64 and seg_offsets.numel() == n_expert + 1
    y = out if out is not None else x.new_empty((x.shape[0], out_feat))
    assert y.shape == (x.shape[0], out_feat) and y.dtype == x.dtype and y.is_contiguous()
    pre = x.new_empty((x.shape[0], out_feat)) if want_pre else None
    with torch.cuda.device(x.device):
        arriving = arrival is not None and arrival.open
        if arriving or departure is not None:
            if arriving:
                arrival.open = False
            _run("linear_forward", lib.fmoe_linear_forward_overlapped, _ptr(x), _ptr(weight), _ptr(bias), _ptr(seg_offsets),
                 _ptr(y), _ptr(pre), x.shape[0], in_feat, out_feat, n_expert, _dtype_code(x), activation,
                 ctypes.byref(arrival.handle) if arriving else None,
                 ctypes.byref(departure.handle) if departure is not None else None, _stream())
            return y, pre
        _run("linear_forward", lib.fmoe_linear_forward, _ptr(x), _ptr(weight), _ptr(bias), _ptr(seg_offsets), _ptr(y),
                                      _ptr(pre), x.shape[0], in_feat, out_feat, n_expert, _dtype_code(x),
                                      activation, _stream())
    return y, pre


def linear_backward_act(grad_y, x, seg_offsets, weight, act_pre, activation, need_bias=True,
                        need_input_grad=True, grad_w=None, grad_b=None, accumulate=False, want_gx_colsum=False,
                        arrival=None, departure=None, grad_x=None):
    """Grouped GEMM backward.  ``act_pre`` (shape of x) fuses the backward of the
    activation that produced ``x`` into the input gradient: for ReLU pass the activation
    output, for GELU the derivative buffer of linear_forward_act.  Returns (dX, dW, db), and with
    ``want_gx_colsum`` a fourth tensor [E, in_feat]: the per-expert column sums of dX (the bias
    gradient of the layer that produced ``x``), which the input-gradient kernel computes on the way."""
    _check_cuda(grad_y, x, seg_offsets, weight, act_pre)
    n_expert, out_feat, in_feat = weight.shape
    n_rows = grad_y.shape[0]
    gx = (grad_x if grad_x is not None else x.new_empty((n_rows, in_feat))) if need_input_grad else None
    gw = grad_w if grad_w is not None else torch.empty_like(weight)
    gb = grad_b if grad_b is not None else (weight.new_empty((n_expert, out_feat)) if need_bias else None)
    with torch.cuda.device(x.device):
        nbytes = lib.fmoe_linear_scratch_bytes(n_rows, in_feat, out_feat, n_expert, _dtype_code(x))
        scratch = _scratch(nbytes, x.device)
        arriving = arrival is not None and arrival.open
        if arriving or departure is not None:
            # grad_y is still arriving (the call closes that exchange) and / or grad_x is forwarded as it is produced
            if arriving:
                arrival.open = False
            cs = weight.new_empty((n_expert, in_feat)) if want_gx_colsum else None
            _run("linear_backward", lib.fmoe_linear_backward_overlapped, _ptr(grad_y), _ptr(x), _ptr(weight),
                 _ptr(seg_offsets), _ptr(act_pre), _ptr(gx), _ptr(gw), _ptr(gb), _ptr(cs), n_rows, in_feat,
                 out_feat, n_expert, _dtype_code(x), activation, 1 if accumulate else 0, _ptr(scratch),
                 ctypes.byref(arrival.handle) if arriving else None,
                 ctypes.byref(departure.handle) if departure is not None else None, _stream())
            return (gx, gw, gb, cs) if want_gx_colsum else (gx, gw, gb)
        if want_gx_colsum:
            assert need_input_grad
            cs = weight.new_empty((n_expert, in_feat))
            _run("linear_backward", lib.fmoe_linear_backward_colsum, _ptr(grad_y), _ptr(x), _ptr(weight),
                 _ptr(seg_offsets), _ptr(act_pre), _ptr(gx), _ptr(gw), _ptr(gb), _ptr(cs), n_rows, in_feat,
                 out_feat, n_expert, _dtype_code(x), activation, 1 if accumulate else 0, _ptr(scratch), _stream())
            return gx, gw, gb, cs
        _run("linear_backward", lib.fmoe_linear_backward, _ptr(grad_y), _ptr(x), _ptr(weight), _ptr(seg_offsets),
                                       _ptr(act_pre), _ptr(gx), _ptr(gw), _ptr(gb), n_rows, in_feat,
                                       out_feat, n_expert, _dtype_code(x), activation,
                                       1 if accumulate else 0, _ptr(scratch), _stream())
    return gx, gw, gb


# ---------------------------------------------------------------------------
# fused_compute: cuda/fmoe_cuda.cpp:80-100 (smart schedule)
# ---------------------------------------------------------------------------

_comm_streams = {}


def _comm_stream(device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    s = _comm_streams.get(idx)
    if s is None:
        s = torch.cuda.Stream(device=device)
        _comm_streams[idx] = s
    return s


def _fused_staging(like, rows, d_model):
    """Staging for the one-send-per-peer exchange of the smart schedule (None: per-expert sends)."""
    # Every rank must make the same choice (the two forms pair sends and receives
    # differently), so the buffer exists even on a rank that receives nothing.
    if os.environ.get("FMOE_B200_EXCHANGE") == "split":
        return None
    return like.new_empty((max(int(rows), 1), d_model))


def fuse_gran():
    """Peers per pipeline step: env FMOE_FUSE_GRAN, default 4 (cuda/fused_compute.cu:21-28).
    Read on every call (the reference caches the first value in a process global)."""
    try:
        return max(1, int(os.environ.get("FMOE_FUSE_GRAN", "4")))
    except ValueError:
        return 4


def fused_geometry(local_expert_count, global_expert_count, stored_models, n_workers, rank, gran=None):
    """Returns (n_steps, gran, global_rows B, shadow_rows S) of a smart-schedule call."""
    lec, gec, st = _host_i64(local_expert_count), _host_i64(global_expert_count), _host_flags(stored_models)
    n_expert = lec.numel() // n_workers
    geo = _lib.FusedGeometry()
    check(lib.fmoe_fused_geometry(_ptr(lec), _ptr(gec), _ptr(st), rank, n_expert, n_workers,
                                  fuse_gran() if gran is None else gran, ctypes.byref(geo)), "fused_geometry")
    return geo.n_steps, geo.gran, geo.global_rows, geo.shadow_rows


def _split_params(ps):
    """(w1, b1, w2, b2) from a worker's parameter tuple: (w1, w2) or (w1, b1, w2, b2)."""
    ps = tuple(ps)
    if len(ps) == 2:
        return ps[0], None, ps[1], None
    if len(ps) == 4:
        return ps
    raise RuntimeError(f"fmoe_cuda: expected 2 or 4 expert parameter tensors per worker, got {len(ps)}")


def _mlp_table(params, grads, n_workers):
    table = (_lib.MlpParams * n_workers)()
    keep = []
    for j in range(n_workers):
        if not params[j]:
            continue
        w1, b1, w2, b2 = _split_params(params[j][0])
        _check_cuda(w1, b1, w2, b2)
        table[j].w1, table[j].b1, table[j].w2, table[j].b2 = (t.data_ptr() if t is not None else None
                                                              for t in (w1, b1, w2, b2))
        if grads is not None and grads[j]:
            g1, gb1, g2, gb2 = _split_params(grads[j][0])
            _check_cuda(g1, gb1, g2, gb2)
            table[j].gw1, table[j].gb1, table[j].gw2, table[j].gb2 = (t.data_ptr() if t is not None else None
                                                                      for t in (g1, gb1, g2, gb2))
        keep.append((w1, b1, w2, b2))
    return table, keep


def fused_forward(input_buf, params, local_expert_count, global_expert_count, stored_models,
                  global_batch_size, n_workers, has_bias, activation=_lib.ACT_RELU):
    """Smart-schedule forward (cuda/fused_compute.cu:12-62).

    ``params[j]`` is ``[tuple_of_parameters]`` for the own worker and for shadowed
    workers, else ``[]``.  Returns ``[out [A,d], global_in, middle, global_out]``
    (+ the pre-activation buffer when ``activation`` is GELU); the expert-side
    buffers have B+S rows (see fused_geometry) and are what fused_backward needs.
    ``global_batch_size`` is accepted for signature compatibility and checked.
    The reference hard-codes ReLU and ignores biases; here ``activation`` selects the
    function and biases in the parameter tuples are applied.
    """
    _check_cuda(input_buf)
    dev = input_buf.device
    lec, gec, st = _host_i64(local_expert_count), _host_i64(global_expert_count), _host_flags(stored_models)
    n_expert = lec.numel() // n_workers
    rank = comm_rank(dev)[0] if n_workers > 1 else 0
    w1 = _split_params(params[rank][0])[0]
    d_hidden, d_model = w1.shape[1], w1.shape[2]
    gran = fuse_gran()
    _, _, B, S = fused_geometry(lec, gec, st, n_workers, rank, gran)
    if global_batch_size is not None and int(global_batch_size) != B + S:
        raise RuntimeError(f"fused_forward: global_batch_size={global_batch_size} but the counts give {B + S} rows")
    A = input_buf.shape[0]
    gib = input_buf.new_empty((B + S, d_model))
    gmb = input_buf.new_empty((B + S, d_hidden))
    pre = input_buf.new_empty((B + S, d_hidden)) if activation == _lib.ACT_GELU else None
    gob = input_buf.new_empty((B + S, d_model))
    out = input_buf.new_empty((A, d_model))
    table, keep = _mlp_table(params, None, n_workers)
    with torch.cuda.device(dev):
        comm = _comm(dev) if n_workers > 1 else None
        _run("fused_forward", lib.fmoe_fused_forward, comm, _ptr(input_buf), _ptr(out), _ptr(gib), _ptr(gmb),
             _ptr(pre), _ptr(gob), table, _ptr(lec), _ptr(gec), _ptr(st), A, d_model, d_hidden, n_expert,
             n_workers, _dtype_code(input_buf), activation, gran, _ptr(_fused_staging(input_buf, B, d_model)), _stream(),
             ctypes.c_void_p(_comm_stream(dev).cuda_stream))
    res = [out, gib, gmb, gob]
    if pre is not None:
        res.append(pre)
    return res


def fused_backward(input_buf, params, middle_buf, output_buf, grad_out, local_expert_count,
                   global_expert_count, inp, stored_models, global_batch_size, buf_batch_size, n_workers,
                   has_bias, activation=_lib.ACT_RELU, middle_pre=None, grads=None):
    """Smart-schedule backward (cuda/fused_compute.cu:64-131).  Returns ``[grad_in [A,d]]``.

    Weight gradients: with ``grads`` (same nesting as ``params``) they are written
    there; otherwise into ``param.grad`` of every tensor in ``params``, created when
    missing -- the own experts' gradients are OVERWRITTEN (first pipeline step) and
    shadowed experts' accumulated, exactly as the reference does.
    ``output_buf`` and ``inp`` are unused (kept for signature compatibility).
    """
    _check_cuda(input_buf, middle_buf, grad_out)
    dev = input_buf.device
    lec, gec, st = _host_i64(local_expert_count), _host_i64(global_expert_count), _host_flags(stored_models)
    n_expert = lec.numel() // n_workers
    rank = comm_rank(dev)[0] if n_workers > 1 else 0
    d_hidden, d_model = middle_buf.shape[1], input_buf.shape[1]
    if grads is None:
        grads = []
        for j in range(n_workers):
            if not params[j]:
                grads.append([])
                continue
            gs = []
            for p in params[j][0]:
                if p.grad is None:
                    p.grad = torch.zeros_like(p)
                gs.append(p.grad)
            grads.append([tuple(gs)])
    rows = input_buf.shape[0]
    ggo = input_buf.new_empty((rows, d_model))
    gmid = input_buf.new_empty((rows, d_hidden))
    ggi = input_buf.new_empty((rows, d_model))
    grad_in = input_buf.new_empty((grad_out.shape[0], d_model))
    table, keep = _mlp_table(params, grads, n_workers)
    gran = fuse_gran()
    with torch.cuda.device(dev):
        comm = _comm(dev) if n_workers > 1 else None
        _run("fused_backward", lib.fmoe_fused_backward, comm, _ptr(grad_out), _ptr(grad_in), _ptr(input_buf),
             _ptr(middle_buf), _ptr(middle_pre), _ptr(ggo), _ptr(gmid), _ptr(ggi), table, _ptr(lec), _ptr(gec),
             _ptr(st), grad_out.shape[0], d_model, d_hidden, n_expert, n_workers, _dtype_code(input_buf),
             activation, gran, _ptr(_fused_staging(input_buf, rows, d_model)), _stream(), ctypes.c_void_p(_comm_stream(dev).cuda_stream))
    return [grad_in]
