"""Rank bodies of the multi-process tests (spawned by test_dist_gpu.py / test_dist_cpu.py)."""
import contextlib
import ctypes
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import moe_oracle as O  # noqa: E402


def init(rank, world, port, backend):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"] = str(rank), str(world), str(rank)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if backend == "nccl":
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)


def finish(backend):
    if backend == "nccl":
        from fastermoe_b200 import fmoe_cuda
        torch.cuda.synchronize()
        fmoe_cuda.destroy_comms()
    dist.barrier()
    dist.destroy_process_group()


def all_lecs(world, E, seed, lo=0, hi=9):
    rng = np.random.default_rng(seed)
    return [rng.integers(lo, hi, size=world * E) for _ in range(world)]


# ------------------------------------------------------------------ GPU / NCCL

def gpu_exchange(rank, world, port):
    init(rank, world, port, "nccl")
    os.environ.setdefault("FMOE_B200_PEER_TIMEOUT_MS", "4000")    # a protocol error should fail fast here
    check_exchange(rank, world, torch.device("cuda", rank))
    finish("nccl")


def check_exchange(rank, world, dev):
    """Count exchange, both forms of global_scatter / global_gather (with shadowed experts), bounded
    waits, the device-built plan, shadow bookkeeping and the capacity gate across ranks, each
    against the oracle.  Needs an initialised NCCL process group; usable from any launcher."""
    from fastermoe_b200 import fmoe_cuda as fc
    fc.ensure_nccl(None, torch.zeros(1, device=dev))
    E, d = 3, 40
    lecs = all_lecs(world, E, 5)
    aec_w, agec_w, gecs = O.expert_exchange(lecs, E, world)
    aec, agec, gec = fc.expert_exchange(torch.from_numpy(lecs[rank]).to(dev), E, world)
    assert np.array_equal(aec.cpu().numpy(), aec_w) and np.array_equal(agec.cpu().numpy(), agec_w)
    assert np.array_equal(gec.cpu().numpy(), gecs[rank])
    for stored in (np.zeros(world * E, bool), np.repeat(np.arange(world) == 0, E), np.repeat(np.arange(world) == world - 1, E)):
        rng = np.random.default_rng(9)
        bufs = [rng.standard_normal((int(l.sum()), d)).astype(np.float32) for l in lecs]
        want = O.global_scatter(bufs, lecs, stored, E, world)
        # "split": one send/receive per (expert, peer) as in the reference; default: one per peer + staging
        for mode, dtype in (("", torch.float32), ("", torch.bfloat16), ("split", torch.float32)):
            os.environ["FMOE_B200_EXCHANGE"] = mode
            mine = torch.from_numpy(bufs[rank]).to(dev).to(dtype)
            out = fc.global_scatter(mine, torch.from_numpy(lecs[rank]), torch.from_numpy(gecs[rank]),
                                    torch.from_numpy(stored), want[rank].shape[0], world)
            assert torch.equal(out, torch.from_numpy(want[rank]).to(dev).to(dtype)), "global_scatter layout"
            back = fc.global_gather(out, torch.from_numpy(lecs[rank]), torch.from_numpy(gecs[rank]),
                                    torch.from_numpy(stored), mine.shape[0], world)
            assert torch.equal(back, mine), "global_gather is not the inverse"
        os.environ["FMOE_B200_EXCHANGE"] = ""
        # the same exchange by direct stores into the peers' memory; several rounds reuse both landing slots
        if fc.peer_slot_bytes(dev) > 0:
            table = torch.from_numpy(aec_w.copy())
            for rnd in range(5):
                for dtype in (torch.float32, torch.bfloat16):
                    mine = (torch.from_numpy(bufs[rank]).to(dev) + rnd).to(dtype)
                    out = fc.peer_global_scatter(mine, table, torch.from_numpy(stored), want[rank].shape[0], E, world)
                    assert out is not None, "peer form refused a call it can serve"
                    assert torch.equal(out, (torch.from_numpy(want[rank]).to(dev) + rnd).to(dtype)), "peer scatter layout"
                    back = fc.peer_global_gather(out, table, torch.from_numpy(stored), mine.shape[0] + 2, E, world)
                    assert torch.equal(back[:-2], mine) and not back[-2:].any(), "peer gather is not the inverse"
            odd = torch.zeros(int(lecs[rank].sum()), 3, device=dev)        # 12-byte rows: not served, on any rank
            assert fc.peer_global_scatter(odd, table, torch.from_numpy(stored), want[rank].shape[0], E, world) is None
            st = ctypes.c_int32(-1)
            assert fc.lib.fmoe_device_status(ctypes.byref(st)) == 0 and st.value == 0, f"device status {st.value}"
            # a wait for an announcement (push) or for rows (consume) that nobody sends ends by itself,
            # raises the status bit and leaves the exchange usable
            import time
            for push, bit in ((0, 32), (1, 16)):
                t0 = time.time()
                with torch.cuda.device(dev):
                    assert fc.lib.fmoe_peer_wait_probe(fc._comm(dev), 150, push, fc._stream()) == 0, fc._lib.last_error()
                assert fc.lib.fmoe_device_status(ctypes.byref(st)) == 0 and st.value == bit, f"status {st.value}"
                assert 0.1 < time.time() - t0 < 5.0
                assert fc.lib.fmoe_device_status_clear() == 0
                assert fc.lib.fmoe_device_status(ctypes.byref(st)) == 0 and st.value == 0
                mine = torch.from_numpy(bufs[rank]).to(dev)
                out = fc.peer_global_scatter(mine, table, torch.from_numpy(stored), want[rank].shape[0], E, world)
                assert torch.equal(out, torch.from_numpy(want[rank]).to(dev)), "exchange after an expired wait"
        else:
            print(f"[rank {rank}] peer-memory exchange is off on this machine; NCCL form only", flush=True)
        cc = fc.generate_cached_count(torch.from_numpy(lecs[rank]).to(dev).view(world, E),
                                      torch.from_numpy(gecs[rank]).to(dev).view(world, E),
                                      torch.from_numpy(stored).to(dev).view(world, E), E, world)
        assert np.array_equal(cc.cpu().numpy(), O.generate_cached_count(lecs[rank], gecs[rank], stored, rank, E, world))
    # more row segments than one launch of the peer kernels takes (128): several launches per phase
    if fc.peer_slot_bytes(dev) > 0:
        E2 = 80
        lecs2 = all_lecs(world, E2, 6, lo=0, hi=5)
        table2, _, _ = O.expert_exchange(lecs2, E2, world)
        none2 = np.zeros(world * E2, bool)
        bufs2 = [np.random.default_rng(10 + r).standard_normal((int(lecs2[r].sum()), 8)).astype(np.float32) for r in range(world)]
        want2 = O.global_scatter(bufs2, lecs2, none2, E2, world)
        for rnd in range(3):
            mine = torch.from_numpy(bufs2[rank]).to(dev) + rnd
            out = fc.peer_global_scatter(mine, torch.from_numpy(table2.copy()), torch.from_numpy(none2), want2[rank].shape[0], E2, world)
            assert out is not None and torch.equal(out, torch.from_numpy(want2[rank]).to(dev) + rnd), "many-segment scatter"
            back = fc.peer_global_gather(out, torch.from_numpy(table2.copy()), torch.from_numpy(none2), mine.shape[0], E2, world)
            assert torch.equal(back, mine), "many-segment gather"
    if fc.peer_slot_bytes(dev) > 0:
        _late_rank_exchange(fc, rank, world, dev)
        _planned_exchange_with_capacity(fc, rank, world, dev)
    # shadow flags of every rank (cuda/global_exchange.cuh:232-249)
    mine = torch.from_numpy(np.random.default_rng(40 + rank).random(E) < 0.5).to(dev)
    sent, stored_all = fc.exchange_cache_info(mine, E, world)
    want_flags = np.stack([np.random.default_rng(40 + r).random(E) < 0.5 for r in range(world)])
    assert sent is mine and np.array_equal(stored_all.cpu().numpy(), want_flags)
    # mismatched buffer size is caught before anything is queued
    try:
        fc.global_scatter(torch.zeros(int(lecs[rank].sum()), d, device=dev), torch.from_numpy(lecs[rank]),
                          torch.from_numpy(gecs[rank]), torch.zeros(world * E, dtype=torch.bool), 1, world)
        raise AssertionError("size mismatch not detected")
    except RuntimeError as e:
        assert "rows" in str(e)
    # capacity gate across ranks
    from fastermoe_b200.gates.utils import limit_by_capacity
    gates = [np.random.default_rng(100 + r).integers(0, world * E, size=(64, 2)) for r in range(world)]
    for g in gates:
        g[:40, 0] = 1
    want = O.limit_by_capacity_gate(gates, E, world, 30)
    new_lec, new_gec, pruned = limit_by_capacity(torch.from_numpy(gates[rank]).to(dev), E, world, 30)
    assert np.array_equal(pruned.cpu().numpy(), want[rank][2])
    assert np.array_equal(new_lec.cpu().numpy(), want[rank][0]) and np.array_equal(new_gec.cpu().numpy(), want[rank][1])
    # prepare_forward's tuple at world_size > 1 (fmoe/functions.py:45-69)
    from fastermoe_b200.functions import prepare_forward
    os.environ["FMOE_B200_NOSYNC"] = "0"
    pos, lec_c, gec_c, aec_c, agec_c, fwd_c = prepare_forward(torch.from_numpy(gates[rank]).to(dev), E, world)
    os.environ["FMOE_B200_NOSYNC"] = "1"
    g_lecs = [O.expert_count(g, world * E).astype(np.int64) for g in gates]
    g_aec, g_agec, g_gecs = O.expert_exchange(g_lecs, E, world)
    assert np.array_equal(pos.cpu().numpy(), O.assign_pos(gates[rank], world * E))
    assert np.array_equal(lec_c.numpy(), g_lecs[rank]) and np.array_equal(gec_c.numpy(), g_gecs[rank])
    assert np.array_equal(aec_c.numpy().reshape(-1), g_aec.reshape(-1)) and np.array_equal(agec_c.numpy().reshape(-1), g_agec.reshape(-1))
    assert np.array_equal(fwd_c.numpy(), g_gecs[rank].reshape(world, E).sum(0))


def _late_rank_exchange(fc, rank, world, dev):
    """One rank joins an exchange only after the others have given up waiting for it (a failure made
    on the host; every wait involved is bounded).  The others must not have stored a single row into
    the late rank's memory -- neither where it receives this exchange nor where it received the
    exchanges before (the addresses its stale announcements still name) -- they report the expired
    waits in the status word, and the next exchange works again."""
    E, d = 2, 16
    late = world - 1
    lecs = all_lecs(world, E, 77, lo=1, hi=6)
    table, _, _ = O.expert_exchange(lecs, E, world)
    none = np.zeros(world * E, bool)
    bufs = [np.random.default_rng(50 + r).standard_normal((int(lecs[r].sum()), d)).astype(np.float32) for r in range(world)]
    want = O.global_scatter(bufs, lecs, none, E, world)
    plan = fc.peer_plan_from_table(torch.from_numpy(table.copy()).to(dev), None, rank, E, world)
    mine = torch.from_numpy(bufs[rank]).to(dev)
    rows = want[rank].shape[0]
    # two ordinary exchanges first: their outputs stay alive and are what stale announcements name
    old = [fc.peer_scatter_planned(mine, plan, rows) for _ in range(2)]
    for o in old:
        assert torch.equal(o, torch.from_numpy(want[rank]).to(dev))
    snap = [o.clone() for o in old]

    def exchange_into_sevens():
        out = fc._recv_empty(mine, rows)
        out.fill_(7.0)
        with torch.cuda.device(dev):
            rc = fc.lib.fmoe_peer_scatter_planned(fc._comm(dev), fc._ptr(mine), fc._ptr(out), fc._ptr(plan.buf), mine.shape[0],
                                                  rows, d * 4, E, fc._stream())
        assert rc == 0, fc._lib.last_error()
        torch.cuda.synchronize()
        return out

    moves, _ = O.scatter_moves(lecs, none, rank, E, world)
    if rank != late:
        assert fc.lib.fmoe_peer_set_timeout_ms(fc._comm(dev), 300) == 0
        out = exchange_into_sevens()
        assert fc.lib.fmoe_peer_set_timeout_ms(fc._comm(dev), int(os.environ.get("FMOE_B200_PEER_TIMEOUT_MS", "20000"))) == 0
        st = fc.device_status(dev)
        assert st & 16 and st & 32, f"expired waits not reported: {st}"
        assert fc.lib.fmoe_device_status_clear() == 0
        for (src, src_row, dst_row, n) in moves:       # rows of the ranks that took part arrived, the late rank's did not
            got = out[dst_row:dst_row + n]
            if src == late:
                assert bool((got == 7).all()), "rows appeared from a rank that never pushed"
            else:
                assert torch.equal(got, torch.from_numpy(bufs[src][src_row:src_row + n]).to(dev))
    dist.barrier()
    if rank == late:
        out = exchange_into_sevens()               # the others' announcements and arrival flags are long there
        assert fc.device_status(dev) == 0
        for (src, src_row, dst_row, n) in moves:
            got = out[dst_row:dst_row + n]
            if src == late:
                assert torch.equal(got, torch.from_numpy(bufs[src][src_row:src_row + n]).to(dev))
            else:
                assert bool((got == 7).all()), "a rank that gave up waiting stored rows all the same"
        for o, s_ in zip(old, snap):
            assert torch.equal(o, s_), "rows were stored at an address from an older announcement"
    dist.barrier()
    out = fc.peer_scatter_planned(mine, plan, rows)
    assert torch.equal(out, torch.from_numpy(want[rank]).to(dev)), "exchange after a late rank"
    assert fc.device_status(dev) == 0


def _planned_exchange_with_capacity(fc, rank, world, dev):
    """Counts swapped through peer memory, plan built on the device, buffers larger than what arrives;
    then a capacity that one rank exceeds: every rank's plan comes out empty, nothing is stored."""
    E, d = 3, 24
    lecs = all_lecs(world, E, 91, lo=0, hi=7)
    table, _, gecs = O.expert_exchange(lecs, E, world)
    none = np.zeros(world * E, bool)
    bufs = [np.random.default_rng(60 + r).standard_normal((int(lecs[r].sum()), d)).astype(np.float32) for r in range(world)]
    want = O.global_scatter(bufs, lecs, none, E, world)
    recv = want[rank].shape[0]
    mine = torch.from_numpy(bufs[rank]).to(dev)
    for rnd in range(3):
        cap = recv + 5 + rnd
        plan = fc.peer_plan_exchange(torch.from_numpy(lecs[rank]).to(dev), None, cap, E)
        assert plan is not None and torch.equal(plan.table.cpu(), torch.from_numpy(table))
        own = np.concatenate([[0], np.cumsum(gecs[rank].reshape(world, E).sum(0))])
        assert np.array_equal(plan.own_offsets.cpu().numpy(), own)
        out = fc.peer_scatter_planned(mine + rnd, plan, cap)
        assert torch.equal(out[:recv], torch.from_numpy(want[rank]).to(dev) + rnd), "planned scatter layout"
        back = fc.peer_gather_planned(out, plan, mine.shape[0] + 3)
        assert torch.equal(back[:-3], mine + rnd) and not back[-3:].any(), "planned gather is not the inverse"
    assert fc.device_status(dev) == 0
    # rank 0 announces one row less than it would receive
    cap = want[0].shape[0] - 1 if rank == 0 else recv + 1
    plan = fc.peer_plan_exchange(torch.from_numpy(lecs[rank]).to(dev), None, max(cap, 0), E)
    assert plan.read(0)[3] == 1 and not plan.own_offsets.any()
    out = fc._recv_empty(mine, recv + 1)
    out.fill_(3.0)
    with torch.cuda.device(dev):
        assert fc.lib.fmoe_peer_scatter_planned(fc._comm(dev), fc._ptr(mine), fc._ptr(out), fc._ptr(plan.buf), mine.shape[0],
                                                recv + 1, d * 4, E, fc._stream()) == 0
    assert bool((out == 3).all()), "rows moved although a rank had no room"
    assert fc.device_status(dev) & 64
    assert fc.lib.fmoe_device_status_clear() == 0
    dist.barrier()


def _make_layer(world, rank, E, d, h, k, act, bias, tens, dtype=torch.float32, gate=None):
    from fastermoe_b200 import FMoETransformerMLP
    fn = {"gelu": torch.nn.GELU(), "relu": torch.nn.ReLU()}[act]
    kw = {} if gate is None else {"gate": gate}
    m = FMoETransformerMLP(num_expert=E, d_model=d, d_hidden=h, world_size=world, activation=fn, top_k=k, bias=bias, **kw)
    sl = slice(rank * E, (rank + 1) * E)
    with torch.no_grad():
        m.gate.gate.weight.copy_(tens["gate_w"]); m.gate.gate.bias.copy_(tens["gate_b"])
        m.experts.htoh4.weight.copy_(tens["w1"][sl]); m.experts.h4toh.weight.copy_(tens["w2"][sl])
        if bias:
            m.experts.htoh4.bias.copy_(tens["b1"][sl]); m.experts.h4toh.bias.copy_(tens["b2"][sl])
    return m.to(dtype).cuda()


def _run_layer(m, x, loss_weight=None):
    m.zero_grad(set_to_none=True)
    x = x.detach().clone().requires_grad_(True)
    out = m(x)
    (out.sum() if loss_weight is None else (out * loss_weight).sum()).backward()
    g = {"out": out.detach(), "x": x.grad, "w1": m.experts.htoh4.weight.grad.clone(),
         "w2": m.experts.h4toh.weight.grad.clone(), "gate_w": m.gate.gate.weight.grad.clone()}
    if m.experts.htoh4.bias is not None:
        g["b1"], g["b2"] = m.experts.htoh4.bias.grad.clone(), m.experts.h4toh.bias.grad.clone()
    return g


def gpu_layer(rank, world, port):
    init(rank, world, port, "nccl")
    check_layer(rank, world)
    finish("nccl")


def check_layer(rank, world):
    """Expert-parallel layer against the brute-force oracle; smart schedule == plain schedule;
    shadowed == not shadowed (the reference's tests/test_fused.py and tests/test_cache.py)."""
    import fastermoe_b200.transformer as tr
    T, d, h, E, k = 96, 64, 128, 2, 2
    tens = O.make_layer_inputs(T * world, d, h, E * world, seed=3)
    xs = tens["x"].view(world, T, d)
    tol = dict(rtol=1e-5, atol=5e-5)
    for act, bias in (("gelu", True), ("relu", False)):
        m = _make_layer(world, rank, E, d, h, k, act, bias, tens)
        got = _run_layer(m, xs[rank].cuda())
        # oracle: every rank's tokens through all experts; expert grads summed over ranks
        wants = [O.moe_layer_fwd_bwd(xs[r], tens["gate_w"], tens["gate_b"], tens["w1"], tens["b1"] if bias else None,
                                     tens["w2"], tens["b2"] if bias else None, k, act=act) for r in range(world)]
        sl = slice(rank * E, (rank + 1) * E)
        torch.testing.assert_close(got["out"].cpu(), wants[rank]["out"], **tol)
        torch.testing.assert_close(got["x"].cpu(), wants[rank]["grad_x"], **tol)
        torch.testing.assert_close(got["gate_w"].cpu(), wants[rank]["grad_gate_w"], rtol=1e-5, atol=2e-4)
        for name in ("w1", "w2") + (("b1", "b2") if bias else ()):
            want = sum(w["grad_" + name][sl] for w in wants)
            torch.testing.assert_close(got[name].cpu(), want, rtol=1e-5, atol=2e-4, msg=lambda s, n=name: f"{n}: {s}")
        # the same layer when the host reads the counts (no device-built plan): bit-identical
        os.environ["FMOE_B200_NOSYNC"] = "0"
        synced = _run_layer(m, xs[rank].cuda())
        os.environ["FMOE_B200_NOSYNC"] = "1"
        for name, v in got.items():
            assert torch.equal(synced[name], v), f"host-planned and device-planned exchange differ in {name}"
        # smart schedule against the plain one, all pipeline granularities
        m.enable_fuse = True          # nothing shadowed: the flag selects the device-planned path itself
        same = _run_layer(m, xs[rank].cuda())
        m.enable_fuse = False
        for name, v in got.items():
            assert torch.equal(same[name], v), f"smart-schedule flag without shadows differs in {name}"
        for gran in ("1", "2", "4"):
            os.environ["FMOE_FUSE_GRAN"] = gran
            m.enable_fuse = True
            with switches(SMART="nccl"):
                fused = _run_layer(m, xs[rank].cuda())
            m.enable_fuse = False
            for name, v in got.items():
                torch.testing.assert_close(fused[name], v, rtol=1e-5, atol=2e-5, msg=lambda s, n=name: f"fused {gran} {n}: {s}")
        # dynamic shadowing: force worker 0 (then the last worker) to be shadowed everywhere
        for hot in (0, world - 1):
            def policy(aec, agec, num_expert, world_size, d_model, fused, hot=hot):
                res = torch.zeros(world_size, num_expert, dtype=torch.bool)
                res[hot] = True
                return res
            m.policy_fn = policy
            for fuse in (False, True):
                m.enable_fuse = fuse
                shadow = _run_layer(m, xs[rank].cuda())
                for name, v in got.items():
                    torch.testing.assert_close(shadow[name], v, rtol=1e-5, atol=5e-5,
                                               msg=lambda s, n=name: f"shadow hot={hot} fuse={fuse} {n}: {s}")
            m.enable_fuse = False
            m.policy_fn = tr._gen_policy(h / d)


def gpu_layer_bf16(rank, world, port):
    init(rank, world, port, "nccl")
    check_layer_bf16(rank, world)
    finish("nccl")


def fc_nosync(x, world, top_k):
    """Rows the layer would give its expert-side buffers on the device-planned path (0: that path is off)."""
    from fastermoe_b200 import fmoe_cuda as fc
    if os.environ.get("FMOE_B200_NOSYNC", "1") == "0":
        return 0
    return fc.nosync_capacity(x.shape[0] * top_k, x.shape[1] * x.element_size(), world, x.device)


@contextlib.contextmanager
def switches(**kv):
    """Sets FMOE_B200_<NAME> switches for a block and puts the previous values back."""
    old = {k: os.environ.get("FMOE_B200_" + k) for k in kv}
    try:
        for k, v in kv.items():
            os.environ["FMOE_B200_" + k] = str(v)
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop("FMOE_B200_" + k, None)
            else:
                os.environ["FMOE_B200_" + k] = v


def check_layer_bf16(rank, world):
    """bf16 shapes that take the tensor-core kernels, smart schedule and shadowing included."""
    from parity import assert_half_close, rms
    T, d, h, E, k = 1024, 256, 512, 2, 2
    tens = O.make_layer_inputs(T * world, d, h, E * world, seed=4, gate_std=0.02)
    xs = tens["x"].view(world, T, d)
    m = _make_layer(world, rank, E, d, h, k, "gelu", True, tens, dtype=torch.bfloat16)
    x = xs[rank].bfloat16().cuda()
    with switches(OVERLAP_SMS=0, FUSED_GATHER=0, FUSED_SCATTER=0, FUSED_PUSH=0):      # local scatter, push, GEMMs, push
        base = _run_layer(m, x)
    with torch.no_grad():
        idx, _ = m.gate(x)
    idx_all = [torch.empty_like(idx) for _ in range(world)]
    dist.all_gather(idx_all, idx)
    r = {n: t.bfloat16().float() for n, t in tens.items()}
    want = O.moe_layer_fwd_bwd(r["x"].view(world, T, d)[rank], r["gate_w"], r["gate_b"], r["w1"], r["b1"], r["w2"],
                               r["b2"], k, gate_idx=idx.cpu())
    assert_half_close(base["out"], want["out"], 4, "out")
    assert_half_close(base["x"], want["grad_x"], 5, "grad_x")

    def same_up_to_rounding(a, b_, name, roundings):
        # two 16-bit runs that order their (fp32) sums differently, e.g. per pipeline step
        torch.testing.assert_close(a.float(), b_.float(), rtol=2e-2, atol=8 * roundings * 2.0 ** -9 * rms(b_),
                                   msg=lambda s_: f"{name}: {s_}")
    # the scatter's push running beside the GEMM that reads its rows: same bits
    for sms in ("4", "16"):
        with switches(OVERLAP_SMS=sms, FUSED_GATHER=0):
            for _ in range(2):
                over = _run_layer(m, x)
        for name, v in base.items():
            assert torch.equal(over[name], v), f"overlapped exchange ({sms} SMs) differs in {name}"
    # the gather done by the GEMM that produces its rows (stores into the owners' buffers): same bits,
    # alone and together with an overlapped scatter
    for sms in ("0", "8"):
        with switches(OVERLAP_SMS=sms, FUSED_GATHER=1, FUSED_SCATTER=0):
            for _ in range(2):
                over = _run_layer(m, x)
        for name, v in base.items():
            assert torch.equal(over[name], v), f"gather fused into the GEMM (scatter on {sms} SMs) differs in {name}"
    # the scatters' pushes picking (forward) and scaling (backward) their rows themselves: same bits,
    # also with an output gradient that differs from element to element
    lw = torch.randn(x.shape, generator=torch.Generator().manual_seed(7 + rank)).to(x)
    with switches(OVERLAP_SMS=0, FUSED_GATHER=0, FUSED_SCATTER=0):
        base_w = _run_layer(m, x, lw)
    for fg in ("0", "1"):
        with switches(OVERLAP_SMS=0, FUSED_GATHER=fg, FUSED_SCATTER=1):
            for _ in range(2):
                over = _run_layer(m, x)
            over_w = _run_layer(m, x, lw)
        for name, v in base.items():
            assert torch.equal(over[name], v), f"scatter that produces its rows (fused gather {fg}) differs in {name}"
            assert torch.equal(over_w[name], base_w[name]), f"scatter that scales its rows (fused gather {fg}) differs in {name}"
    # the scatters done by the GEMMs that consume their rows (spare warps push, tensor-core warps wait per expert)
    with switches(OVERLAP_SMS=0, FUSED_GATHER=1, FUSED_SCATTER=1, FUSED_PUSH=1):
        for _ in range(3):
            over = _run_layer(m, x)
        over_w = _run_layer(m, x, lw)
    for name, v in base.items():
        assert torch.equal(over[name], v), f"scatter fused into the consuming GEMM differs in {name}"
        assert torch.equal(over_w[name], base_w[name]), f"scaled scatter fused into the consuming GEMM differs in {name}"
    # the quiet-point hook: once after the forward's scatter, once after the backward's
    from fastermoe_b200 import set_phase_hook
    calls = []
    set_phase_hook(calls.append)
    try:
        with switches(OVERLAP_SMS=0, FUSED_PUSH=0):
            _run_layer(m, x)
    finally:
        set_phase_hook(None)
    # (with a receive pool too small for the device-planned path the layer reads the counts back and the
    # hook stays silent)
    planned = fc_nosync(x, world, k) > 0
    assert calls == (["scatter_done", "scatter_done"] if planned else []), calls
    from fastermoe_b200 import fmoe_cuda as fc
    assert fc.device_status() == 0
    os.environ["FMOE_FUSE_GRAN"] = "1"
    m.enable_fuse = True
    with switches(SMART="nccl"):
        fused = _run_layer(m, x)
    m.enable_fuse = False
    for name in ("out", "x", "w1", "w2", "b1", "b2"):
        # the smart schedule accumulates weight gradients step by step in 16 bits
        same_up_to_rounding(fused[name], base[name], "fused " + name, 1 if name in ("out", "x") else world)

    def policy(aec, agec, num_expert, world_size, d_model, fused):
        res = torch.zeros(world_size, num_expert, dtype=torch.bool)
        res[0] = True
        return res
    m.policy_fn = policy
    shadow = _run_layer(m, x)
    for name in ("out", "x", "w1", "w2", "b1", "b2"):
        # shadowed experts' gradients are reduced over the ranks in 16 bits
        same_up_to_rounding(shadow[name], base[name], "shadow " + name, 1 if name in ("out", "x") else world)


def gpu_graph_step(rank, world, port):
    init(rank, world, port, "nccl")
    check_graph_step(rank, world)
    finish("nccl")


def check_graph_step(rank, world):
    """A whole expert-parallel forward+backward step replayed as one CUDA graph on every rank equals the
    eager step, also when the routing of the replayed batch differs from the captured one."""
    from fastermoe_b200 import GraphedStep
    T, d, h, E, k = 1000, 256, 512, 2, 2
    tens = O.make_layer_inputs(T * world, d, h, E * world, seed=8, gate_std=0.5)
    m = _make_layer(world, rank, E, d, h, k, "gelu", True, tens, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(100 + rank)
    xs = [torch.randn(T, d, generator=g).bfloat16().cuda() for _ in range(3)]

    def eager(x):
        m.zero_grad(set_to_none=True)
        xi = x.clone().requires_grad_(True)
        out = m(xi)
        loss = out.sum(dtype=torch.float32)
        loss.backward()
        return out.detach().clone(), loss.detach().clone(), xi.grad.clone(), {n: p.grad.clone() for n, p in m.named_parameters()}

    with switches(OVERLAP_SMS=0, FUSED_GATHER=0, FUSED_SCATTER=0, FUSED_PUSH=0):
        want = [eager(x) for x in xs[1:]]
    # without and with the pushes running beside the GEMMs (a second stream in the graph), and with
    # the gathers done by the GEMMs' own epilogues
    for sms, fused_gather, fused_scatter, fused_push in (("0", "0", "0", "0"), ("8", "0", "0", "0"), ("0", "1", "0", "0"),
                                                         ("0", "1", "1", "0"), ("0", "1", "1", "1")):
        with switches(OVERLAP_SMS=sms, FUSED_GATHER=fused_gather, FUSED_SCATTER=fused_scatter, FUSED_PUSH=fused_push):
            step = GraphedStep(m, xs[0], input_grad=True)
            for x, (out, loss, gx, grads) in zip(xs[1:], want):
                got_loss = step(x)
                torch.cuda.synchronize()
                assert torch.equal(step.output, out) and torch.equal(got_loss, loss)
                assert torch.equal(step.input_grad, gx)
                for n, p in m.named_parameters():
                    assert torch.equal(p.grad, grads[n]), n
        del step
    from fastermoe_b200 import fmoe_cuda as fc
    assert fc.device_status() == 0
    dist.barrier()


def gpu_config5(rank, world, port):
    init(rank, world, port, "nccl")
    check_config5(rank, world)
    finish("nccl")


def check_config5(rank, world):
    """Dynamic shadowing driven by the real cost-model policy (fmoe/transformer.py:33-86, the reference's
    constants) + capacity limit + topology-aware gate, in both orders: the capacity cuts every expert
    (the policy then sees balanced counts), or experts the policy replicates are spared from the
    capacity (the shadow path is active).  Small fp32 shapes; one expert receives most rows."""
    import math
    from fastermoe_b200 import FMoETransformerMLP
    from fastermoe_b200.gates import gen_hir_capacity_gate
    T, d, h, E, k = 1024, 64, 256, 2, 2
    wpn = max(world // 2, 1)
    tens = O.make_layer_inputs(T * world, d, h, E * world, seed=5, gate_std=0.1)
    tens["gate_b"] = torch.zeros(E * world)
    tens["gate_b"][0] = 2.0                                 # expert 0 (on worker 0) is hot
    xs = tens["x"].view(world, T, d)
    cap = math.ceil(1.2 * T)
    env = {n: os.environ.get(n) for n in ("FMOE_ENABLE_DYNREP", "FMOE_POLICY_CONSTANTS")}
    os.environ["FMOE_ENABLE_DYNREP"], os.environ["FMOE_POLICY_CONSTANTS"] = "1", "reference"
    shadowed_any = {}
    try:
        for spare in (False, True):
            m = _make_layer(world, rank, E, d, h, k, "gelu", True, tens,
                            gate=gen_hir_capacity_gate(rank, wpn, 1.2, spare_shadowed=spare))
            seen = {}
            m.gate_hook = lambda idx, score, _x: seen.update(idx=idx.detach().clone())
            got = _run_layer(m, xs[rank].cuda())
            final, sel = seen["idx"], m.gate.last_selection
            finals = [torch.empty_like(final) for _ in range(world)]
            sels = [torch.empty_like(sel) for _ in range(world)]
            dist.all_gather(finals, final)
            dist.all_gather(sels, sel)
            # what the gate's policy saw (raw counts) and decided
            raw = np.stack([O.expert_count(torch.topk(torch.nn.functional.linear(xs[r], tens["gate_w"], tens["gate_b"]), 2)[1].numpy(),
                                           world * E).reshape(world, E) for r in range(world)]).astype(np.int64)
            want_stored = O.global_policy(raw, raw.transpose(1, 0, 2), E, world, d, True, h / d)
            assert np.array_equal(m.gate.last_stored.numpy(), want_stored), "shadowing policy decision"
            shadowed_any[spare] = bool(want_stored.any())
            kept = sum(O.expert_count(f.cpu().numpy(), world * E).astype(np.int64) for f in finals)
            for e in range(world * E):
                if not (spare and want_stored.reshape(-1)[e]):
                    assert kept[e] <= cap, f"expert {e} kept {kept[e]} rows, capacity {cap}"
            wants = [O.moe_layer_fwd_bwd(xs[r], tens["gate_w"], tens["gate_b"], tens["w1"], tens["b1"], tens["w2"],
                                         tens["b2"], k, softmax_scores=True, gate_idx=finals[r].cpu(), score_idx=sels[r].cpu())
                     for r in range(world)]
            sl = slice(rank * E, (rank + 1) * E)
            tol = dict(rtol=1e-5, atol=5e-5)
            torch.testing.assert_close(got["out"].cpu(), wants[rank]["out"], **tol)
            torch.testing.assert_close(got["x"].cpu(), wants[rank]["grad_x"], **tol)
            for name in ("w1", "w2", "b1", "b2"):
                want = sum(w["grad_" + name][sl] for w in wants)
                torch.testing.assert_close(got[name].cpu(), want, rtol=1e-5, atol=1e-5 * float(want.abs().max()) + 2e-4,
                                           msg=lambda s_, n=name: f"spare={spare} {n}: {s_}")
    finally:
        for n, v in env.items():
            if v is None:
                os.environ.pop(n, None)
            else:
                os.environ[n] = v
    assert shadowed_any[True], "the policy was expected to replicate the hot worker on the raw counts"
    return shadowed_any


# ------------------------------------------------------------------ CPU / gloo

def gpu_full_size(rank, world, port):
    """The Zipf-routed (4 experts, d 2048, h 8192) and the one-expert (d 4096, h 16384) workloads at their
    per-GPU sizes, checked through properties that need no CPU oracle of that size: the exchange over peer
    memory and over NCCL give bit-identical layers; the smart schedule equals the plain schedule
    within bf16 rounding; gradients are finite; no bounded wait expired."""
    init(rank, world, port, "nccl")
    from fastermoe_b200 import FMoETransformerMLP, fmoe_cuda as fc
    import fastermoe_b200.functions as F
    dev = torch.device("cuda", rank)

    def build(E, d, h, seed, zipf):
        g = torch.Generator().manual_seed(seed)
        m = FMoETransformerMLP(num_expert=E, d_model=d, d_hidden=h, world_size=world, top_k=2, activation=torch.nn.GELU())
        with torch.no_grad():
            m.gate.gate.weight.copy_(torch.randn(E * world, d, generator=g) * 0.02)
            m.gate.gate.bias.zero_()
            if zipf:      # expert popularity ~ rank^-1.2
                m.gate.gate.bias.copy_(-1.2 * torch.log(torch.arange(1, E * world + 1).float()))
            ge = torch.Generator().manual_seed(seed * 1000 + rank)
            for lin, fan in ((m.experts.htoh4, d), (m.experts.h4toh, h)):
                lin.weight.copy_((torch.rand(lin.weight.shape, generator=ge) * 2 - 1) / fan ** 0.5)
                lin.bias.copy_((torch.rand(lin.bias.shape, generator=ge) * 2 - 1) / fan ** 0.5)
        return m.bfloat16().to(dev)

    def status():
        st = ctypes.c_int32(-1)
        assert fc.lib.fmoe_device_status(ctypes.byref(st)) == 0
        return st.value

    # configuration 3: 4 experts per GPU, d_model 2048, d_hidden 8192, 8192 tokens per GPU, Zipf routing
    m = build(4, 2048, 8192, 2, zipf=True)
    x = torch.randn(8192, 2048, generator=torch.Generator().manual_seed(20 + rank)).bfloat16().to(dev)
    peer = _run_layer(m, x)
    if fc.peer_slot_bytes(dev) > 0:
        plain_exchange = F.Exchange.__init__

        def without_table(self, lec, gec, stored, fwd_batch_size, world_size, table=None):
            plain_exchange(self, lec, gec, stored, fwd_batch_size, world_size, table=None)
        F.Exchange.__init__ = without_table
        os.environ["FMOE_B200_NOSYNC"] = "0"          # counts read back, rows over NCCL send/receive
        try:
            nccl = _run_layer(m, x)
        finally:
            F.Exchange.__init__ = plain_exchange
            os.environ["FMOE_B200_NOSYNC"] = "1"
        for name, v in peer.items():
            assert torch.equal(nccl[name], v), f"config 3: peer-memory and NCCL exchange differ in {name}"
    for name, v in peer.items():
        assert torch.isfinite(v.float()).all(), f"config 3: {name} not finite"
    assert status() == 0
    del m, peer
    torch.cuda.empty_cache()

    # configuration 4: smart schedule, 1 expert per GPU, d_model 4096, d_hidden 16384, 16384 tokens per GPU
    m = build(1, 4096, 16384, 3, zipf=False)
    x = torch.randn(16384, 4096, generator=torch.Generator().manual_seed(30 + rank)).bfloat16().to(dev)
    plain = _run_layer(m, x)
    os.environ["FMOE_FUSE_GRAN"] = "1"
    m.enable_fuse = True
    with switches(SMART="nccl"):
        fused = _run_layer(m, x)
    m.enable_fuse = False
    for name, v in plain.items():
        assert torch.isfinite(v.float()).all(), f"config 4: {name} not finite"
        scale = float(v.float().abs().mean()) + 1e-6
        torch.testing.assert_close(fused[name].float(), v.float(), rtol=2e-2, atol=2e-2 * scale * 8,
                                   msg=lambda s_, n=name: f"config 4 smart schedule vs plain, {n}: {s_}")
    assert status() == 0
    finish("nccl")


def cpu_plan_exchange(rank, world, port):
    """Executes the library's exchange plan with gloo point-to-point on CPU tensors and
    compares with the oracle: the host-side planning that the NCCL executor follows."""
    import ctypes
    init(rank, world, port, "gloo")
    from fastermoe_b200 import _lib
    E, d = 3, 8
    lecs = all_lecs(world, E, 21)
    _, _, gecs = O.expert_exchange(lecs, E, world)
    # count exchange through the process group, as the layer does through NCCL
    mine = torch.from_numpy(lecs[rank])
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    aec = torch.stack(gathered).view(world, world, E)
    assert np.array_equal(aec.transpose(0, 1)[rank].reshape(-1).numpy(), gecs[rank])
    for stored in (np.zeros(world * E, bool), np.repeat(np.arange(world) == 1, E)):
        rng = np.random.default_rng(2)
        bufs = [rng.standard_normal((int(l.sum()), d)).astype(np.float32) for l in lecs]
        want = O.global_scatter(bufs, lecs, stored, E, world)
        lec = np.ascontiguousarray(lecs[rank], dtype=np.int64)
        gec = np.ascontiguousarray(gecs[rank], dtype=np.int64)
        st = stored.astype(np.uint8)
        moves = (_lib.Move * (4 * E * world + 8))()
        n, rows = ctypes.c_int32(), ctypes.c_int64()
        rc = _lib.lib.fmoe_plan_global_scatter(lec.ctypes.data, gec.ctypes.data, st.ctypes.data, rank, E, world,
                                               ctypes.cast(moves, ctypes.c_void_p), len(moves), ctypes.byref(n),
                                               ctypes.byref(rows))
        assert rc == 0 and rows.value == want[rank].shape[0]
        src = torch.from_numpy(bufs[rank])
        dst = torch.zeros(rows.value, d)
        ops = []
        for i in range(n.value):
            m = moves[i]
            if m.local:
                dst[m.dst_row:m.dst_row + m.rows] = src[m.src_row:m.src_row + m.rows]
            elif m.is_send:
                ops.append(dist.P2POp(dist.isend, src[m.src_row:m.src_row + m.rows].contiguous(), m.peer))
            else:
                ops.append(dist.P2POp(dist.irecv, dst[m.dst_row:m.dst_row + m.rows], m.peer))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        assert np.array_equal(dst.numpy(), want[rank]), f"rank {rank}: plan does not reproduce the reference layout"
        # shadow bookkeeping on the host
        from fastermoe_b200.functions import cached_count_host
        cc = cached_count_host(torch.from_numpy(lec.copy()), torch.from_numpy(gec.copy()), torch.from_numpy(stored),
                               rank, E, world)
        assert np.array_equal(cc.numpy(), O.generate_cached_count(lec, gec, stored, rank, E, world))
        assert int(cc.sum()) == rows.value
        geo = _lib.FusedGeometry()
        for gran in (1, 2, 3, 4):
            assert _lib.lib.fmoe_fused_geometry(lec.ctypes.data, gec.ctypes.data, st.ctypes.data, rank, E, world, gran,
                                                ctypes.byref(geo)) == 0
            assert world % geo.gran == 0 and geo.n_steps * geo.gran == world and geo.gran <= max(gran, 1)
            assert geo.global_rows + geo.shadow_rows == rows.value
    finish("gloo")


def cpu_grouped_ddp(rank, world, port):
    """DistributedGroupedDataParallel: gradients are averaged per tag; 'none' is left alone."""
    init(rank, world, port, "gloo")
    from fastermoe_b200.distributed import DistributedGroupedDataParallel
    torch.manual_seed(rank)
    net = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.Linear(4, 2))
    for p in net[0].parameters():
        p.dp_comm = "moe"
    for p in net[1].parameters():
        p.dp_comm = "none"
    ddp = DistributedGroupedDataParallel(net)
    w0 = [torch.empty_like(net[0].weight) for _ in range(world)]
    dist.all_gather(w0, net[0].weight.data)
    assert all(torch.equal(w0[0], w) for w in w0), "tagged parameters were not broadcast"
    ddp(torch.randn(3, 4)).sum().backward()
    g_local = net[0].weight.grad.clone()
    g_none = net[1].weight.grad.clone()
    gs = [torch.empty_like(g_local) for _ in range(world)]
    dist.all_gather(gs, g_local)
    ddp.allreduce_params()
    torch.testing.assert_close(net[0].weight.grad, sum(gs) / world)
    assert torch.equal(net[1].weight.grad, g_none)
    finish("gloo")


def cpu_megatron_ddp_checkpoint(rank, world, port, root):
    """The Megatron-style wrapper on real ranks: gradients of replicated tensors are averaged over the
    data-parallel group, expert tensors are left alone; every rank then writes its checkpoint shard and a
    rank other than 0 gets back rank 0's replicated tensors with its own experts (optimizer state included)."""
    init(rank, world, port, "gloo")
    from fastermoe_b200 import megatron as M

    class Mpu:
        def get_model_parallel_group(self):
            return None

        def get_data_parallel_group(self):
            return dist.group.WORLD

    M.bind(mpu=Mpu())
    torch.manual_seed(rank)
    net = torch.nn.ModuleDict({"shared": torch.nn.Linear(4, 4), "experts": torch.nn.Linear(4, 4)})
    for p in net["shared"].parameters():
        p.dp_comm = "dp"
    for p in net["experts"].parameters():
        p.dp_comm = "none"
    ddp = M.DistributedDataParallel(net)                       # broadcasts the replicated tensors from rank 0
    opt = torch.optim.Adam(net.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(50 + rank)
    for _ in range(3):
        opt.zero_grad()
        (net["experts"](net["shared"](torch.randn(5, 4, generator=g))) ** 2).sum().backward()
        ddp.allreduce_params()
        opt.step()
    shared = [torch.empty_like(net["shared"].weight) for _ in range(world)]
    dist.all_gather(shared, net["shared"].weight.data)
    assert all(torch.allclose(shared[0], w) for w in shared), "replicated tensors drifted apart"
    experts = [torch.empty_like(net["experts"].weight) for _ in range(world)]
    dist.all_gather(experts, net["experts"].weight.data)
    assert not torch.allclose(experts[0], experts[1]), "expert tensors were averaged"
    assert set(ddp.state_dict()) == set(net.state_dict())       # the wrapper's state dict is the module's

    pos = M.GridPosition(dp_rank=rank)
    M.save_shard(root, 3, net, opt, pos)
    dist.barrier()
    if rank == 0:
        M.write_tracker(root, 3)
    dist.barrier()
    want = {k: v.clone() for k, v in net.state_dict().items()}
    want_opt = opt.state_dict()["state"]
    with torch.no_grad():
        for p in net.parameters():
            p.add_(1.0)                                         # what the load must undo
    opt2 = torch.optim.Adam(net.parameters(), lr=0.05)
    blob = M.load_shard(root, net, opt2, pos)
    assert blob["iteration"] == 3
    for k, v in net.state_dict().items():
        assert torch.equal(v, want[k]), k
    got_opt = opt2.state_dict()["state"]
    for i in (2, 3):                                            # this rank's experts: its own moments
        assert torch.equal(got_opt[i]["exp_avg"], want_opt[i]["exp_avg"])
    M.unbind()
    finish("gloo")


def cpu_megatron_named_checkpoint(rank, world, port, root):
    """save_checkpoint / load_checkpoint with the reference's signatures, inside a process that has a module
    named ``megatron`` (a stand-in with the attributes those functions use): data-parallel rank 0 goes through
    the host framework's own functions, the other rank writes and reads its expert shard."""
    import types
    init(rank, world, port, "gloo")
    native = {"saved": 0, "loaded": 0}
    args = types.SimpleNamespace(save=root, load=root, no_save_optim=False, no_load_optim=False, finetune=False)
    mpu = types.SimpleNamespace(get_data_parallel_rank=lambda: rank, get_tensor_model_parallel_rank=lambda: 0,
                                get_pipeline_model_parallel_rank=lambda: 0,
                                get_pipeline_model_parallel_world_size=lambda: 1)
    from fastermoe_b200.megatron import checkpoint as C

    def native_save(iteration, model, optimizer, lr_scheduler):
        native["saved"] += 1
        C.save_shard(root, iteration, model, optimizer, C.GridPosition(0), extra={"lr_scheduler": {"step": iteration}})
        dist.barrier()
        C.write_tracker(root, iteration)
        dist.barrier()

    def native_load(model, optimizer, lr_scheduler, load_arg="load"):
        native["loaded"] += 1
        blob = C.load_shard(root, model, optimizer, C.GridPosition(0))
        dist.barrier()
        return blob["iteration"]

    fake = types.ModuleType("megatron")
    fake.get_args, fake.mpu = (lambda: args), mpu
    fake.checkpointing = types.ModuleType("megatron.checkpointing")
    fake.checkpointing.save_checkpoint, fake.checkpointing.load_checkpoint = native_save, native_load
    sys.modules["megatron"], sys.modules["megatron.checkpointing"] = fake, fake.checkpointing
    try:
        torch.manual_seed(7 + rank)
        net = torch.nn.ModuleDict({"shared": torch.nn.Linear(3, 3), "experts": torch.nn.Linear(3, 3)})
        for p in net["experts"].parameters():
            p.dp_comm = "none"
        with torch.no_grad():                                  # replicated tensors agree, experts differ
            for p in net["shared"].parameters():
                p.copy_(torch.full_like(p, 0.5))
        opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9)
        (net["experts"](net["shared"](torch.ones(2, 3))) ** 2).sum().backward()
        for p in net["shared"].parameters():                   # what data parallelism does for replicated tensors
            dist.all_reduce(p.grad)
            p.grad /= world
        opt.step()
        want = {k: v.clone() for k, v in net.state_dict().items()}

        class Sched:
            state = None

            def load_state_dict(self, sd):
                self.state = sd

        C.save_checkpoint(12, net, opt, None)
        assert native["saved"] == (1 if rank == 0 else 0)
        assert os.path.isfile(C.checkpoint_name(root, 12, C.GridPosition(rank)))
        with torch.no_grad():
            for p in net.parameters():
                p.zero_()
        sched = Sched()
        it = C.load_checkpoint(net, torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9), sched)
        assert it == 12 and native["loaded"] == (1 if rank == 0 else 0)
        for k, v in net.state_dict().items():
            assert torch.equal(v, want[k]), k
        if rank > 0:
            assert sched.state == {"step": 12}                 # the scheduler's state comes from rank 0's file
    finally:
        sys.modules.pop("megatron", None)
        sys.modules.pop("megatron.checkpointing", None)
    finish("gloo")


def cpu_slice_allgather(rank, world, port):
    """Slice / AllGather over a model-parallel group (fmoe/functions.py:333-375): the forward of one is
    the backward of the other."""
    init(rank, world, port, "gloo")
    from fastermoe_b200.functions import AllGather, Slice
    group = dist.group.WORLD
    rows = 3
    x = torch.arange(world * rows * 4, dtype=torch.float32).view(world * rows, 4).requires_grad_(True)   # the same on every rank
    mine = Slice.apply(x, rank, world, group)
    assert torch.equal(mine, x.detach()[rank * rows:(rank + 1) * rows])
    full = AllGather.apply(mine * (rank + 1), rank, world, group)
    want = torch.cat([x.detach()[r * rows:(r + 1) * rows] * (r + 1) for r in range(world)])
    assert torch.equal(full.detach(), want)
    full.sum().backward()
    # AllGather.backward keeps this rank's slice of the gradient, Slice.backward gathers the slices
    assert torch.equal(x.grad, torch.cat([torch.full((rows, 4), float(r + 1)) for r in range(world)]))
    finish("gloo")
