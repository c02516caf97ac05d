#!/usr/bin/env python
r"""MoE layer forward+backward throughput (tokens/s) on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config c2|c3|c4|c5] [--extra c3,c4,c5|none] [--no-parity]

Workloads (all synthetic, seeded; "per GPU" sizes, experts sharded over the ranks):

  c2  16384 tokens, d_model 1024, d_hidden 4096, 16 experts per GPU, top-2, bf16, GELU, bias,
      NaiveGate with weight ~ N(0, 0.02): near-uniform routing.  THE HEADLINE: N = 1 runs it as is,
      N > 1 (torch.distributed.run, one rank per GPU) keeps the per-GPU work: weak scaling.
  c3  8192 tokens, d 2048, h 8192, 4 experts per GPU, gate bias -1.2 ln(rank of expert): Zipf(1.2)
      popularity, the first GPU owns the popular experts.
  c4  16384 tokens, d 4096, h 16384, 1 expert per GPU, two distinct experts per token drawn uniformly,
      ReLU, no bias; FMOE_ENABLE_FUSE=1, measured in both forms the flag can select: the exchange fused
      with the GEMMs on the device-planned path, and the reference-shaped NCCL pipeline (FMOE_B200_SMART=nccl).
  c5  8192 tokens, d 1024, h 4096, 2 experts per GPU, one expert receives 40 % of all assignments,
      capacity ceil(1.2 x tokens) per expert, topology-aware HirGate (2 groups of GPUs), dynamic
      shadowing (FMOE_ENABLE_DYNREP=1), in both orders: capacity cuts every expert ("5a"), or experts
      the policy replicates are spared ("5b").

One "step" = forward + backward (loss = sum of the output) of the layer on one batch; where the step has
no host read (N = 1; N > 1 with the device-planned exchange) it is replayed as one CUDA graph through the
library's GraphedStep (``step_form``; ``eager_ms_per_step`` is the same step launched from Python, and
``--eager`` times that instead).  The printed
JSON line carries: ``value`` (device-resident inputs), ``e2e`` (inputs copied from pinned host memory
and the loss read back every step -- when the step replays as a CUDA graph, the host reads step i's
loss, copied to pinned memory, while the next two steps run), ``roofline`` of the dominant kernel (the grouped expert GEMM,
timed with CUDA events on the launching stream), ``cpu_baseline`` (the reference's CPU path on a
bounded sample of the same workload).  With N > 1 it also carries ``parity`` -- an untimed
self-check of the multi-GPU path against the CPU oracle, run after the timed region -- and, with N = 8
(or ``--extra``), ``configs``: the other workloads above, each timed with its own warm-up.

``--kernel-list PATH`` / ``--kernel-list-e2e PATH`` also write a per-kernel device-time table of a few
resident / e2e steps (CUPTI through torch.profiler; works on every rank count).  Progress markers go to
stderr.  ``--impl reference`` times the reference's own CPU path alone on the host cores.
All working sets are several hundred MB per step, larger than the 126 MB L2: no explicit flush.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    "c2": dict(tokens_per_gpu=16384, d_model=1024, d_hidden=4096, experts_per_gpu=16, top_k=2, seed=1,
               gate_std=0.02, activation="gelu", bias=True, routing="near-uniform (NaiveGate, weight~N(0,0.02))"),
    "c3": dict(tokens_per_gpu=8192, d_model=2048, d_hidden=8192, experts_per_gpu=4, top_k=2, seed=2,
               gate_std=0.02, zipf=1.2, activation="gelu", bias=True, routing="Zipf(1.2) by gate bias"),
    "c4": dict(tokens_per_gpu=16384, d_model=4096, d_hidden=16384, experts_per_gpu=1, top_k=2, seed=3,
               gate_std=0.02, uniform_pairs=True, activation="relu", bias=False,
               routing="two distinct experts per token, uniform"),
    "c5": dict(tokens_per_gpu=8192, d_model=1024, d_hidden=4096, experts_per_gpu=2, top_k=2, seed=4,
               gate_std=0.02, hot_share=0.4, capacity=1.2, activation="gelu", bias=True,
               routing="one expert gets 40 % of the assignments; HirGate; capacity 1.2; dynamic shadowing"),
}
CFG = CONFIGS["c2"]
CPU_SAMPLE_TOKENS = 2048
NVLINK_GBS = 770.0       # measured peer-copy bandwidth per direction per GPU on this pool (nominal 900)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self, t0=None, t1=None):
        """Summary of the samples taken between the wall-clock times t0 and t1 (all samples when none fall
        inside, or when no window is given)."""
        if self.proc is None:
            return None
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime
        rows = []
        for r in self.rows:
            try:
                ts = datetime.datetime.strptime(r[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
            except (ValueError, IndexError):
                ts = None
            rows.append((ts, r[1:]))
        inside = [r for ts, r in rows if ts is not None and t0 is not None and t1 is not None and t0 <= ts <= t1]
        window = "timed region" if inside else "whole run under load"
        clocks, reasons, mx = [], set(), None
        for r in (inside or [r for _, r in rows]):
            try:
                clocks.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return None
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks), "window": window}


# ------------------------------------------------------------------------------- CPU reference arm

def cpu_reference_run(steps, warmup, tokens):
    """The reference's pure-PyTorch brute-force MoE on ``tokens`` tokens of the headline workload, fp32,
    all host threads: its own NaiveGate (fmoe/gates/naive_gate.py:21-42) and BruteForceMoELinear
    (tests/moe.py:6-49) when a copy of the reference's Python package is staged under baseline/_ref
    (oracle/stage_reference.py; kind "reference"), else the oracle's restatement of them (kind "port").
    Returns (tokens/s, ms/step, threads, kind)."""
    import torch
    import types
    from oracle import moe_oracle as O
    from oracle import stage_reference
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    E, d, h, k = CFG["experts_per_gpu"], CFG["d_model"], CFG["d_hidden"], CFG["top_k"]
    tens = O.make_layer_inputs(tokens, d, h, E, seed=CFG["seed"], gate_std=CFG["gate_std"])
    ref = None
    try:
        ref = stage_reference.import_reference(types.ModuleType("fmoe_cuda"))
    except Exception:
        ref = None
    if ref is not None:
        from fmoe.gates.naive_gate import NaiveGate
        gate = NaiveGate(d, E, 1, top_k=k)
        moe = ref[1].BruteForceMoELinear(torch.nn.functional.gelu, num_expert=E, d_model=d, d_hidden=h, world_size=1, top_k=k)
        with torch.no_grad():
            gate.gate.weight.copy_(tens["gate_w"]); gate.gate.bias.copy_(tens["gate_b"])
            moe.weight_htoh4.copy_(tens["w1"]); moe.bias_htoh4.copy_(tens["b1"])
            moe.weight_h4toh.copy_(tens["w2"]); moe.bias_h4toh.copy_(tens["b2"])

        def step():
            for p in list(gate.parameters()) + list(moe.parameters()):
                p.grad = None
            x = tens["x"].clone().requires_grad_(True)
            idx, score = gate(x)
            moe(x, idx, score).sum().backward()
        kind = "reference"
    else:
        def step():
            O.moe_layer_fwd_bwd(tens["x"], tens["gate_w"], tens["gate_b"], tens["w1"], tens["b1"], tens["w2"],
                                tens["b2"], k, act=CFG["activation"])
        kind = "port"
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        step()
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    return tokens / (ms / 1e3), ms, threads, kind


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 10))
    warm = max(1, min(args.warmup, 2))
    val, ms, threads, kind = cpu_reference_run(steps, warm, CPU_SAMPLE_TOKENS)
    sample = (f"{CPU_SAMPLE_TOKENS} of {CFG['tokens_per_gpu']} tokens, same experts and widths, fp32 "
              f"(the reference has no bf16), {steps} timed fwd+bwd steps")
    print(json.dumps({
        "impl": "reference", "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config("c2", args.gpus),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(name, n_gpus):
    c = CONFIGS[name]
    return {"workload": f"benchmark config {name[1:]} per GPU: MoE MLP layer fwd+bwd, expert-parallel over the GPUs",
            "tokens_per_gpu": c["tokens_per_gpu"], "d_model": c["d_model"], "d_hidden": c["d_hidden"],
            "experts_per_gpu": c["experts_per_gpu"], "top_k": c["top_k"], "activation": c["activation"],
            "routing": c["routing"], "seed": c["seed"], "parallelism": f"ep{n_gpus}",
            "l2": "inputs larger than L2 (no flush)"}


def bind_to_gpu_cpus(local_rank):
    """Sets this process's CPU affinity to the cores NVML reports as local to its GPU (no-op on failure)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        index = int(visible.split(",")[local_rank]) if visible and visible.split(",")[local_rank].isdigit() else local_rank
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1}
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
    except Exception:
        pass


# ------------------------------------------------------------------------------- workloads

class Env:
    """Process-wide facts shared by the legs of a run."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        assert self.world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={self.world}; launch with torch.distributed.run"
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            # One process per GPU: run it (and allocate its pinned batch) on the CPUs next to its GPU, as a
            # launcher with NUMA binding would; otherwise the ranks' host-to-device copies cross sockets.
            bind_to_gpu_cpus(self.local_rank)
            # receive pools large enough for the largest workload of this run (see nosync_capacity)
            os.environ.setdefault("FMOE_B200_PEER_POOL_MB", "6144" if self.world >= 4 else "3072")
            import datetime
            dist.init_process_group("nccl", device_id=self.dev, timeout=datetime.timedelta(seconds=600))
        self.peaks = measured_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, steps, after=None):
        """ms for `steps` calls (and `after()`, if given, inside the timed region): CUDA events on the
        launching stream, barrier + synchronize on both sides, max over ranks."""
        torch = self.torch
        self.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        if after is not None:
            after()
        b.record()
        self.barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return float(ms.item())


def hot_bias_for_share(gate_w, share_tokens, seed, d):
    """Bias of expert 0's logit such that it is among a token's top-2 for `share_tokens` of the tokens
    (bisection on a fixed seeded sample: the same on every rank)."""
    import torch
    g = torch.Generator().manual_seed(seed + 999)
    logits = torch.randn(8192, d, generator=g) @ gate_w.t()
    lo, hi = 0.0, 20.0
    for _ in range(40):
        mid = 0.5 * (lo + hi)
        l2 = logits.clone()
        l2[:, 0] += mid
        frac = float((torch.topk(l2, 2, dim=1)[1] == 0).any(dim=1).float().mean())
        lo, hi = (mid, hi) if frac < share_tokens else (lo, mid)
    return 0.5 * (lo + hi)


def build_layer(env, name, variant=None):
    """Layer + pinned host batch of workload `name`.  variant: c4 "fuse" (FMOE_ENABLE_FUSE=1) / "nccl" (the same
    flag with FMOE_B200_SMART=nccl: the reference-shaped NCCL pipeline); c5 "5a"/"5b"."""
    import torch
    from fastermoe_b200 import FMoETransformerMLP
    from fastermoe_b200.gates import NaiveGate, gen_hir_capacity_gate
    c = CONFIGS[name]
    world, rank, dev = env.world, env.rank, env.dev
    T, d, h, E, k = (c[n] for n in ("tokens_per_gpu", "d_model", "d_hidden", "experts_per_gpu", "top_k"))
    g = torch.Generator().manual_seed(c["seed"])
    gate_w = torch.randn(E * world, d, generator=g) * c["gate_std"]
    gate_b = torch.zeros(E * world)
    gate_cls = NaiveGate
    saved_env = {n: os.environ.get(n) for n in ("FMOE_ENABLE_DYNREP", "FMOE_POLICY_CONSTANTS", "FMOE_ENABLE_FUSE")}
    if c.get("zipf"):
        gate_b = -c["zipf"] * torch.log(torch.arange(1, E * world + 1).float())
    if c.get("uniform_pairs"):
        gp = torch.Generator().manual_seed(c["seed"] * 7919 + rank)
        first = torch.randint(0, E * world, (T,), generator=gp)
        second = (first + torch.randint(1, max(E * world, 2), (T,), generator=gp)) % (E * world)
        pairs = torch.stack([first, second], dim=1)

        class UniformPairGate(NaiveGate):
            """Prescribed expert pairs; scores are the gate's logits of those experts."""

            def forward(self, inp):
                logits = self.gate(inp)
                return self.pairs, torch.gather(logits, 1, self.pairs)
        gate_cls = UniformPairGate
    if c.get("hot_share"):
        gate_b[0] = hot_bias_for_share(gate_w, 2 * c["hot_share"], c["seed"], d)
        os.environ["FMOE_ENABLE_DYNREP"], os.environ["FMOE_POLICY_CONSTANTS"] = "1", "reference"
        gate_cls = gen_hir_capacity_gate(rank, max(world // 2, 1), c["capacity"], spare_shadowed=(variant == "5b"))
    act = {"gelu": torch.nn.GELU(), "relu": torch.nn.ReLU()}[c["activation"]]
    os.environ["FMOE_ENABLE_FUSE"] = "1" if variant in ("fuse", "nccl") else "0"
    try:
        layer = FMoETransformerMLP(num_expert=E, d_model=d, d_hidden=h, world_size=world, top_k=k, activation=act,
                                   gate=gate_cls, bias=c["bias"])
    finally:
        for n, v in saved_env.items():
            if v is None:
                os.environ.pop(n, None)
            else:
                os.environ[n] = v
    with torch.no_grad():
        layer.gate.gate.weight.copy_(gate_w)
        layer.gate.gate.bias.copy_(gate_b)
    layer = layer.to(torch.bfloat16).to(dev)
    if c.get("uniform_pairs"):
        layer.gate.pairs = pairs.to(dev)
    with torch.no_grad():      # expert weights U(+-1/sqrt(fan_in)), generated on the device (seeded per rank)
        ge = torch.Generator(device=dev).manual_seed(c["seed"] * 1000 + rank)
        for lin, fan in ((layer.experts.htoh4, d), (layer.experts.h4toh, h)):
            lin.weight.copy_(((torch.rand(lin.weight.shape, generator=ge, device=dev) * 2 - 1) / fan ** 0.5))
            if lin.bias is not None:
                lin.bias.copy_(((torch.rand(lin.bias.shape, generator=ge, device=dev) * 2 - 1) / fan ** 0.5))
    gx = torch.Generator().manual_seed(c["seed"] + 17 * rank)
    x_host = torch.randn(T, d, generator=gx).to(torch.bfloat16).pin_memory()
    return layer, x_host


def make_steps(env, layer, x_host):
    """(step_resident, step_e2e): the device-resident step and the one whose batch starts in pinned host
    memory and whose loss is read back.  The copy of the NEXT step's batch is issued on a copy stream
    before this step's loss is read, so it travels while this step computes (what an input pipeline does)."""
    torch = env.torch
    dev = env.dev
    x_dev = x_host.to(dev).requires_grad_(True)

    def step_resident():
        layer.zero_grad(set_to_none=True)
        x_dev.grad = None
        out = layer(x_dev)
        out.sum().backward()

    # Four device staging buffers taken in turn (no allocation inside a step): the copy of batch i+1 runs on
    # the copy stream while step i computes, and waits until the step that last read its buffer is over.
    # The copy goes in as many parts as the layer signals quiet points (env.quiet: events that a replayed
    # step records after each of its scatters): a host-to-device copy beside a scatter's stores into peer
    # memory slowed those kernels by 80 % (measured), beside the GEMMs it costs nothing.
    copy_stream = torch.cuda.Stream(device=dev)
    stages = [torch.empty_like(x_dev.detach()) for _ in range(4)]
    pending = {"next": None, "i": 0, "last": None, "free": [None] * 4}

    def prefetch():
        slot = pending["i"] % 4
        pending["i"] += 1
        gates = list(getattr(env, "quiet", None) or [None])
        n_rows = x_host.shape[0]
        with torch.cuda.stream(copy_stream):
            if pending["free"][slot] is not None:
                copy_stream.wait_event(pending["free"][slot])
            # the window behind the forward's scatter (until the backward's) is about half as long as the one
            # behind the backward's (until the next step's): a third of the rows, then the rest
            cuts = [0, n_rows] if len(gates) == 1 else [0, n_rows // 3, n_rows]
            for part, gate in enumerate(gates[:len(cuts) - 1]):
                lo, hi = cuts[part], cuts[part + 1]
                if gate is not None:
                    copy_stream.wait_event(gate)
                stages[slot][lo:hi].copy_(x_host[lo:hi], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        return slot, ev

    def take():
        cur = torch.cuda.current_stream()
        if pending["last"] is not None:       # the step that read the previous buffer has been queued by now
            done = torch.cuda.Event()
            done.record(cur)
            pending["free"][pending["last"]] = done
        if pending["next"] is None:
            pending["next"] = prefetch()
        slot, ev = pending["next"]
        cur.wait_event(ev)
        pending["last"] = slot
        pending["next"] = prefetch()
        return stages[slot].detach()

    def step_e2e():
        layer.zero_grad(set_to_none=True)
        x = take().requires_grad_(True)
        out = layer(x)
        loss = out.sum(dtype=torch.float32)      # fp32 accumulation without an fp32 copy of the output
        loss.backward()
        return loss.item()

    return step_resident, step_e2e, take, x_dev


def exchange_form(layer, dev):
    from fastermoe_b200 import fmoe_cuda
    shadowing = not getattr(layer.policy_fn, "never_shadows", False)
    if layer.enable_fuse and (shadowing or os.environ.get("FMOE_B200_SMART", "peer") == "nccl"):
        return "smart schedule in the reference's shape (one NCCL group per pipeline step beside the step's expert GEMMs)"
    if fmoe_cuda.peer_slot_bytes(dev) > 0:
        sync = os.environ.get("FMOE_B200_NOSYNC", "1") == "0" or shadowing
        if sync:
            return "direct stores into peer memory over NVLink, host-planned (count table read back)"
        return ("direct stores into peer memory over NVLink, planned on the device (no host read of the counts); "
                "gathers stored by the GEMM epilogues, scatters form their rows on the way" +
                (" [selected by FMOE_ENABLE_FUSE=1]" if layer.enable_fuse else ""))
    return "NCCL send/receive, one pair per peer"


def graph_or_eager(env, layer, x_dev, step_resident, allow=True):
    """(callable that runs one resident step, description, GraphedStep or None): one CUDA graph replay per
    step where the step has no host read, else the eager step."""
    graphable = allow and (env.world == 1 or "planned on the device" in (exchange_form(layer, env.dev) or ""))
    if graphable:
        from fastermoe_b200 import GraphedStep
        graphed, why = None, ""
        try:
            graphed = GraphedStep(layer, x_dev.detach(), input_grad=True)
        except Exception as e:              # e.g. a receive pool too small for this workload's arena
            env.torch.cuda.synchronize()
            why = f"{type(e).__name__}: {str(e)[:120]}"
        # every rank replays or none does: a rank that launches eagerly beside ranks that replay would still
        # meet them in every exchange, but the legs would no longer measure one thing
        ok = env.torch.tensor([1 if graphed is not None else 0], device=env.dev)
        if env.world > 1:
            env.dist.all_reduce(ok, op=env.dist.ReduceOp.MIN)
        if int(ok.item()):
            return graphed.replay, "one CUDA graph replay per step (fastermoe_b200.GraphedStep)", graphed
        del graphed
        # ranks that captured may have waited in vain for the one that did not: start the eager legs clean
        from fastermoe_b200 import fmoe_cuda
        env.torch.cuda.synchronize()
        fmoe_cuda.lib.fmoe_device_status_clear()
        env.barrier()
        return step_resident, f"eager (graph capture failed on some rank{': ' + why if why else ''})", None
    return step_resident, "eager: every kernel launched from Python", None


def realised_rows(env, layer, x_dev):
    """The gate's decisions of all ranks in one step, as the count table [source rank, destination rank,
    expert] (int64, CPU), and the fraction of assignments that survived capacity pruning."""
    torch, dist = env.torch, env.dist
    seen = {}
    hook = layer.gate_hook
    layer.gate_hook = lambda idx, score, _x: seen.update(idx=idx.detach())
    with torch.no_grad():
        layer(x_dev.detach())
    layer.gate_hook = hook
    E, W = layer.num_expert, env.world
    flat = seen["idx"].reshape(-1)
    lec = torch.bincount(flat[flat >= 0], minlength=E * W)
    table = [torch.empty_like(lec) for _ in range(W)]
    if W > 1:
        dist.all_gather(table, lec)
    else:
        table = [lec]
    table = torch.stack(table).cpu().view(W, W, E)
    return table, float(table.sum()) / max(flat.numel() * W, 1)


def layer_roofline(env, name, table, ms_per_step):
    """Perfect-overlap bound of one step on the most-loaded GPU:
    max(12 B d h / P_tensor, HBM bytes / BW_hbm, NVLink bytes / BW_nvlink) / measured,
    B = rows routed to that GPU's experts (without shadowing; a shadowed expert's rows are computed
    where they originate, which only lowers B)."""
    c = CONFIGS[name]
    d, h, E = c["d_model"], c["d_hidden"], c["experts_per_gpu"]
    W = env.world
    per_pair = table.sum(2)                              # [src, dst] rows
    rows = per_pair.sum(0)                               # rows each GPU's experts process
    B = int(rows.max())
    t_tc = 12.0 * B * d * h / (env.peaks["bf16_tflops_sustained"] * 1e12)
    # activations: every [B,d] / [B,h] tensor written once by its producer and read once by each consumer
    # (x: fwd1 + wgrad1; hidden: fwd2 + wgrad2; derivative: dgrad2; y; dy: dgrad2 + wgrad2; dh: dgrad1 + wgrad1; dx);
    # weights read by the forward and input-gradient products, weight gradients written once
    hbm_bytes = 2.0 * ((3 + 1 + 3 + 1) * B * d + (3 + 2 + 3) * B * h) + 2.0 * 3 * 2 * E * d * h
    t_hbm = hbm_bytes / (env.peaks["hbm_gbs"] * 1e9)
    # four exchanges per step; each moves a GPU's remote rows in one direction and the peers' rows in the other
    remote_in = rows - per_pair.diagonal()
    remote_out = per_pair.sum(1) - per_pair.diagonal()
    worst = int(torch_max(remote_in, remote_out)) if W > 1 else 0
    t_nvl = 4.0 * worst * d * 2.0 / (NVLINK_GBS * 1e9)
    bound = max(t_tc, t_hbm, t_nvl)
    return {"busiest_gpu_rows": B, "t_tensor_ms": t_tc * 1e3, "t_hbm_ms": t_hbm * 1e3, "t_nvlink_ms": t_nvl * 1e3,
            "bound": "tensor" if bound == t_tc else ("hbm" if bound == t_hbm else "nvlink"),
            "frac": bound / (ms_per_step / 1e3),
            "peaks": "sustained cuBLAS bf16 and copy bandwidth (measured); NVLink 770 GB/s per direction (measured)"}


def torch_max(a, b):
    return max(int(a.max()), int(b.max()))


def measure_config(env, name, variant, steps, warmup):
    """One extra workload, timed on its own: tokens/s, ms/step, realised row histogram, roofline fraction."""
    import gc
    torch = env.torch
    from fastermoe_b200 import fmoe_cuda
    layer, x_host = build_layer(env, name, variant)
    step_resident, _, _, x_dev = make_steps(env, layer, x_host)
    old_smart = os.environ.get("FMOE_B200_SMART")
    if variant == "nccl":
        os.environ["FMOE_B200_SMART"] = "nccl"        # read by every forward
    try:
        return _measure_built(env, name, variant, steps, warmup, layer, x_host, step_resident, x_dev)
    finally:
        if old_smart is None:
            os.environ.pop("FMOE_B200_SMART", None)
        else:
            os.environ["FMOE_B200_SMART"] = old_smart


def _measure_built(env, name, variant, steps, warmup, layer, x_host, step_resident, x_dev):
    import gc
    torch = env.torch
    from fastermoe_b200 import fmoe_cuda
    for _ in range(max(warmup, 3)):
        step_resident()
    eager_ms = env.timed(step_resident, steps) / steps
    step, form, graphed = graph_or_eager(env, layer, x_dev, step_resident)
    if graphed is not None:
        for _ in range(3):
            step()
        ms = env.timed(step, steps) / steps
    else:
        ms = eager_ms
    del step, graphed
    table, kept = realised_rows(env, layer, x_dev)
    rows = table.sum(2).sum(0).tolist()
    status = fmoe_cuda.device_status(env.dev)
    if status:
        fmoe_cuda.lib.fmoe_device_status_clear()
    T = CONFIGS[name]["tokens_per_gpu"]
    res = {"config": name + (f" ({variant})" if variant else ""), "tokens_per_s": T * env.world / (ms / 1e3), "ms_per_step": ms,
           "step_form": form, "eager_ms_per_step": eager_ms,
           "steps": steps, "warmup": max(warmup, 3), "rows_per_gpu": rows, "kept_fraction_of_assignments": kept,
           "exchange": exchange_form(layer, env.dev) if env.world > 1 else None, "device_status": status,
           "roofline": layer_roofline(env, name, table, ms), "workload": workload_config(name, env.world)}
    if name == "c5":
        st = getattr(layer.gate, "last_stored", None)
        res["gate_policy_shadows_workers"] = st.any(1).nonzero().reshape(-1).tolist() if st is not None else None
        res["shadow_modules_in_use"] = sorted(layer._shadows.keys())
    del layer, x_host, x_dev, step_resident
    gc.collect()
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------- parity self-check

def parity_checks(env, layer, x_dev):
    """Untimed self-check of the multi-GPU path after the timed region.  Each entry is True or the text
    of the failure.  The small-shape checks are the bodies of the repository's own multi-GPU tests
    (tests/dist_worker.py), run here on this job's ranks; the two "step" checks use the benchmark's own
    layer and batch."""
    import numpy as np
    torch, dist = env.torch, env.dist
    from fastermoe_b200 import fmoe_cuda
    from oracle import moe_oracle as O
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import dist_worker
    res = {}
    # the oracle runs on the host: give every rank its share of the cores this process may use
    # (the launcher sets OMP_NUM_THREADS=1)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0)) // max(1, min(env.world, 4))))
    except (AttributeError, RuntimeError):
        pass

    def run(name, fn):
        try:
            t0 = time.time()
            fn()
            progress(env, f"  parity {name}: {time.time() - t0:.1f} s")
            ok = True
        except Exception as e:      # the message names the first mismatch
            ok = f"{type(e).__name__}: {str(e)[:300]}"
        flag = torch.tensor([1 if ok is True else 0], device=env.dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        res[name] = ok if ok is not True else (True if int(flag.item()) == 1 else "failed on another rank")

    E, W, k = layer.num_expert, env.world, layer.top_k

    def step_exchange():
        # the step's real routing: counts and positions against the oracle; scatter -> gather round trip
        # bit-exact; expert-side layout against the oracle's row map, with rows that carry (rank, row)
        with torch.no_grad():
            idx, _ = layer.gate(x_dev.detach())
        gate = idx.cpu().numpy()
        lec, off, pos, inv = fmoe_cuda.count_and_pos(idx.reshape(-1), E * W)
        assert np.array_equal(lec.cpu().numpy(), O.expert_count(gate, E * W))
        want_pos = O.assign_pos(gate, E * W)
        assert np.array_equal(pos.cpu().numpy()[:len(want_pos)], want_pos)
        A = idx.numel()
        cap = fmoe_cuda.nosync_capacity(A, x_dev.shape[1] * 2, W, env.dev)
        assert cap > 0, "the device-planned exchange is not available"
        plan = fmoe_cuda.peer_plan_exchange(lec, None, cap, E)
        lecs = [t.numpy() for t in plan.table.cpu().reshape(W, W * E)]
        none = np.zeros(W * E, bool)
        moves, total = O.scatter_moves(lecs, none, env.rank, E, W)
        tag = torch.zeros(A, 4, device=env.dev)            # 16-byte rows: (source rank, source row, 0, 0)
        tag[:, 0] = env.rank
        tag[:, 1] = torch.arange(A, device=env.dev)
        got = fmoe_cuda.peer_scatter_planned(tag, plan, cap)[:total].cpu()
        want = torch.zeros(total, 4)
        for (src, src_row, dst_row, n) in moves:
            want[dst_row:dst_row + n, 0] = src
            want[dst_row:dst_row + n, 1] = torch.arange(src_row, src_row + n)
        assert torch.equal(got, want), "expert-side layout of global_scatter"
        buf = fmoe_cuda.local_scatter(x_dev.detach(), pos, pos_div=k, n_rows=A)
        there = fmoe_cuda.peer_scatter_planned(buf, plan, cap)
        back = fmoe_cuda.peer_gather_planned(there, plan, A)
        assert torch.equal(back, buf), "global_gather(global_scatter(x)) != x"
        # the NCCL form moves the same rows to the same places
        own = plan.own_offsets.cpu()
        gec = np.ascontiguousarray(np.stack(lecs)[:, env.rank * E:(env.rank + 1) * E]).reshape(-1)
        nccl = fmoe_cuda.global_scatter(buf, torch.from_numpy(lecs[env.rank]), torch.from_numpy(gec),
                                        torch.from_numpy(none), int(own[-1]), W)
        assert torch.equal(nccl, there[:int(own[-1])]), "peer-memory and NCCL global_scatter differ"

    def step_layer_slice():
        # the benchmark's layer on 1024 tokens per rank: rank 0's output and input gradient against the
        # CPU oracle (fp32, the same bf16-rounded tensors, the device's gate decisions)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from parity import half_tol
        n = 1024
        xs = x_dev.detach()[:n].clone().requires_grad_(True)
        layer.zero_grad(set_to_none=True)
        with torch.no_grad():
            idx, _ = layer.gate(xs)
        out = layer(xs)
        out.sum().backward()
        parts = {}
        for pname, p in (("w1", layer.experts.htoh4.weight), ("b1", layer.experts.htoh4.bias),
                         ("w2", layer.experts.h4toh.weight), ("b2", layer.experts.h4toh.bias)):
            allp = [torch.empty_like(p.data) for _ in range(W)]
            dist.all_gather(allp, p.data.contiguous())
            if env.rank == 0:
                parts[pname] = torch.cat(allp).float().cpu()
        if env.rank == 0:
            want = O.moe_layer_fwd_bwd(xs.detach().float().cpu(), layer.gate.gate.weight.detach().float().cpu(),
                                       layer.gate.gate.bias.detach().float().cpu(), parts["w1"], parts["b1"], parts["w2"],
                                       parts["b2"], k, act=CFG["activation"], gate_idx=idx.cpu(), grads_for=("x",))
            torch.testing.assert_close(out.detach().float().cpu(), want["out"], **half_tol(want["out"], 4))
            torch.testing.assert_close(xs.grad.float().cpu(), want["grad_x"], **half_tol(want["grad_x"], 5))
        layer.zero_grad(set_to_none=True)

    run("step_routing_and_exchange_vs_oracle", step_exchange)
    run("step_layer_slice_vs_oracle", step_layer_slice)
    run("exchange_ops_vs_oracle", lambda: dist_worker.check_exchange(env.rank, W, env.dev))
    run("layer_fp32_fused_shadow_vs_oracle", lambda: dist_worker.check_layer(env.rank, W))
    run("layer_bf16_fused_shadow", lambda: dist_worker.check_layer_bf16(env.rank, W))
    run("shadow_policy_capacity_hirgate_vs_oracle", lambda: dist_worker.check_config5(env.rank, W))
    st = fmoe_cuda.device_status(env.dev)
    res["device_status_zero"] = True if st == 0 else f"status word {st}"
    if st:
        fmoe_cuda.lib.fmoe_device_status_clear()
    return res


# ------------------------------------------------------------------------------- main leg

def write_kernel_list(env, step, path, name, steps=3):
    """Every kernel of `steps` resident steps with its device time (CUPTI through torch.profiler: no
    replay, no clock control, usable on every rank of a multi-GPU run where a kernel profiler that
    serialises launches is not), written by rank 0 as a markdown table: launches per step, mean time,
    share of the summed kernel time, and the step's span on the device."""
    torch = env.torch
    from torch.profiler import profile, ProfilerActivity
    for _ in range(2):
        step()
    env.barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as tp:
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
    if env.rank != 0:
        return
    rows = [(e.key, e.count, e.device_time_total) for e in tp.key_averages() if e.device_time_total > 0]
    total = sum(r[2] for r in rows) or 1.0
    ev = [e for e in tp.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    span = (max(e.time_range.end for e in ev) - min(e.time_range.start for e in ev)) if ev else 0.0
    with open(path, "w") as f:
        f.write(f"kernel list of {steps} steps of {name} on rank 0 of {env.world} (torch.profiler, CUDA activities)\n\n")
        f.write(f"summed kernel time {total / steps:.1f} us per step; first kernel start to last kernel end "
                f"{span / steps:.1f} us per step (kernels on the side streams overlap the main stream)\n\n")
        f.write("| kernel | launches/step | mean us | share |\n|---|---|---|---|\n")
        for key, count, t in sorted(rows, key=lambda r: -r[2]):
            f.write(f"| {key[:110]} | {count / steps:g} | {t / count:.1f} | {100 * t / total:.1f} % |\n")


def progress(env, what):
    """Progress marker on stderr (rank 0): tells where a run that died was."""
    if env.rank == 0:
        print(f"[bench {time.strftime('%H:%M:%S')}] {what}", file=sys.stderr, flush=True)


def run_ours(args):
    import ctypes
    env = Env(args)
    torch, dist = env.torch, env.dist
    from fastermoe_b200 import fmoe_cuda
    world, rank, dev = env.world, env.rank, env.dev
    name = args.config
    c = CONFIGS[name]
    T, d, h, E, k = (c[n] for n in ("tokens_per_gpu", "d_model", "d_hidden", "experts_per_gpu", "top_k"))
    variant = {"c4": "fuse", "c5": "5b"}.get(name)
    layer, x_host = build_layer(env, name, variant)
    step_resident, step_e2e, take, x_dev = make_steps(env, layer, x_host)

    progress(env, "layer built; warm-up")
    for _ in range(max(args.warmup, 3)):
        step_resident()
    progress(env, "per-kernel timing pass")
    # Per-kernel timing pass: CUDA events around every library call on the launching stream, eager steps,
    # right after the warm-up (before the long legs below have brought the GPU to its power cap: the roofline's
    # denominator is the burst figure of a kernel timed alone).
    tprof = fmoe_cuda.Profile(timing=True)
    fmoe_cuda.set_profile(tprof)
    env.barrier()
    for _ in range(args.steps):
        step_resident()
    dur = tprof.durations_ms()
    fmoe_cuda.set_profile(None)
    # kernels of this library launched per step (counted on an eager step; a replayed graph runs the same ones)
    prof = fmoe_cuda.Profile()
    fmoe_cuda.set_profile(prof)
    step_resident()
    fmoe_cuda.set_profile(None)
    launches = prof.launches * args.steps
    # A step that never waits on the host (N = 1; N > 1 with the counts swapped through peer memory and the
    # plan built on the device) is replayed as ONE CUDA graph (fastermoe_b200.GraphedStep, the library's own
    # public wrapper): the GPU then sees the kernels back to back instead of at the pace of the Python glue.
    eager_ms = None
    if world > 1 and not args.eager:
        # quiet points of a replayed step: an external event after each of its two scatters (forward, backward),
        # recorded by the graph's own event nodes; the e2e leg's input copies start behind them
        from fastermoe_b200.functions import set_phase_hook
        env.quiet = [torch.cuda.Event(external=True), torch.cuda.Event(external=True)]
        seen = {"n": 0}

        def at_phase(phase):
            if phase == "scatter_done" and torch.cuda.is_current_stream_capturing():
                env.quiet[seen["n"] % 2].record()
                seen["n"] += 1
        set_phase_hook(at_phase)
    sampler = ClockSampler(env.local_rank) if rank == 0 else None
    if sampler:
        sampler.start()      # early: the tool takes longer to start than the timed region lasts
    progress(env, "graph capture")
    step, step_form, graphed = graph_or_eager(env, layer, x_dev, step_resident, allow=not args.eager)
    progress(env, f"timed region ({step_form[:24]})")
    if graphed is not None:
        for _ in range(3):
            step()
    t_region = time.time()
    total_ms = env.timed(step, args.steps)
    clocks = sampler.stop(t_region, time.time()) if sampler else None

    progress(env, "e2e legs")
    e2e_ms = e2e_eager_ms = h2d_alone_ms = None
    used_graph = False
    if not args.skip_e2e:
        # the batch's host-to-device copy on its own, all ranks copying at once: when this is close to the
        # e2e step time, the step is bound by the host link, not by the layer
        stage = torch.empty_like(x_dev.detach())
        h2d_alone_ms = env.timed(lambda: stage.copy_(x_host, non_blocking=True), 10) / 10
        del stage
        if graphed is None:
            for _ in range(2):
                step_e2e()
            e2e_eager_ms = e2e_ms = env.timed(step_e2e, args.steps)
        if graphed is not None:
            # per step one device-to-device copy of the prefetched batch into the captured input, one graph
            # launch, one read of the loss
            used_graph = True

            # The loss of every step is copied to pinned host memory on the stream and read by the host up to
            # two steps later, while the next steps already run: the host never leaves the GPU idle to fetch
            # a scalar (what a training loop that logs its loss does).
            lag = 2                      # steps the host may run ahead of the loss it reads
            loss_host = torch.zeros(lag + 1, dtype=torch.float32).pin_memory()
            loss_ready = [torch.cuda.Event() for _ in range(lag + 1)]
            state = {"i": 0, "read": 0, "losses": []}

            def read_until(n):
                while state["read"] < n:
                    slot = state["read"] % (lag + 1)
                    loss_ready[slot].synchronize()
                    state["losses"].append(float(loss_host[slot]))
                    state["read"] += 1

            def step_e2e_graph():
                loss = graphed(take())
                slot = state["i"] % (lag + 1)
                loss_host[slot:slot + 1].copy_(loss.detach().reshape(1), non_blocking=True)
                loss_ready[slot].record()
                state["i"] += 1
                read_until(state["i"] - lag)

            def read_last():
                read_until(state["i"])
                state["i"] = state["read"] = 0

            for _ in range(2):
                step_e2e_graph()
            read_last()
            state["losses"].clear()
            e2e_ms = env.timed(step_e2e_graph, args.steps, after=read_last)
            assert len(state["losses"]) == args.steps and all(math.isfinite(v) for v in state["losses"])
            if args.kernel_list_e2e:
                write_kernel_list(env, step_e2e_graph, args.kernel_list_e2e, f"{name} (e2e, graph replay)", steps=6)
                read_last()
                state["losses"].clear()
            layer.zero_grad(set_to_none=True)
            # for comparison, after the legs that count: the same e2e step launched from Python
            for _ in range(2):
                step_e2e()
            e2e_eager_ms = env.timed(step_e2e, args.steps)
    if getattr(env, "quiet", None):
        from fastermoe_b200.functions import set_phase_hook
        set_phase_hook(None)
        env.quiet_keep, env.quiet = env.quiet, None     # the captured graph refers to the events: keep them alive
    if graphed is not None:       # likewise the resident step launched from Python
        for _ in range(3):        # (the allocator hands out fresh blocks again after the graph legs)
            step_resident()
        eager_ms = env.timed(step_resident, args.steps)

    progress(env, "eager comparison legs done")
    if args.kernel_list:
        write_kernel_list(env, step, args.kernel_list, f"{name} ({step_form.split(':')[0].split(' (')[0]})")

    form = exchange_form(layer, dev) if world > 1 else None
    status = fmoe_cuda.device_status(dev)
    assert status == 0, f"device status word {status}: a bounded wait expired or a buffer overflowed"
    peaks = env.peaks
    ms_per_step = total_ms / args.steps
    tokens = T * world
    value = tokens / (ms_per_step / 1e3)
    e2e_val = tokens / (e2e_ms / args.steps / 1e3) if e2e_ms else None

    # Dominant kernel: the grouped expert GEMM forward (one launch per call).  Algorithmic
    # work per launch: 2 * rows * d_model * d_hidden flop with rows = tokens * top_k routed
    # to this GPU's experts (balanced routing: T*k).
    rows = T * k
    flops_per_launch = 2.0 * rows * d * h
    fwd = dur.get("linear_forward", [])
    bwd = dur.get("linear_backward", [])
    roofline = None
    if fwd:
        avg = sum(fwd) / len(fwd)
        ach = flops_per_launch / (avg / 1e3) / 1e12
        roofline = {"bound": "tensor", "kernel": "grouped expert GEMM forward (fmoe_linear_forward)",
                    "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": ach / peaks["bf16_tflops"], "peak_source": peaks["source"] + " burst cuBLAS bf16",
                    "avg_launch_ms": avg, "launches_timed": len(fwd),
                    # dram__bytes_read.sum + dram__bytes_write.sum per forward launch, mean of the two
                    # forward products of a step (690.0 MB and 490.9 MB), from the ncu capture summarised in
                    # profiles/grouped_gemm_config2_ncu_full.md; algorithmic bytes: 738 MB and 470 MB
                    "traffic": 590.5e6 if (world == 1 and name == "c2") else None, "traffic_unit": "bytes per launch"}
        if bwd:
            avg_b = sum(bwd) / len(bwd)
            roofline["backward_call"] = {"avg_ms": avg_b, "achieved": 2 * flops_per_launch / (avg_b / 1e3) / 1e12,
                                         "note": "one call = input-gradient + weight-gradient (+bias) products"}
    per_op = {n: {"calls_per_step": len(v) / args.steps, "avg_ms": sum(v) / len(v)} for n, v in dur.items()}
    layer_flops = 12.0 * rows * d * h
    layer_frac = layer_flops / (ms_per_step / 1e3) / 1e12 / peaks["bf16_tflops_sustained"]

    line = {
        "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "step_form": step_form,
        "eager_ms_per_step": (eager_ms / args.steps if eager_ms is not None else ms_per_step),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload_config(name, world), **({"exchange": form} if world > 1 else {})),
        "e2e": ({"value": e2e_val, "unit": "tokens/s",
                 "h2d_bytes_per_step": x_host.numel() * x_host.element_size(), "d2h_bytes_per_step": 4,
                 "note": "a training step: the batch is copied in, only the scalar loss is read back (the [T,d] "
                         "output and the gradients stay on the device)" +
                         ("; graphed steps: every step's loss is copied to pinned host memory and read by the host "
                          "while the next two steps run; eager steps: loss.item() each step" if used_graph else ""),
                 "ms_per_step": e2e_ms / args.steps, "cuda_graph": used_graph, "h2d_copy_alone_ms": h2d_alone_ms,
                 "eager_ms_per_step": e2e_eager_ms / args.steps} if e2e_ms else None),
        "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
        "layer_tensor_roofline_frac": layer_frac, "per_op_ms": per_op,
    }

    # Everything below is untimed and must not cost the headline: a watchdog prints the line as it
    # stands and ends the process if the extra legs do not finish in time.
    done = threading.Event()

    def emit():
        if rank == 0:
            print(json.dumps(line), flush=True)

    def watchdog():
        if not done.wait(args.extra_limit_s):
            line.setdefault("notes", []).append(f"extra legs did not finish within {args.extra_limit_s} s")
            emit()
            os._exit(0)
    threading.Thread(target=watchdog, daemon=True).start()

    try:
        if rank == 0 and world == 1 and not args.skip_cpu:
            cpu_val, cpu_ms, threads, kind = cpu_reference_run(3, 1, CPU_SAMPLE_TOKENS)
            line["cpu_baseline"] = {
                "value": cpu_val, "unit": "tokens/s", "cores": threads, "kind": kind,
                "sample": f"{CPU_SAMPLE_TOKENS} of {T} tokens, same experts and widths, fp32, 3 timed fwd+bwd steps "
                          f"({cpu_ms:.0f} ms each)"}
        if world > 1:
            progress(env, "row histogram and layer roofline")
            table_now, _ = realised_rows(env, layer, x_dev)
            line["rows_per_gpu"] = table_now.sum(2).sum(0).tolist()
            line["layer_roofline"] = layer_roofline(env, name, table_now, ms_per_step)
        if world > 1 and not args.no_parity and name == "c2":
            progress(env, "parity self-check")
            line["parity"] = parity_checks(env, layer, x_dev)
        extra = args.extra
        if extra is None:
            extra = "c3,c4,c5" if world == 8 else "none"
        if extra != "none" and world > 1:
            import gc
            del layer, step_resident, step_e2e, take, x_dev
            graphed = None
            gc.collect()
            torch.cuda.empty_cache()
            line["configs"] = []
            for item in extra.split(","):
                for variant in {"c4": ("fuse", "nccl"), "c5": ("5a", "5b")}.get(item, (None,)):
                    progress(env, f"extra workload {item} {variant or ''}")
                    try:
                        line["configs"].append(measure_config(env, item, variant, args.extra_steps, 3))
                    except Exception as e:
                        line["configs"].append({"config": f"{item} ({variant})", "error": f"{type(e).__name__}: {str(e)[:300]}"})
                        raise
    except Exception as e:
        line.setdefault("notes", []).append(f"extra legs stopped: {type(e).__name__}: {str(e)[:300]}")
        emit()
        done.set()
        os._exit(0)       # ranks may be out of step after a failed collective: do not wait for them
    done.set()
    emit()
    if world > 1:
        fmoe_cuda.destroy_comms()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS), help="workload of the main (timed) leg")
    ap.add_argument("--extra", default=None, help="other workloads to time after it: e.g. c3,c4,c5 or none "
                                                  "(default: all three at 8 GPUs, else none)")
    ap.add_argument("--extra-steps", type=int, default=10)
    ap.add_argument("--extra-limit-s", type=int, default=600, help="wall-clock limit of the untimed legs")
    ap.add_argument("--no-parity", action="store_true", help="omit the multi-GPU self-check")
    ap.add_argument("--kernel-list", default=None, metavar="PATH", help="also write a per-kernel device-time table "
                    "of three resident steps (rank 0) to PATH")
    ap.add_argument("--kernel-list-e2e", default=None, metavar="PATH", help="the same table for six e2e steps")
    ap.add_argument("--eager", action="store_true", help="time eager steps even where the step can replay as a CUDA graph")
    ap.add_argument("--skip-e2e", action="store_true", help="omit the host-buffer (e2e) leg (profiling runs)")
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
