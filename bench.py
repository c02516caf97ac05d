#!/usr/bin/env python
r"""MoE layer forward+backward throughput (tokens/s) on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1 runs BASELINE configuration 2: 16384 tokens, d_model 1024, d_hidden 4096,
16 experts, top-2, bf16 (fp32 accumulate), near-uniform softmax-free gate
(weight ~ N(0, 0.02)), GELU, seed 1.  N > 1 (launched with torch.distributed.run,
one rank per GPU) keeps that work per GPU and shards 16 experts per GPU over the
ranks (expert parallel, NCCL all-to-all-v), i.e. weak scaling.

One "step" = forward + backward (loss = sum of the output) of the layer on one
batch.  The printed JSON line carries: ``value`` (device-resident inputs),
``e2e`` (inputs copied from pinned host memory and the loss read back every
step), ``roofline`` of the dominant kernel (the grouped expert GEMM, timed with
CUDA events on the launching stream), ``cpu_baseline`` (the CPU port of the
reference's brute-force path on a bounded sample of the same workload).

``--impl reference`` times that CPU path alone on the host cores.
All data is synthetic (seeded); working set per step is several hundred MB,
larger than the 126 MB L2, so no explicit L2 flush is needed between steps.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(tokens_per_gpu=16384, d_model=1024, d_hidden=4096, experts_per_gpu=16, top_k=2, seed=1,
           gate_std=0.02, activation="gelu")
CPU_SAMPLE_TOKENS = 2048


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
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return None
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, mx = [], set(), None
        for r in self.rows:
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
                "samples": len(clocks)}


def cpu_reference_run(steps, warmup, tokens):
    """The reference's pure-PyTorch brute-force MoE (NaiveGate + per-expert matmuls, its
    tests/moe.py path) as restated by the oracle, fp32, all host threads, on `tokens`
    tokens of the benchmark workload.  Returns (tokens/s, ms/step, threads)."""
    import torch
    from oracle import moe_oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    E = CFG["experts_per_gpu"]
    tens = O.make_layer_inputs(tokens, CFG["d_model"], CFG["d_hidden"], E, seed=CFG["seed"], gate_std=CFG["gate_std"])
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.moe_layer_fwd_bwd(tens["x"], tens["gate_w"], tens["gate_b"], tens["w1"], tens["b1"], tens["w2"],
                            tens["b2"], CFG["top_k"], act=CFG["activation"])
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    return tokens / (ms / 1e3), ms, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 10))
    warm = max(1, min(args.warmup, 2))
    val, ms, threads = cpu_reference_run(steps, warm, CPU_SAMPLE_TOKENS)
    sample = (f"{CPU_SAMPLE_TOKENS} of {CFG['tokens_per_gpu']} tokens, same experts and widths, fp32 "
              f"(the reference has no bf16), {steps} timed fwd+bwd steps")
    print(json.dumps({
        "impl": "reference", "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(n_gpus):
    return {"workload": "BASELINE config 2 per GPU: MoE MLP layer fwd+bwd, expert-parallel over the GPUs",
            "tokens_per_gpu": CFG["tokens_per_gpu"], "d_model": CFG["d_model"], "d_hidden": CFG["d_hidden"],
            "experts_per_gpu": CFG["experts_per_gpu"], "top_k": CFG["top_k"], "activation": CFG["activation"],
            "gate": "NaiveGate, weight~N(0,0.02), raw top-k logits as scores", "seed": CFG["seed"],
            "parallelism": f"ep{n_gpus}", "l2": "inputs larger than L2 (no flush)"}


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


def run_ours(args):
    import torch
    import torch.distributed as dist
    from fastermoe_b200 import FMoETransformerMLP, fmoe_cuda

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # One process per GPU: run it (and allocate its pinned batch) on the CPUs next to its GPU, as a
        # launcher with NUMA binding would; otherwise the ranks' host-to-device copies cross sockets.
        bind_to_gpu_cpus(local_rank)
        dist.init_process_group("nccl", device_id=dev)

    T, d, h, E, k = (CFG[n] for n in ("tokens_per_gpu", "d_model", "d_hidden", "experts_per_gpu", "top_k"))
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(CFG["seed"])
    layer = FMoETransformerMLP(num_expert=E, d_model=d, d_hidden=h, world_size=world, top_k=k,
                               activation=torch.nn.GELU())
    with torch.no_grad():
        layer.gate.gate.weight.copy_(torch.randn(E * world, d, generator=g) * CFG["gate_std"])
        layer.gate.gate.bias.zero_()
        ge = torch.Generator().manual_seed(CFG["seed"] * 1000 + rank)
        for lin, fan in ((layer.experts.htoh4, d), (layer.experts.h4toh, h)):
            lin.weight.copy_((torch.rand(lin.weight.shape, generator=ge) * 2 - 1) / fan ** 0.5)
            lin.bias.copy_((torch.rand(lin.bias.shape, generator=ge) * 2 - 1) / fan ** 0.5)
    layer = layer.to(dtype).to(dev)
    gx = torch.Generator().manual_seed(CFG["seed"] + 17 * rank)
    x_host = torch.randn(T, d, generator=gx).to(dtype).pin_memory()
    x_dev = x_host.to(dev).requires_grad_(True)

    def step_resident():
        layer.zero_grad(set_to_none=True)
        x_dev.grad = None
        out = layer(x_dev)
        out.sum().backward()

    # End-to-end step: the batch starts in pinned host memory, the loss is read back.  The
    # copy of the NEXT step's batch is issued on a copy stream before this step's loss is
    # read, so it travels while this step computes (what an input pipeline does).
    copy_stream = torch.cuda.Stream(device=dev)

    def prefetch():
        with torch.cuda.stream(copy_stream):
            buf = x_host.to(dev, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        return buf, ev

    pending = {"next": None}

    def step_e2e():
        layer.zero_grad(set_to_none=True)
        if pending["next"] is None:
            pending["next"] = prefetch()
        x, ev = pending["next"]
        torch.cuda.current_stream().wait_event(ev)
        x.record_stream(torch.cuda.current_stream())
        x.requires_grad_(True)
        pending["next"] = prefetch()
        out = layer(x)
        loss = out.sum(dtype=torch.float32)      # fp32 accumulation without an fp32 copy of the output
        loss.backward()
        return loss.item()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step_resident()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    prof = fmoe_cuda.Profile()
    fmoe_cuda.set_profile(prof)
    total_ms = timed(step_resident, args.steps)
    fmoe_cuda.set_profile(None)
    clocks = sampler.stop() if sampler else None
    launches = prof.launches

    e2e_ms = e2e_eager_ms = None
    if not args.skip_e2e:
        for _ in range(2):
            step_e2e()
        e2e_eager_ms = e2e_ms = timed(step_e2e, args.steps)
        if world == 1:
            # The single-GPU step never waits on the host, so the whole forward+backward is replayed as
            # one CUDA graph (fastermoe_b200.GraphedStep): per step one device-to-device copy of the
            # prefetched batch into the captured input, one graph launch, one read of the loss.
            from fastermoe_b200 import GraphedStep
            graphed = GraphedStep(layer, x_dev.detach(), input_grad=True)

            def step_e2e_graph():
                if pending["next"] is None:
                    pending["next"] = prefetch()
                x, ev = pending["next"]
                torch.cuda.current_stream().wait_event(ev)
                x.record_stream(torch.cuda.current_stream())
                pending["next"] = prefetch()
                return graphed(x).item()

            for _ in range(2):
                step_e2e_graph()
            e2e_ms = timed(step_e2e_graph, args.steps)
            layer.zero_grad(set_to_none=True)

    # Per-kernel timing pass: CUDA events around every library call on the launching stream.
    tprof = fmoe_cuda.Profile(timing=True)
    fmoe_cuda.set_profile(tprof)
    barrier()
    for _ in range(args.steps):
        step_resident()
    dur = tprof.durations_ms()
    fmoe_cuda.set_profile(None)

    exchange_form = None
    if world > 1:
        exchange_form = ("smart schedule (NCCL, pipelined with the expert GEMMs)" if layer.enable_fuse else
                         "direct stores into peer memory over NVLink" if fmoe_cuda.peer_slot_bytes(dev) > 0 else
                         "NCCL send/receive, one pair per peer")
        st = ctypes.c_int32(0)
        fmoe_cuda.lib.fmoe_device_status(ctypes.byref(st))
        assert st.value == 0, f"device status word {st.value}: a bounded wait expired"
    peaks = measured_peaks()
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
                    "traffic": 590.5e6 if world == 1 else None, "traffic_unit": "bytes per launch"}
        if bwd:
            avg_b = sum(bwd) / len(bwd)
            roofline["backward_call"] = {"avg_ms": avg_b, "achieved": 2 * flops_per_launch / (avg_b / 1e3) / 1e12,
                                         "note": "one call = input-gradient + weight-gradient (+bias) products"}
    per_op = {name: {"calls_per_step": len(v) / args.steps, "avg_ms": sum(v) / len(v)} for name, v in dur.items()}
    layer_flops = 12.0 * rows * d * h
    layer_frac = layer_flops / (ms_per_step / 1e3) / 1e12 / peaks["bf16_tflops_sustained"]

    if rank == 0:
        cpu_val, cpu_ms, threads = (cpu_reference_run(3, 1, CPU_SAMPLE_TOKENS)
                                    if world == 1 and not args.skip_cpu else (None, None, None))
        line = {
            "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(workload_config(world), **({"exchange": exchange_form} if world > 1 else {})),
            "e2e": ({"value": e2e_val, "unit": "tokens/s",
                     "h2d_bytes_per_step": x_host.numel() * x_host.element_size(), "d2h_bytes_per_step": 4,
                     "ms_per_step": e2e_ms / args.steps, "cuda_graph": world == 1,
                     "eager_ms_per_step": e2e_eager_ms / args.steps} if e2e_ms else None),
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
            "layer_tensor_roofline_frac": layer_frac, "per_op_ms": per_op,
        }
        if cpu_val is not None:
            line["cpu_baseline"] = {
                "value": cpu_val, "unit": "tokens/s", "cores": threads, "kind": "port",
                "sample": f"{CPU_SAMPLE_TOKENS} of {T} tokens, same experts and widths, fp32, 3 timed fwd+bwd steps "
                          f"({cpu_ms:.0f} ms each)"}
        print(json.dumps(line))
    if world > 1:
        fmoe_cuda.destroy_comms()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-e2e", action="store_true", help="omit the host-buffer (e2e) leg (profiling runs)")
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
